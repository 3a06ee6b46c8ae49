// SpMM kernel for the dense-B operand form on PAIRS of SMs (thread-block clusters of two CTAs, tcgen05 cta_group::2).
//
// Same operand form and pipeline as vnm_spmm_dense_b.cu, but one B stage now feeds four 128-row tiles of A: the two
// CTAs of a cluster each hold two row tiles (two accumulators of 240 tensor-memory columns) and HALF of every B
// stage (32 rows x 120 of the 240 columns); one tcgen05.mma.sp.cta_group::2 multiplies 256 rows (128 from each CTA)
// with the 240 columns assembled from both halves.  Per k-tile a CTA therefore takes in 36 KiB of A and 32 KiB of B
// instead of 36 + 64 KiB, which moves the mainloop from the SM's L2 intake limit to the tensor pipe.
//
// Cluster protocol (rank 0 = leader, rank 1 = peer); every load stays local to the CTA that issues it:
//   * both CTAs run their own A producer, B producers and epilogue on their own shared / tensor memory;
//   * the peer forwards "my A blocks of k-tile it landed" and "my half of stage j landed" to the leader with remote
//     mbarrier arrivals on the leader's own a_full / b_full barriers (which expect two arrivals there: the leader's
//     loads and the peer's message), so the leader's sequencer and MMA issuer wait on one barrier per hand-off,
//     exactly as in the single-CTA kernel -- anything more on the issuing thread leaves the tensor pipe idle;
//   * only the leader issues tensor-core work: tcgen05.cp.cta_group::2 copies each CTA's metadata image into that
//     CTA's tensor memory, tcgen05.mma.sp.cta_group::2 reads A and B from both CTAs' shared memory;
//   * the leader's tcgen05.commit.cta_group::2 arrives on the stage-free / accumulator-full barriers of BOTH CTAs
//     (two commits: the local barrier and the peer's barrier through its shared::cluster address; a spare thread
//     forwarding the arrivals instead measured 1-2 % slower), and the peer's epilogue warps arrive remotely on the
//     leader's accumulator-empty barrier.
// No copy with cluster multicast is used anywhere.  Every wait is bounded (status bit, drain, return), and the two CTAs
// meet at a cluster barrier before tensor memory is freed, so neither leaves while the other may still touch it.
#include "vnm_internal.h"

namespace vnm {

namespace {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at B200 clocks

constexpr int RT = 2;            // row tiles (accumulators) per CTA; a pair tile has 2 * RT = 4 row tiles
constexpr int BN = 240;          // output columns per pair tile
constexpr int PART = 40;         // columns per epilogue part / TMA store
constexpr int SA = 3;            // A ring: k-tiles (each RT blocks)
constexpr int SB = 6;            // B ring: stages of 64 rows x 128 columns (this CTA's half of two K=32 blocks of the MMAs)
constexpr int SF = 12;           // stage "free" barriers (twice the stages, so that a late waiter never sees a wrapped phase)
constexpr int SR = 4;            // k-tile "ready" barriers
constexpr int META_SETS = 3;     // metadata column sets in tensor memory (4 columns per row tile each)
constexpr int KB_PER_STAGE = 2;                     // K=32 blocks per B stage: one 16 KiB TMA box (smaller boxes keep the copy engine less busy)
constexpr int STAGES_PER_KT = 4 / KB_PER_STAGE;
constexpr int B_CHUNK_BYTES = KB_PER_STAGE * 32 * 128;  // 64 rows x 64 columns
constexpr int B_STAGE_BYTES = 2 * B_CHUNK_BYTES;    // 16 KiB: two 64-column slices of which 120 columns are used (or 128 n-rows of 64 k)
constexpr int A_STAGE_BYTES = RT * AM_BLOCK_BYTES;  // 36 KiB
constexpr int A_RING_BYTES = SA * A_STAGE_BYTES;
constexpr int B_RING_BYTES = SB * B_STAGE_BYTES;
constexpr int OUT_STAGE_BYTES = TILE_M * PART * 2;  // 128 rows x 40 fp16 columns, staging of one TMA store
constexpr int OUT_RING_BYTES = RT * OUT_STAGE_BYTES;  // one staging buffer per accumulator
constexpr int BAR_BYTES = 640;
constexpr int SMEM_BYTES = A_RING_BYTES + B_RING_BYTES + OUT_RING_BYTES + BAR_BYTES + 1024;
static_assert(A_RING_BYTES % 1024 == 0 && B_RING_BYTES % 1024 == 0, "swizzled staging needs 1024-byte alignment");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
constexpr int NUM_THREADS = 512;  // warps 0-3 single-thread roles, 4-7 B producers, 8-15 epilogue (2 x 4 warps)
constexpr int EPI_WARP0 = 8;
constexpr int NBP = 3;            // B producer warps (SB % NBP == 0: a ring slot always has the same owner)
constexpr int TMEM_COLS = 512;
// tensor-memory columns: accumulator 0 at 0..239, metadata sets at 240 and 248, accumulator 1 at 256..495, metadata set at 496
__device__ __forceinline__ uint32_t acc_col(int rt) { return (uint32_t)rt * 256u; }
__device__ __forceinline__ uint32_t meta_col(int set) { return set == 0 ? 240u : (set == 1 ? 248u : 496u); }
static_assert(SB % NBP == 0 && NBP <= 4, "B producers");
constexpr int KT_RING = SB / STAGES_PER_KT;  // k-tiles the B ring holds
static_assert(SB % STAGES_PER_KT == 0 && KT_RING == SA && KT_RING == META_SETS && SF == 2 * SB, "the rings and the metadata sets advance one k-tile at a time");
static_assert(BN <= 240 && META_SETS == 3 && RT == 2 && BN % 16 == 0 && BN == 6 * PART, "tensor-memory column plan");
static_assert((SA + SB + SF + SR + 4) * 8 + 16 <= BAR_BYTES, "barrier area too small");
constexpr int HALF_N = BN / 2;   // columns of a B stage held by each CTA of the pair

__device__ __forceinline__ bool wait_one(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((it & 1023u) == 1023u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicOr(status, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void drain_slot(uint64_t *bar, uint32_t parity, int *status)
{
    const long long t0 = clock64();
    while (clock64() - t0 < WAIT_LIMIT_CYCLES / 4) {
        if (mbar_try_wait(bar, parity)) return;
    }
    atomicOr(status, DEV_TIMEOUT_DRAIN);
}

// ---- cluster helpers ----
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t saddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// ---- tcgen05, cta_group::2 forms ----
__device__ __forceinline__ void tmem_alloc2(uint32_t *smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrives on the barrier at shared::cluster address `bar_addr` once every tcgen05 operation issued so far by this thread
// has completed in both CTAs
__device__ __forceinline__ void tc_commit2(uint32_t bar_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// each CTA's shared-memory image (same offset in both) -> that CTA's tensor memory, 128 lanes x 128 bits
__device__ __forceinline__ void tc_cp2_128x128b(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// D[256 x N] (+)= A_sparse[256 x 32] * B[32 x N]: rows 0-127 / A / D / metadata of the leader, rows 128-255 of the peer;
// B columns 0..N/2-1 from the leader's shared memory, N/2..N-1 from the peer's
__device__ __forceinline__ void tc_mma2_sp_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t meta_tmem, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%3], %4, {%6, %6, %6, %6, %6, %6, %6, %6}, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(meta_tmem), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ bool wait_warp(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = wait_one(bar, parity, abort_flag, status, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Warp roles (512 threads per CTA, as in the single-CTA kernel):
//   warp 0      A producer: two bulk copies per k-tile (this CTA's two row tiles).
//   warp 1      leader: sequencer (waits for both CTAs' A blocks, copies both metadata images to tensor memory, waits
//               for the four B stages of the k-tile, then flips the k-tile's "ready" barrier);
//               peer: forwards "A blocks landed" to the leader.
//   warp 3      tensor-memory owner in both CTAs; leader: MMA issuer (one wait, eight MMAs and two commits per k-tile);
//               peer: forwards "B half landed" to the leader.
//   warps 4..6  B producers: one 16 KiB TMA box per stage (64 rows of this CTA's 128-column half).
//   warps 8..15 epilogue of this CTA's two accumulators.
template <int R>
__global__ void __launch_bounds__(NUM_THREADS, 1) spmm_dense_b_pair_kernel(const __grid_constant__ CUtensorMap tmap_tile, const __grid_constant__ CUtensorMap tmap_tile2,
                                                                           const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ OutMaps more_out,
                                                                           const SpmmParams p)
{
    static_assert(R == 1 || R == RT, "row tiles per CTA");  // R = 1: pair tiles of 256 x 240 for problems with few row tiles
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *a_ring = smem;
    uint8_t *b_ring = smem + A_RING_BYTES;
    uint8_t *out_ring = smem + A_RING_BYTES + B_RING_BYTES;
    uint64_t *a_full = reinterpret_cast<uint64_t *>(smem + A_RING_BYTES + B_RING_BYTES + OUT_RING_BYTES);
    uint64_t *b_full = a_full + SA;
    uint64_t *b_free = b_full + SB;   // b_free[j % SF]: the MMAs that read B stage j have completed (arrives in both CTAs)
    uint64_t *kready = b_free + SF;
    // accumulator hand-off.  R = 2: one barrier pair, both accumulators of a CTA belong to the same tile.  R = 1: a CTA has one
    // row tile, so its two accumulators alternate between consecutive tiles (barrier pair ti & 1) and the epilogue of one
    // tile runs beside the MMAs of the next.
    uint64_t *acc_full_bar = kready + SR;      // [2]
    uint64_t *acc_empty_bar = acc_full_bar + 2;  // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty_bar + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader_cta = crank == 0;
    const int pair = (int)blockIdx.x >> 1, npairs = (int)gridDim.x >> 1;
    // tiles of the pair: groups of 2 * R row tiles x column tiles, in the banded order of tile_coords()
    const int mquads = (p.mtiles + 2 * R - 1) / (2 * R);
    const int total_tiles = mquads * p.ntiles;
    const int my_tiles = (pair < total_tiles) ? (total_tiles - pair + npairs - 1) / npairs : 0;
    const int total_it = my_tiles * p.ktiles;

    if (threadIdx.x == 0) {
        // in the leader a slot is full once its own loads have landed AND the peer has reported the same for its half
        for (int s = 0; s < SA; s++) mbar_init(&a_full[s], leader_cta ? 2 : 1);
        for (int s = 0; s < SB; s++) mbar_init(&b_full[s], leader_cta ? 2 : 1);
        for (int s = 0; s < SF; s++) mbar_init(&b_free[s], 1);
        for (int s = 0; s < SR; s++) mbar_init(&kready[s], 2);  // metadata copied to tensor memory + all operands landed
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 2 * 4);  // R = 1: the four warps of one epilogue group in both CTAs
        }
        if (R == 2) mbar_init(&acc_empty_bar[0], 2 * 4 * R);  // every epilogue warp of both CTAs
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 3) {
        tmem_alloc2(tmem_slot, TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anyone arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // row tile of accumulator rt of this CTA in pair tile (mq, *)
    auto row_tile = [&](int mq, int rt) { return mq * 2 * R + (int)crank * R + rt; };

    if (warp == 0) {
        // ---------------- A producer ----------------
        setmaxnreg_dec<64>();
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int tile = pair; alive && tile < total_tiles; tile += npairs) {
                int mq, nt_unused;
                tile_coords(tile, mquads, p.ntiles, p.group_m, &mq, &nt_unused);
                for (int kt = 0; kt < p.ktiles; ++kt, ++it) {
                    const int s = it % SA;
                    if (it >= SA) {
                        const int jd = STAGES_PER_KT * (it - SA) + STAGES_PER_KT - 1;  // last B stage of the k-tile that used this slot
                        if (!wait_one(&b_free[jd % SF], (uint32_t)(jd / SF) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) { alive = false; break; }
                    }
                    mbar_arrive_expect_tx(&a_full[s], R * AM_BLOCK_BYTES);
#pragma unroll
                    for (int rt = 0; rt < R; rt++) {
                        // a row tile past the end of the matrix re-reads the last one; its rows are never stored
                        const int mt = row_tile(mq, rt) < p.mtiles ? row_tile(mq, rt) : p.mtiles - 1;
                        bulk_g2s_hint(a_ring + s * A_STAGE_BYTES + rt * AM_BLOCK_BYTES, p.am + ((size_t)mt * p.ktiles + kt) * AM_BLOCK_BYTES, AM_BLOCK_BYTES,
                                      &a_full[s], p.hint_a);
                    }
                    if (p.l2_ahead > 0) {
                        // the same blocks of a later k-tile (of this tile, or of the next one of this pair) on their way into L2
                        int kp = kt + p.l2_ahead, mqp = mq;
                        bool ok = true;
                        if (kp >= p.ktiles) {
                            kp -= p.ktiles;
                            ok = kp < p.ktiles && tile + npairs < total_tiles;
                            if (ok) tile_coords(tile + npairs, mquads, p.ntiles, p.group_m, &mqp, &nt_unused);
                        }
                        if (ok) {
#pragma unroll
                            for (int rt = 0; rt < R; rt++) {
                                const int mt = row_tile(mqp, rt) < p.mtiles ? row_tile(mqp, rt) : p.mtiles - 1;
                                bulk_prefetch_l2(p.am + ((size_t)mt * p.ktiles + kp) * AM_BLOCK_BYTES, AM_BLOCK_BYTES);
                            }
                        }
                    }
                }
            }
            if (*abort_flag) {
                for (int k = it > SA ? it - SA : 0; k < it; ++k) drain_slot(&a_full[k % SA], (uint32_t)(k / SA) & 1u, p.status);
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < EPI_WARP0) {
        // ---------------- B producers: warp 4 + w loads the stages j = w, w + NBP, ... of this CTA's half ----------------
        setmaxnreg_dec<64>();
        if (lane == 0 && warp - 4 < NBP) {
            tma_prefetch_desc(&tmap_tile);
            tma_prefetch_desc(&tmap_tile2);
            const int per_tile = STAGES_PER_KT * p.ktiles;
            int j = warp - 4;
            int tile_i = j / per_tile, jl = j - tile_i * per_tile;
            const int total_j = my_tiles * per_tile;
            for (; j < total_j; j += NBP) {
                const int tile = pair + tile_i * npairs;
                int mq_unused, nt;
                tile_coords(tile, mquads, p.ntiles, p.group_m, &mq_unused, &nt);
                const int n0 = nt * BN + (int)crank * HALF_N;  // first column of this CTA's half
                const int s = j % SB;
                if (j >= SB) {
                    const int jd = j - SB;
                    if (!wait_one(&b_free[jd % SF], (uint32_t)(jd / SF) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) break;
                }
                uint8_t *dst = b_ring + s * B_STAGE_BYTES;
                if (p.gather_mode == GATHER_NONE) {  // ablation: no loads of B at all (timing floor; results are meaningless)
                    mbar_arrive(&b_full[s]);
                    jl += NBP;
                    while (jl >= per_tile) { jl -= per_tile; ++tile_i; }
                    continue;
                }
                // 64 rows x 128 columns come along per stage; the MMAs read the first 120 columns
                mbar_arrive_expect_tx(&b_full[s], B_STAGE_BYTES);
                if (p.b_nk) {
                    tma_load_2d_hint(dst, &tmap_tile, jl * 64, n0, &b_full[s], p.hint_b);  // 128 rows (n) x 64 k, 128-byte swizzle
                } else if (p.b_wide_ok && n0 + 128 <= p.N) {
                    tma_load_4d_hint(dst, &tmap_tile, 0, jl * 64, 0, n0 / 8, &b_full[s], p.hint_b);  // {64 columns, 64 rows, 2 slices} from column n0
                } else {  // ragged right edge: two boxes that clip (and zero-fill) at N
                    for (int c = 0; c < 2; c++) tma_load_2d_hint(dst + c * B_CHUNK_BYTES, &tmap_tile2, n0 + c * 64, jl * 64, &b_full[s], p.hint_b);
                }
                if (p.l2_ahead > 0) {
                    // this warp's stage a few of its own turns later, on its way into L2
                    int jlp = jl + NBP * ((STAGES_PER_KT * p.l2_ahead + NBP - 1) / NBP), n0p = n0;
                    bool ok = true;
                    if (jlp >= per_tile) {
                        jlp -= per_tile;
                        ok = jlp < per_tile && tile + npairs < total_tiles;
                        if (ok) {
                            int ntp;
                            tile_coords(tile + npairs, mquads, p.ntiles, p.group_m, &mq_unused, &ntp);
                            n0p = ntp * BN + (int)crank * HALF_N;
                        }
                    }
                    if (ok) {
                        if (p.b_nk) tma_prefetch_2d(&tmap_tile, jlp * 64, n0p);
                        else if (p.b_wide_ok && n0p + 128 <= p.N) tma_prefetch_4d(&tmap_tile, 0, jlp * 64, 0, n0p / 8);
                        else for (int c = 0; c < 2; c++) tma_prefetch_2d(&tmap_tile2, n0p + c * 64, jlp * 64);
                    }
                }
                jl += NBP;
                while (jl >= per_tile) { jl -= per_tile; ++tile_i; }
            }
            if (*abort_flag && p.gather_mode != GATHER_NONE) {
                for (int k = j - NBP, n = 0; k >= 0 && n < SB / NBP; k -= NBP, ++n) drain_slot(&b_full[k % SB], (uint32_t)(k / SB) & 1u, p.status);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        setmaxnreg_dec<64>();
        if (lane == 0 && leader_cta) {
            // ---------------- sequencer (leader) ----------------
            const uint64_t mdesc0 = make_smem_desc(smem_u32(a_ring) + A_IMG_BYTES, 0, 128, 0);
            for (int it = 0; it < total_it; ++it) {
                const int sa = it % SA;
                if (it >= META_SETS) {  // column set it % META_SETS was last read by the MMAs of k-tile it - META_SETS
                    const int jd = STAGES_PER_KT * (it - META_SETS) + STAGES_PER_KT - 1;
                    if (!wait_one(&b_free[jd % SF], (uint32_t)(jd / SF) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                }
                if (!wait_one(&a_full[sa], (uint32_t)(it / SA) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;  // both CTAs' blocks
                tc_fence_after();
                const uint32_t mcol = tmem_base + meta_col(it % META_SETS);
#pragma unroll
                for (int rt = 0; rt < R; rt++)
                    tc_cp2_128x128b(mcol + rt * 4, mdesc0 + ((uint32_t)(sa * A_STAGE_BYTES + rt * AM_BLOCK_BYTES) >> 4));
                tc_commit2(smem_u32(&kready[it % SR]));  // first arrival: the metadata copies are done
                // The B stages of the k-tile are waited for here, not by the MMA issuer: every probe of a barrier
                // costs the issuing thread about as much as one MMA takes to execute, and the tensor pipe queues next to
                // nothing, so a wait between two MMAs is a bubble in the pipe.
                bool alive = true;
#pragma unroll
                for (int st = 0; st < STAGES_PER_KT; st++) {
                    const int j = STAGES_PER_KT * it + st;
                    if (!wait_one(&b_full[j % SB], (uint32_t)(j / SB) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }  // both halves
                }
                if (!alive) break;
                mbar_arrive(&kready[it % SR]);  // second arrival: every operand of the k-tile is in shared memory
            }
        } else if (lane == 0) {
            // ---------------- peer: forward "A blocks landed" ----------------
            const uint32_t remote0 = mapa_shared(smem_u32(a_full), 0);
            for (int it = 0; it < total_it; ++it) {
                const int sa = it % SA;
                if (!wait_one(&a_full[sa], (uint32_t)(it / SA) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                mbar_arrive_cluster(remote0 + sa * 8);
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        setmaxnreg_dec<64>();
        if (lane == 0 && leader_cta) {
            // ---------------- MMA issuer (leader) ----------------
            const bool b_nk = p.b_nk != 0;
            const uint32_t idesc0 = make_idesc_f16(2 * TILE_M, BN, true, 0u, !b_nk);
            const uint64_t adesc0 = make_smem_desc(smem_u32(a_ring), 16, 1024, 2);
            // this CTA's half of a stage: N-major (two 64-column slices of 64 rows x 128 bytes, 128-byte swizzle; a K=32 block is
            // 32 rows = 4096 bytes further) or K-major (128 n-rows of 128 bytes = 64 k of which 120 rows are used, 128-byte swizzle,
            // 8-row groups 1024 bytes apart; a K=32 block is 64 bytes further inside the row)
            const uint64_t bdesc0 = b_nk ? make_smem_desc(smem_u32(b_ring), 16, 1024, 2) : make_smem_desc(smem_u32(b_ring), B_CHUNK_BYTES, 1024, 2);
            const uint32_t kb_step = b_nk ? 64u : 32u * 128u;  // bytes between the K=32 blocks of a stage
            const uint32_t free_local = smem_u32(b_free), free_peer = mapa_shared(smem_u32(b_free), 1);
            const uint32_t full_local = smem_u32(acc_full_bar), full_peer = mapa_shared(smem_u32(acc_full_bar), 1);
            // The thread runs about one MMA ahead of the tensor pipe, so whatever it does between two MMAs must take less
            // than one MMA (about 140 clocks).  A k-tile is therefore one wait, eight MMAs and two commits, and the wait for
            // the NEXT k-tile sits in front of the last two MMAs, where the pipe still has work queued.
            int it = 0, slot = 0;  // slot = it % KT_RING
            bool alive = total_it > 0 && wait_one(&kready[0], 0u, abort_flag, p.status, DEV_TIMEOUT_MMA);
            tc_fence_after();
            for (int ti = 0; alive && ti < my_tiles; ++ti) {
                for (int kt = 0; alive && kt < p.ktiles; ++kt, ++it) {
                    // accumulator set of this tile: R = 2 always set 0 (phase ti), R = 1 set ti & 1 (phase ti / 2)
                    const int aset = R == 1 ? (ti & 1) : 0;
                    const uint32_t aphase = R == 1 ? (uint32_t)(ti >> 1) & 1u : (uint32_t)ti & 1u;
                    if (kt == 0) {
                        if (!wait_one(&acc_empty_bar[aset], aphase ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t mcol = tmem_base + meta_col(slot);
                    const uint32_t aoff = (uint32_t)(slot * A_STAGE_BYTES) >> 4;
                    const uint32_t boff0 = (uint32_t)(slot * STAGES_PER_KT * B_STAGE_BYTES) >> 4;
#pragma unroll
                    for (int kb = 0; kb < 4; kb++) {  // K=32 blocks of the k-tile, KB_PER_STAGE of them per B stage
                        if (kb == 3 && it + 1 < total_it) {
                            if (!wait_one(&kready[(it + 1) % SR], (uint32_t)((it + 1) / SR) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                            tc_fence_after();
                        }
                        const uint32_t boff = boff0 + (((uint32_t)(kb / KB_PER_STAGE) * B_STAGE_BYTES + (uint32_t)(kb % KB_PER_STAGE) * kb_step) >> 4);
#pragma unroll
                        for (int rt = 0; rt < R; rt++)
                            tc_mma2_sp_f16(tmem_base + acc_col(R == 1 ? aset : rt), adesc0 + aoff + (uint32_t)((rt * AM_BLOCK_BYTES + kb * 32) >> 4), bdesc0 + boff,
                                           mcol + rt * 4 + (uint32_t)(kb & ~1), idesc0 | (uint32_t)(kb & 1), (kt | kb) != 0 ? 1u : 0u);
                        if (kb % KB_PER_STAGE == KB_PER_STAGE - 1) {
                            // the stage (and, after the last, the A blocks and the metadata set) may be refilled in both CTAs
                            const int j = STAGES_PER_KT * it + kb / KB_PER_STAGE;
                            tc_commit2(free_local + (uint32_t)(j % SF) * 8u);
                            tc_commit2(free_peer + (uint32_t)(j % SF) * 8u);
                        }
                    }
                    if (!alive) break;
                    if (kt == p.ktiles - 1) {
                        tc_commit2(full_local + (uint32_t)aset * 8u);
                        tc_commit2(full_peer + (uint32_t)aset * 8u);
                    }
                    slot = slot + 1 == KT_RING ? 0 : slot + 1;
                }
            }
        } else if (lane == 0) {
            // ---------------- peer: forward "my half of stage j landed" ----------------
            const uint32_t remote0 = mapa_shared(smem_u32(b_full), 0);
            const int total_j = STAGES_PER_KT * total_it;
            for (int j = 0; j < total_j; ++j) {
                if (!wait_one(&b_full[j % SB], (uint32_t)(j / SB) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                mbar_arrive_cluster(remote0 + (uint32_t)(j % SB) * 8u);
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        setmaxnreg_dec<64>();  // idle warp of the first warpgroup
    } else {
        // ---------------- epilogue (both CTAs, own accumulators) ----------------
        setmaxnreg_inc<192>();
        const int q = warp & 3;
        const int i = q * 32 + lane;
        const int arow = mma_row_to_actual(i);
        const int grp = (warp - EPI_WARP0) >> 2;  // R = 2: the accumulator (row tile) this group drains; R = 1: the tiles ti with ti & 1 == grp
        const uint32_t empty_leader = mapa_shared(smem_u32(&acc_empty_bar[R == 1 ? grp : 0]), 0);
        int ti = 0;
        for (int tile = pair; tile < total_tiles; tile += npairs, ++ti) {
            if (R == 1 && (ti & 1) != grp) continue;
            int mq, nt;
            tile_coords(tile, mquads, p.ntiles, p.group_m, &mq, &nt);
            const int n0 = nt * BN;
            // the four warps of a group leave the loop together (they meet at named barriers below)
            const bool got = wait_warp(&acc_full_bar[R == 1 ? grp : 0], R == 1 ? (uint32_t)(ti >> 1) & 1u : (uint32_t)ti & 1u, abort_flag, p.status,
                                       DEV_TIMEOUT_EPILOGUE);
            if (!named_barrier_and(1 + grp, 128, got)) break;
            tc_fence_after();
            {
                const int rt = R == 1 ? 0 : grp;  // row tile of this CTA
                const int mt = row_tile(mq, rt);
                const int64_t row = (int64_t)mt * TILE_M + arow;
                const bool row_ok = mt < p.mtiles && row < p.M;
                const bool has_bias = p.layout == 1 && p.bias != nullptr;
                const __half bias = (has_bias && row_ok) ? p.bias[row] : __ushort_as_half((unsigned short)0);
                const bool leader = (warp == EPI_WARP0 + 4 * grp) && lane == 0;
                const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16) + acc_col(grp);
                // 40 accumulator columns of this thread's row -> 20 registers of packed halves
                auto drain = [&](int part, uint32_t *pk) {
                    uint32_t v0[32], v1[8];
                    tc_ld_32x32b_x32(trow + (uint32_t)(part * PART), v0);
                    tc_ld_32x32b_x8(trow + (uint32_t)(part * PART) + 32u, v1);
                    tc_wait_ld();
#pragma unroll
                    for (int jj = 0; jj < 16; jj++) {
                        __half2 h0 = __floats2half2_rn(__uint_as_float(v0[2 * jj]), __uint_as_float(v0[2 * jj + 1]));
                        pk[jj] = *reinterpret_cast<uint32_t *>(&h0);
                    }
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) {
                        __half2 h1 = __floats2half2_rn(__uint_as_float(v1[2 * jj]), __uint_as_float(v1[2 * jj + 1]));
                        pk[16 + jj] = *reinterpret_cast<uint32_t *>(&h1);
                    }
                };
                // one part -> staging buffer -> one TMA store (which clips at M and N).  In the CTA's last tile nothing hides the
                // stores behind later MMAs any more, and the operand rings are idle (every load has landed and every MMA that
                // read them has completed, or this tile's accumulator would not be full): each part then gets a buffer of its
                // own inside the rings, so no part waits for the previous store to release the staging buffer (final epilogue 9.6k ->
                // 6.5k clocks; laying the six parts side by side and storing the 128 x 240 image at once measured slower, 8.1k).
                const bool last_tile = ti == my_tiles - 1;
                static_assert(RT * (BN / PART) * OUT_STAGE_BYTES <= A_RING_BYTES + B_RING_BYTES, "the last tile's staging does not fit into the rings");
                auto store_part = [&](int part, const uint32_t *pk) {
                    const bool in_range = mt < p.mtiles && n0 + part * PART < p.N;
                    uint8_t *stg = last_tile ? a_ring + (size_t)(grp * (BN / PART) + part) * OUT_STAGE_BYTES : out_ring + grp * OUT_STAGE_BYTES;
                    if (!last_tile) {
                        if (leader) bulk_wait_group_read0();  // the previous store has finished reading the staging buffer
                        named_barrier_sync(1 + grp, 128);
                    }
                    if (p.layout == 0) {
#pragma unroll
                        for (int c = 0; c < PART / 8; c++)
                            *reinterpret_cast<uint4 *>(stg + arow * (PART * 2) + c * 16) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                    } else {
                        __half *col = reinterpret_cast<__half *>(stg) + arow;
#pragma unroll
                        for (int jj = 0; jj < PART / 2; jj++) {
                            uint32_t pw = pk[jj];
                            __half2 h = *reinterpret_cast<__half2 *>(&pw);
                            __half lo = __low2half(h), hi = __high2half(h);
                            if (has_bias) { lo = __hadd(lo, bias); hi = __hadd(hi, bias); }
                            col[(2 * jj) * TILE_M] = lo;
                            col[(2 * jj + 1) * TILE_M] = hi;
                        }
                    }
                    fence_proxy_async();
                    named_barrier_sync(1 + grp, 128);
                    if (leader && in_range) {
                        const int cx = p.layout == 0 ? n0 + part * PART : mt * TILE_M, cy = p.layout == 0 ? mt * TILE_M : n0 + part * PART;
                        tma_store_2d(&tmap_out, stg, cx, cy);
                        // further destinations of the same tile (the same rows of the peers' result buffers), one group with the first
                        for (int d = 1; d < p.n_out; d++) tma_store_2d(&more_out.m[d - 1], stg, cx, cy);
                        bulk_commit_group();
                    }
                };
                constexpr int NPARTS = BN / PART, HELD = 5;
#pragma unroll
                for (int part = 0; part < NPARTS - HELD; part++) {
                    uint32_t pk[PART / 2];
                    drain(part, pk);
                    store_part(part, pk);
                }
                uint32_t held[HELD * (PART / 2)];
#pragma unroll
                for (int h = 0; h < HELD; h++) drain(NPARTS - HELD + h, held + h * (PART / 2));
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(empty_leader);  // the leader's MMA issuer waits for both CTAs' epilogues
#pragma unroll
                for (int h = 0; h < HELD; h++) store_part(NPARTS - HELD + h, held + h * (PART / 2));
            }
        }
    }

    if (warp >= EPI_WARP0 && ((warp - EPI_WARP0) & 3) == 0 && lane == 0) bulk_wait_group_read0();  // this thread's TMA stores have read shared memory (their global writes complete with the grid)
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's shared and tensor memory stay alive until the leader's last MMA and commit are done
    if (warp == 3) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, TMEM_COLS);
    }
}

int g_pair_clusters = 0;  // co-resident clusters of two CTAs on this device (0 = not queried yet)

}  // namespace

cudaError_t spmm_dense_b_pair_init()
{
    cudaError_t e = cudaFuncSetAttribute(spmm_dense_b_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(spmm_dense_b_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)) != cudaSuccess) return e;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(sms & ~1), 1, 1);
    lc.blockDim = dim3(NUM_THREADS, 1, 1);
    lc.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, spmm_dense_b_pair_kernel<2>, &lc);
    if (e != cudaSuccess) { (void)cudaGetLastError(); clusters = 0; }
    g_pair_clusters = clusters;
    return cudaSuccess;
}

// Pair tiles are 512 x 240 (two row tiles per CTA) or, where that would leave SM pairs without a tile, 256 x 240 (one
// row tile per CTA: 34 KiB per CTA and k-tile, two alternating accumulators).  Returns false when the pair kernel should not be used for this problem
// (row tiles do not group evenly, too few tiles to occupy the clusters, or clusters unavailable): the caller then
// launches the single-CTA kernel.
bool spmm_dense_b_pair_config(int M, int N, int K, int max_ctas, int force_rows, SpmmConfig *cfg)
{
    if (g_pair_clusters <= 0) return false;
    const int mtiles = (M + TILE_M - 1) / TILE_M;
    (void)K;
    const long long ntiles = (N + BN - 1) / BN;
    int clusters = g_pair_clusters;
    if (max_ctas > 0 && max_ctas / 2 < clusters) clusters = max_ctas / 2;
    if (clusters < 1) return false;
    const long long t2 = (long long)(mtiles / (2 * RT)) * ntiles, t1 = (long long)(mtiles / 2) * ntiles;
    const bool ok2 = mtiles % (2 * RT) == 0 && t2 >= clusters;   // at least one full wave of 512-row tiles
    const bool ok1 = mtiles % 2 == 0 && 4 * t1 >= 3 * clusters;   // most SM pairs get a 256-row tile
    int rt = 0;
    if (force_rows == 1 && ok1) rt = 1;
    else if (force_rows == 2 && ok2) rt = RT;
    // 512-row tiles read every B stage once per 512 rows and win wherever they fill the SM pairs (measured at K = 1024 .. 12288,
    // although 256-row tiles alternate two accumulators and so run a tile's epilogue beside the next tile's MMAs)
    else if (ok2) rt = RT;
    else if (ok1) rt = 1;
    if (rt == 0) return false;
    const long long tiles = rt == RT ? t2 : t1;
    cfg->bn = BN;
    cfg->nb = 2 * rt;  // row tiles per pair tile
    cfg->stages = 2;
    cfg->smem_bytes = SMEM_BYTES;
    cfg->threads = NUM_THREADS;
    cfg->grid = 2 * (int)(tiles < clusters ? tiles : clusters);
    return true;
}

cudaError_t launch_spmm_dense_b_pair(const SpmmConfig &cfg, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_tile2, const CUtensorMap &tmap_out, const OutMaps &more_out,
                                     const SpmmParams &p, cudaStream_t stream)
{
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)cfg.grid, 1, 1);
    lc.blockDim = dim3(NUM_THREADS, 1, 1);
    lc.dynamicSmemBytes = SMEM_BYTES;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    if (cfg.nb == 2) return cudaLaunchKernelEx(&lc, spmm_dense_b_pair_kernel<1>, tmap_tile, tmap_tile2, tmap_out, more_out, p);
    return cudaLaunchKernelEx(&lc, spmm_dense_b_pair_kernel<2>, tmap_tile, tmap_tile2, tmap_out, more_out, p);
}

}  // namespace vnm
