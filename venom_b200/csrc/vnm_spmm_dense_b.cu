// SpMM kernel for the dense-B operand form (the V:2:m pattern re-expressed as 2:4 over all K columns).
//
// Here B is read as ordinary tiles that every row of A shares, so one CTA reuses a B stage for two
// 128-row tiles of A: a 256 x 240 output tile with two accumulators of 240 tensor-memory columns (240 is
// the widest N that leaves room for the metadata columns).  The mainloop runs at the rate at which an SM
// takes in data from L2 (about 64 bytes per clock), so the tile is as large as tensor memory allows: per
// k-tile (128 original columns of A = 128 rows of B) the CTA streams
//     2 x 18 KiB value + metadata blocks   and   4 x 16 KiB stages of B (32 rows x 256 columns, 240 used)
// = 100 KiB for eight 128 x 240 x 32 MMAs (152 clocks each), i.e. 53 KiB per 256 x 128 outputs.
//
// Warp roles (512 threads; the first two warpgroups give registers to the last two):
//   warp 0      A producer (one thread): two bulk copies per k-tile.
//   warp 1      sequencer (one thread): waits for the A blocks, copies both metadata images to tensor memory
//               and flips the k-tile's "ready" barrier.
//   warp 3      MMA issuer (one thread) and tensor-memory owner: per K=32 block one wait for its B stage, two
//               MMAs (one per row tile) and one commit that frees the stage.
//   warps 4..6  B producers (one thread each): stages are dealt round-robin; a stage is one 16 KiB TMA box (a 4-D
//               map {64 columns, K rows, 4 slices of 64 columns, start column / 16} gives the [slice][row][64
//               columns] layout in one instruction; for B given as [N, K] a 2-D box of 256 rows x 32 k).  One
//               thread issuing every TMA tile load keeps the copy engine about a third busy (measured).
//   warps 8..15 epilogue: four warps per accumulator read their rows into registers, hand the accumulator
//               back, and store six parts of 40 columns through shared memory with one TMA store each.
// Every wait is bounded: on expiry the kernel records a status bit, drains and returns.
#include "vnm_internal.h"

namespace vnm {

namespace {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at B200 clocks

constexpr int RT = 2;            // row tiles per CTA tile the shared-memory and tensor-memory plans are sized for; the kernel
                                 // template runs with R = 2, or R = 1 when the problem has too few tiles to fill the GPU otherwise
constexpr int BN = 240;          // output columns per CTA tile
constexpr int PART = 40;         // columns per epilogue part / TMA store
constexpr int SA = 3;            // A ring: k-tiles (each RT blocks)
constexpr int SB = 6;            // B ring: stages of 32 rows x 256 columns (one K=32 block of the MMAs)
constexpr int SF = 12;           // stage "free" barriers (more than stages, so that a late waiter never sees a wrapped phase)
constexpr int SR = 4;            // k-tile "ready" barriers
constexpr int META_SETS = 3;     // metadata column sets in tensor memory (4 columns per row tile each)
constexpr int B_CHUNK_BYTES = 32 * 128;            // 32 rows x 64 columns
constexpr int B_STAGE_BYTES = 4 * B_CHUNK_BYTES;    // 16 KiB: four 64-column slices, the last one used up to column 240 (or 240 rows of 32 k)
constexpr int A_STAGE_BYTES = RT * AM_BLOCK_BYTES;  // 36 KiB
constexpr int A_RING_BYTES = SA * A_STAGE_BYTES;
constexpr int B_RING_BYTES = SB * B_STAGE_BYTES;
constexpr int OUT_STAGE_BYTES = TILE_M * PART * 2;  // 128 rows x 40 fp16 columns, staging of one TMA store
constexpr int OUT_RING_BYTES = RT * OUT_STAGE_BYTES;  // one staging buffer per accumulator
constexpr int BAR_BYTES = 256;
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
static_assert(SF >= 4 * SA && SF >= 4 * META_SETS && SF >= 2 * SB && SF % SB == 0, "too few stage barriers: a waiter could miss a phase");
static_assert(BN <= 240 && META_SETS == 3 && RT == 2 && BN % 16 == 0 && BN == 6 * PART, "tensor-memory column plan");
static_assert((SA + SB + SF + SR + 2) * 8 + 16 <= BAR_BYTES, "barrier area too small");

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

__device__ __forceinline__ bool wait_warp(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = wait_one(bar, parity, abort_flag, status, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void drain_slot(uint64_t *bar, uint32_t parity, int *status)
{
    const long long t0 = clock64();
    while (clock64() - t0 < WAIT_LIMIT_CYCLES / 4) {
        if (mbar_try_wait(bar, parity)) return;
    }
    atomicOr(status, DEV_TIMEOUT_DRAIN);
}

template <int R>
__global__ void __launch_bounds__(NUM_THREADS, 1) spmm_dense_b_kernel(const __grid_constant__ CUtensorMap tmap_tile, const __grid_constant__ CUtensorMap tmap_tile2,
                                                                      const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ OutMaps more_out,
                                                                      const SpmmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *a_ring = smem;
    uint8_t *b_ring = smem + A_RING_BYTES;
    uint8_t *out_ring = smem + A_RING_BYTES + B_RING_BYTES;
    uint64_t *a_full = reinterpret_cast<uint64_t *>(smem + A_RING_BYTES + B_RING_BYTES + OUT_RING_BYTES);
    uint64_t *b_full = a_full + SA;
    uint64_t *b_free = b_full + SB;   // b_free[j % SF]: the MMAs that read B stage j (k-tile j / 4, K=32 block j % 4) have completed
    uint64_t *kready = b_free + SF;
    uint64_t *acc_full_bar = kready + SR;
    uint64_t *acc_empty_bar = acc_full_bar + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // tiles: pairs of row tiles x column tiles, in the banded order of tile_coords()
    static_assert(R == 1 || R == RT, "row tiles per CTA tile");
    const int mpairs = (p.mtiles + R - 1) / R;
    const int total_tiles = mpairs * p.ntiles;
    const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total_it = my_tiles * p.ktiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; s++) mbar_init(&a_full[s], 1);
        for (int s = 0; s < SB; s++) mbar_init(&b_full[s], 1);
        for (int s = 0; s < SF; s++) mbar_init(&b_free[s], 1);
        for (int s = 0; s < SR; s++) mbar_init(&kready[s], 1);  // A block landed and its metadata copied to tensor memory
        mbar_init(acc_full_bar, 1);
        mbar_init(acc_empty_bar, 4 * R);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 3) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Register re-allocation, first statement of every role: the eight epilogue warps hold a whole accumulator
    // row in registers (192 each), the other eight need few (64 each).
    if (warp == 0) {
        // ---------------- A producer ----------------
        setmaxnreg_dec<64>();
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x) {
                int mp, nt_unused;
                tile_coords(tile, mpairs, p.ntiles, p.group_m, &mp, &nt_unused);
                for (int kt = 0; kt < p.ktiles; ++kt, ++it) {
                    const int s = it % SA;
                    if (it >= SA) {
                        const int jd = 4 * (it - SA) + 3;  // last B stage of the k-tile that used this slot
                        if (!wait_one(&b_free[jd % SF], (uint32_t)(jd / SF) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) { alive = false; break; }
                    }
                    mbar_arrive_expect_tx(&a_full[s], R * AM_BLOCK_BYTES);
#pragma unroll
                    for (int rt = 0; rt < R; rt++) {
                        // a missing second row tile (odd number of row tiles) re-reads the first one; its rows are never stored
                        const int mt = (mp * R + rt < p.mtiles) ? mp * R + rt : mp * R;
                        bulk_g2s(a_ring + s * A_STAGE_BYTES + rt * AM_BLOCK_BYTES, p.am + ((size_t)mt * p.ktiles + kt) * AM_BLOCK_BYTES, AM_BLOCK_BYTES,
                                 &a_full[s]);
                    }
                }
            }
            if (*abort_flag) {
                for (int k = it > SA ? it - SA : 0; k < it; ++k) drain_slot(&a_full[k % SA], (uint32_t)(k / SA) & 1u, p.status);
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < EPI_WARP0) {
        // ---------------- B producers: warp 4 + w loads the stages j = w, w + NBP, ... (a ring slot always has the same owner) ----------------
        // One thread keeps the copy engine only about a third busy with TMA tile loads (measured), so the stages
        // are dealt to three threads, and a stage is a single 16 KiB box wherever the tensor map allows it.
        setmaxnreg_dec<64>();
        if (lane == 0 && warp - 4 < NBP) {
            tma_prefetch_desc(&tmap_tile);
            tma_prefetch_desc(&tmap_tile2);
            const int per_tile = 4 * p.ktiles;
            int j = warp - 4;
            int tile_i = j / per_tile, jl = j - tile_i * per_tile;
            const int total_j = my_tiles * per_tile;
            for (; j < total_j; j += NBP) {
                const int tile = (int)blockIdx.x + tile_i * (int)gridDim.x;
                int mp_unused, nt;
                tile_coords(tile, mpairs, p.ntiles, p.group_m, &mp_unused, &nt);
                const int n0 = nt * BN;
                const int s = j % SB;
                if (j >= SB) {
                    const int jd = j - SB;
                    if (!wait_one(&b_free[jd % SF], (uint32_t)(jd / SF) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) break;
                }
                uint8_t *dst = b_ring + s * B_STAGE_BYTES;
                if (p.gather_mode == GATHER_NONE) {
                    mbar_arrive(&b_full[s]);
                } else {
                    // columns n0 + 240 .. n0 + 255 of the next tile come along and are never read by the MMAs
                    mbar_arrive_expect_tx(&b_full[s], B_STAGE_BYTES);
                    if (p.b_nk) {
                        tma_load_2d(dst, &tmap_tile, jl * 32, n0, &b_full[s]);  // 256 rows (n) x 32 k, 64-byte swizzle
                    } else if (p.b_wide_ok && n0 + 256 <= p.N) {
                        tma_load_4d(dst, &tmap_tile, 0, jl * 32, 0, n0 / 16, &b_full[s]);  // {64 columns, 32 rows, 4 slices} from column n0
                    } else {  // ragged right edge: four boxes that clip (and zero-fill) at N
                        for (int c = 0; c < 4; c++) tma_load_2d(dst + c * B_CHUNK_BYTES, &tmap_tile2, n0 + c * 64, jl * 32, &b_full[s]);
                    }
                }
                jl += NBP;
                while (jl >= per_tile) { jl -= per_tile; ++tile_i; }
            }
            if (*abort_flag && p.gather_mode != GATHER_NONE) {
                // this thread's copies still in flight: the last SB / NBP stages it issued
                for (int k = j - NBP, n = 0; k >= 0 && n < SB / NBP; k -= NBP, ++n) drain_slot(&b_full[k % SB], (uint32_t)(k / SB) & 1u, p.status);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- sequencer ----------------
        setmaxnreg_dec<64>();
        if (lane == 0) {
            const uint64_t mdesc0 = make_smem_desc(smem_u32(a_ring) + A_IMG_BYTES, 0, 128, 0);
            bool alive = true;
            for (int it = 0; alive && it < total_it; ++it) {
                const int sa = it % SA;
                // column set it % META_SETS was last read by the MMAs of k-tile it - META_SETS
                if (it >= META_SETS) {
                    const int jd = 4 * (it - META_SETS) + 3;
                    if (!wait_one(&b_free[jd % SF], (uint32_t)(jd / SF) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                }
                if (!wait_one(&a_full[sa], (uint32_t)(it / SA) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                tc_fence_after();
                const uint32_t mcol = tmem_base + meta_col(it % META_SETS);
#pragma unroll
                for (int rt = 0; rt < R; rt++)
                    tc_cp_128x128b(mcol + rt * 4, mdesc0 + ((uint32_t)(sa * A_STAGE_BYTES + rt * AM_BLOCK_BYTES) >> 4));
                tc_commit(&kready[it % SR]);
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ---------------- MMA issuer ----------------
        setmaxnreg_dec<64>();
        if (lane == 0) {
            const bool b_nk = p.b_nk != 0;
            const uint32_t idesc0 = make_idesc_f16(TILE_M, BN, true, 0u, !b_nk);
            const uint64_t adesc0 = make_smem_desc(smem_u32(a_ring), 16, 1024, 2);
            // B stage = the 32 k of one MMA: N-major (four 64-column slices of 32 rows x 128 bytes, 128-byte swizzle)
            // or K-major (256 n-rows of 64 bytes of which 240 are used, 64-byte swizzle, 8-row groups 512 bytes apart)
            const uint64_t bdesc0 = b_nk ? make_smem_desc(smem_u32(b_ring), 16, 512, 4) : make_smem_desc(smem_u32(b_ring), B_CHUNK_BYTES, 1024, 2);
            int it = 0;
            bool alive = true;
            for (int ti = 0; alive && ti < my_tiles; ++ti) {
                for (int kt = 0; alive && kt < p.ktiles; ++kt, ++it) {
                    if (!wait_one(&kready[it % SR], (uint32_t)(it / SR) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                    tc_fence_after();
                    if (kt == 0) {
                        if (!wait_one(acc_empty_bar, ((uint32_t)ti & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t mcol = tmem_base + meta_col(it % META_SETS);
                    const uint32_t aoff = (uint32_t)((it % SA) * A_STAGE_BYTES) >> 4;
#pragma unroll
                    for (int kb = 0; kb < 4; kb++) {  // K=32 blocks of the k-tile, one B stage each
                        const int j = 4 * it + kb;
                        if (!wait_one(&b_full[j % SB], (uint32_t)(j / SB) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                        tc_fence_after();
                        const uint32_t boff = (uint32_t)((j % SB) * B_STAGE_BYTES) >> 4;
#pragma unroll
                        for (int rt = 0; rt < R; rt++)
                            tc_mma_sp_f16(tmem_base + acc_col(rt), adesc0 + aoff + (uint32_t)((rt * AM_BLOCK_BYTES + kb * 32) >> 4), bdesc0 + boff,
                                          mcol + rt * 4 + (uint32_t)(kb & ~1), idesc0 | (uint32_t)(kb & 1), (kt | kb) != 0 ? 1u : 0u, 0u, 0u, 0u, 0u);
                        tc_commit(&b_free[j % SF]);  // the stage (and, after the fourth, the A blocks and metadata set) may be refilled
                    }
                    if (!alive) break;
                    if (kt == p.ktiles - 1) tc_commit(acc_full_bar);
                }
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        setmaxnreg_dec<64>();  // idle warp of the first warpgroup
    } else {
        // ---------------- epilogue ----------------
        setmaxnreg_inc<192>();
        const int q = warp & 3;
        const int i = q * 32 + lane;
        const int arow = mma_row_to_actual(i);
        int ti = 0;
        // with one row tile per CTA tile the second group of four warps has no accumulator to drain
        for (int tile = ((warp - EPI_WARP0) >> 2) < R ? (int)blockIdx.x : total_tiles; tile < total_tiles; tile += gridDim.x, ++ti) {
            int mp, nt;
            tile_coords(tile, mpairs, p.ntiles, p.group_m, &mp, &nt);
            const int n0 = nt * BN;
            // the four warps of a group leave the loop together (they meet at named barriers below)
            const bool got = wait_warp(acc_full_bar, (uint32_t)ti & 1u, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE);
            if (!named_barrier_and(1 + ((warp - EPI_WARP0) >> 2), 128, got)) break;
            tc_fence_after();
            {
                const int rt = (warp - EPI_WARP0) >> 2;  // which accumulator this warp drains
                const int mt = mp * R + rt;
                const int64_t row = (int64_t)mt * TILE_M + arow;
                const bool row_ok = mt < p.mtiles && row < p.M;
                const bool has_bias = p.layout == 1 && p.bias != nullptr;
                const __half bias = (has_bias && row_ok) ? p.bias[row] : __ushort_as_half((unsigned short)0);
                uint8_t *stg = out_ring + rt * OUT_STAGE_BYTES;
                const bool leader = (warp == EPI_WARP0 + 4 * rt) && lane == 0;
                const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16) + acc_col(rt);
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
                // one part -> staging buffer -> one TMA store (which clips at M and N)
                auto store_part = [&](int part, const uint32_t *pk) {
                    const bool in_range = mt < p.mtiles && n0 + part * PART < p.N;
                    if (leader) bulk_wait_group_read0();  // the previous store has finished reading the staging buffer
                    named_barrier_sync(1 + rt, 128);
                    if (p.layout == 0) {
                        // [M,N] output: 128 rows (at their actual position) x 40 columns
#pragma unroll
                        for (int c = 0; c < PART / 8; c++)
                            *reinterpret_cast<uint4 *>(stg + arow * (PART * 2) + c * 16) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                    } else {
                        // [N,M] output (+ bias): the transposed part, 40 rows (n) x 128 columns (m); the 32 lanes
                        // of a warp write 32 m of one n
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
                    named_barrier_sync(1 + rt, 128);
                    if (leader && in_range) {
                        const int cx = p.layout == 0 ? n0 + part * PART : mt * TILE_M, cy = p.layout == 0 ? mt * TILE_M : n0 + part * PART;
                        tma_store_2d(&tmap_out, stg, cx, cy);
                        // further destinations of the same tile (the same rows of the peers' result buffers), one group with the first
                        for (int d = 1; d < p.n_out; d++) tma_store_2d(&more_out.m[d - 1], stg, cx, cy);
                        bulk_commit_group();
                    }
                };
                // The first parts go out one by one; the last HELD parts are all read into registers first, so the
                // MMA issuer gets the accumulator back before their staging and store work (the register file
                // does not hold the packed halves of all six).
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
                if (lane == 0) mbar_arrive(acc_empty_bar);
#pragma unroll
                for (int h = 0; h < HELD; h++) store_part(NPARTS - HELD + h, held + h * (PART / 2));
            }
        }
    }

    if (warp >= EPI_WARP0 && ((warp - EPI_WARP0) & 3) == 0 && lane == 0) bulk_wait_group_read0();  // this thread's TMA stores have read shared memory (their global writes complete with the grid)
    tc_fence_before();
    __syncthreads();
    if (warp == 3) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

int g_num_sms_db = 0;

// Self-test of the bounded waits: two threads wait, through the same wait_one as the product kernels and with the
// same limit, on a barrier that nothing ever signals.  The first to run out of time records its status bit and
// raises the abort flag; the other sees the flag and leaves.  The kernel then returns normally.
__global__ void wait_expiry_selftest_kernel(int *status)
{
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_word = 0;
        fence_barrier_init();
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) wait_one(&bar, 0u, &abort_word, status, DEV_TIMEOUT_EPILOGUE);
    __syncthreads();
}

}  // namespace

cudaError_t launch_wait_expiry_selftest(int *status, cudaStream_t stream)
{
    wait_expiry_selftest_kernel<<<1, 64, 0, stream>>>(status);
    return cudaGetLastError();
}

cudaError_t spmm_dense_b_init()
{
    cudaError_t e = cudaFuncSetAttribute(spmm_dense_b_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(spmm_dense_b_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)) != cudaSuccess) return e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    return cudaDeviceGetAttribute(&g_num_sms_db, cudaDevAttrMultiProcessorCount, dev);
}

void spmm_dense_b_config(int M, int N, int max_ctas, SpmmConfig *cfg)
{
    const int mtiles = (M + TILE_M - 1) / TILE_M;
    const long long ntiles = (N + BN - 1) / BN;
    int sms = g_num_sms_db > 0 ? g_num_sms_db : 148;
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    // Two row tiles per CTA tile take in 100 KiB per k-tile (about 1900 clocks), one takes in 82 KiB (about 1400) for
    // half the outputs: the single form only pays when the double form would leave most of the GPU idle.
    const long long t2 = (long long)((mtiles + 1) / 2) * ntiles, t1 = (long long)mtiles * ntiles;
    const long long cost2 = ((t2 + sms - 1) / sms) * 1900, cost1 = ((t1 + sms - 1) / sms) * 1400;
    const int rt = (mtiles >= 2 && cost1 < cost2) ? 1 : 2;
    const long long tiles = rt == 2 ? t2 : t1;
    cfg->bn = BN;
    cfg->nb = rt;  // row tiles per CTA tile
    cfg->stages = 1;
    cfg->smem_bytes = SMEM_BYTES;
    cfg->threads = NUM_THREADS;
    cfg->grid = (int)(tiles < sms ? tiles : sms);
}

cudaError_t launch_spmm_dense_b(const SpmmConfig &cfg, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_tile2, const CUtensorMap &tmap_out, const OutMaps &more_out,
                                const SpmmParams &p, cudaStream_t stream)
{
    if (cfg.nb == 1)
        spmm_dense_b_kernel<1><<<(unsigned)cfg.grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap_tile, tmap_tile2, tmap_out, more_out, p);
    else
        spmm_dense_b_kernel<2><<<(unsigned)cfg.grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap_tile, tmap_tile2, tmap_out, more_out, p);
    return cudaGetLastError();
}

}  // namespace vnm
