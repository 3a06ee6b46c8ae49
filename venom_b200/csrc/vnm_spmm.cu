// V:N:M SpMM for sm_100a: C[M,N] = A_vnm[M,K] * B[K,N], fp16 in, fp32 accumulate in tensor memory.
//
// Persistent kernel: one CTA per SM walks over 128 x BN output tiles (in the banded order of tile_coords(): the
// CTAs that run together share a few column panels of B and a band of row tiles of A that stays in L2).  The 128 rows of a tile hold NB = 128/V vector
// blocks; each block has its own column-loc, hence its own gathered rows of B.
//
// Two shared-memory rings feed the tensor core:
//   A ring  SA stages of 18 KiB: the value image (128 rows x 64 compressed columns, K-major,
//           128-byte swizzle) and the metadata image of one k-tile, one bulk copy each;
//   B ring  SB stages of 32 KiB: 64 gathered rows (16 groups) of B for each of the NB blocks, N-major,
//           128-byte swizzle, i.e. half a k-tile; two K=32 MMAs per block consume one stage.
// Warp roles:
//   warp 0            A producer (one elected lane).
//   warps 1..PB       B producers.  All of them take part in every B stage: one lane arms the barrier
//                     with the byte count and 64 / PB lanes of each warp issue one TMA gather4 load each
//                     (four absolute row numbers per instruction, precomputed by the prepare step);
//                     spreading the loads over many warps matters because a warp issues them one lane
//                     after the other.
//   warp PB+1         sequencer: per k-tile waits for the A block, copies the metadata image to tensor
//                     memory (tcgen05.cp) and waits for both B stages, then flips one "ready" barrier.
//   warp PB+2         tensor-memory allocation and MMA issue: one wait, 4 * NB tcgen05.mma.sp and one
//                     tcgen05.commit per k-tile; for NB > 1 each MMA runs on all 128 rows of the value
//                     tile with the output lanes of the other blocks disabled.
//   last eight warps  epilogue, two warps per tensor-memory lane quadrant, each draining half of the columns:
//                     tcgen05.ld -> packed fp16 registers, release the accumulator, store.  For [M,N] a warp's
//                     32 rows x 32 columns go through 2 KiB of its own shared memory so that every store
//                     instruction writes full sectors of eight rows; [N,M] with fused bias stores 2-byte elements.
//                     With few k-tiles per tile (high sparsity) the kernel is bound by this part: four warps
//                     storing 16 bytes per lane into 32 different rows took 1.3x longer.
// Producers run ahead into the next tile while the epilogue drains.  Every wait is bounded: on expiry
// the kernel records a status bit, drains and returns.
#include "vnm_internal.h"

namespace vnm {

namespace {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at B200 clocks

constexpr int BS_ROWS = 64;     // gathered rows per B stage
constexpr int BS_GROUPS = 16;   // groups per B stage

template <int BN, int NB, int SA, int SB, int PB>
struct Traits {
    static_assert(BN == 64 || BN == 128 || BN == 256, "tile N must be 64, 128 or 256");
    static_assert(NB == 1 || NB == 2 || NB == 4, "128 rows hold 1, 2 or 4 vector blocks");
    static constexpr int CH = BN / 64;                        // 64-column slices per block
    static constexpr int B_CHUNK_BYTES = BS_ROWS * 128;       // one slice: 64 rows x 128 B
    static constexpr int B_BLOCK_BYTES = CH * B_CHUNK_BYTES;  // gathered half k-tile of one block
    static constexpr int B_STAGE_BYTES = NB * B_BLOCK_BYTES;
    static constexpr int GATHERS = NB * BS_GROUPS * CH;       // gather4 instructions per B stage (always 64)
    static_assert(GATHERS % PB == 0 && GATHERS / PB <= 32 && NB * CH <= PB, "producer warp count does not divide the loads");
    static_assert(B_STAGE_BYTES % 1024 == 0 && AM_BLOCK_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static constexpr int ACC_COLS = BN;
    static constexpr int META_COLS = 8;  // two alternating sets of four columns
    static constexpr int TMEM_COLS = (BN + META_COLS <= 128) ? 128 : (BN + META_COLS <= 256) ? 256 : 512;
    static constexpr int A_RING_BYTES = SA * AM_BLOCK_BYTES;
    static constexpr int B_RING_BYTES = SB * B_STAGE_BYTES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int EPI_WARPS = 8;  // two per tensor-memory lane quadrant, each draining half of the columns
    static constexpr int OUT_STAGE_BYTES = EPI_WARPS * 32 * 64;  // per epilogue warp: 32 rows x 32 fp16 columns
    static constexpr int SMEM_BYTES = A_RING_BYTES + B_RING_BYTES + BAR_BYTES + OUT_STAGE_BYTES + 1024;  // + alignment slack
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
    static constexpr int SEQ_WARP = 1 + PB;      // sequencer: waits for the operands of a k-tile, copies its metadata
    static constexpr int MMA_WARP = 2 + PB;      // MMA issuer (and tensor-memory owner)
    static constexpr int NUM_WARPS = 3 + PB + EPI_WARPS;
    static constexpr int NUM_THREADS = NUM_WARPS * 32;
    static constexpr int SR = 4;                 // "k-tile ready" barriers (sequencer -> MMA issuer)
    static_assert((2 * (SA + SB) + 8) * 8 + 32 <= BAR_BYTES - 16, "barrier area too small");
    static constexpr int SP = 4;  // "k-tile done" barriers (one tcgen05.commit per k-tile releases its A stage and both B stages)
    static_assert(SP >= SA && 2 * SP >= SB + 1, "too few k-tile barriers: a waiter could miss a phase");
};

// Whole-warp bounded wait on an mbarrier phase; lane 0 polls.  Returns false if the wait expired or
// another role already aborted.
__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = 0;
        if (mbar_try_wait(bar, parity)) {
            ok = 1;
        } else {
            const long long t0 = clock64();
            for (uint32_t it = 0;; ++it) {
                if (mbar_try_wait(bar, parity)) { ok = 1; break; }
                if ((it & 63u) == 63u) {
                    if (*abort_flag) break;
                    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                        *abort_flag = 1;
                        atomicOr(status, code);
                        break;
                    }
                }
            }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

// Single-thread bounded wait (no warp convergence needed): the fast path is one try_wait.
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

// Bounded wait used only while draining after an abort: until the copies of one ring slot have landed.
__device__ __forceinline__ void drain_slot(uint64_t *bar, uint32_t parity, int *status)
{
    const long long t0 = clock64();
    while (clock64() - t0 < WAIT_LIMIT_CYCLES / 4) {
        if (mbar_try_wait(bar, parity)) return;
    }
    atomicOr(status, DEV_TIMEOUT_DRAIN);
}

template <int BN, int NB, int SA, int SB, int PB>
__global__ void __launch_bounds__(Traits<BN, NB, SA, SB, PB>::NUM_THREADS, 1)
    spmm_kernel(const __grid_constant__ CUtensorMap tmap_rows, const __grid_constant__ CUtensorMap tmap_tile, const __grid_constant__ CUtensorMap tmap_out,
                const __grid_constant__ OutMaps more_out, const SpmmParams p)
{
    using T = Traits<BN, NB, SA, SB, PB>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *a_ring = smem;
    uint8_t *b_ring = smem + T::A_RING_BYTES;
    uint64_t *a_full = reinterpret_cast<uint64_t *>(smem + T::A_RING_BYTES + T::B_RING_BYTES);
    uint8_t *out_stage = smem + T::A_RING_BYTES + T::B_RING_BYTES + T::BAR_BYTES;
    uint64_t *a_empty = a_full + SA;
    uint64_t *b_full = a_empty + SA;
    uint64_t *b_empty = b_full + SB;
    uint64_t *kdone = b_empty + SB;
    uint64_t *kready = kdone + T::SP;
    uint64_t *acc_full_bar = kready + T::SR;
    uint64_t *acc_empty_bar = acc_full_bar + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int gmode = p.gather_mode;
    const int bstages_per_tile = 2 * p.ktiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; s++) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
        // a B stage is complete after one arrival with a byte count (TMA modes) or after one deferred arrival of every
        // producer thread (per-thread 16-byte asynchronous copies)
        for (int s = 0; s < SB; s++) { mbar_init(&b_full[s], gmode == GATHER_CPASYNC ? PB * 32 + (p.hybrid_rows ? 1 : 0) : 1); mbar_init(&b_empty[s], 1); }
        for (int s = 0; s < T::SP; s++) mbar_init(&kdone[s], 1);
        for (int s = 0; s < T::SR; s++) mbar_init(&kready[s], 2);  // metadata copy done + operands landed
        mbar_init(acc_full_bar, 1);
        mbar_init(acc_empty_bar, T::EPI_WARPS);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == T::MMA_WARP) {
        tmem_alloc(tmem_slot, T::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- A producer (one thread) ----------------
        int it = 0;
        if (lane == 0) {
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < p.total_tiles; tile += gridDim.x) {
                int mt, nt_unused;
                tile_coords(tile, p.mtiles, p.ntiles, p.group_m, &mt, &nt_unused);
                for (int kt = 0; kt < p.ktiles; ++kt, ++it) {
                    const int s = it % SA;
                    if (it >= SA) {
                        // slot s was last used by k-tile it - SA: free once that k-tile's MMAs have completed
                        const int kd = it - SA;
                        if (!wait_one(&kdone[kd % T::SP], (uint32_t)(kd / T::SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) { alive = false; break; }
                    }
                    mbar_arrive_expect_tx(&a_full[s], AM_BLOCK_BYTES);
                    bulk_g2s(a_ring + s * AM_BLOCK_BYTES, p.am + ((size_t)mt * p.ktiles + kt) * AM_BLOCK_BYTES, AM_BLOCK_BYTES, &a_full[s]);
                }
            }
            if (*abort_flag) {
                for (int k = it > SA ? it - SA : 0; k < it; ++k) drain_slot(&a_full[k % SA], (uint32_t)(k / SA) & 1u, p.status);
            }
        }
        __syncwarp();
    } else if (warp <= PB) {
        // ---------------- B producers ----------------
        // Every producer warp takes part in every stage (GATHERS / PB of its lanes issue one load each),
        // so each lane meets the ring slots strictly in order and the phase parity stays unambiguous.
        // The row numbers of the next stage are fetched before waiting for the current slot.
        if (gmode == GATHER_CPASYNC) {
            // ---- per-thread 16-byte asynchronous copies driven by the row table, optionally beside TMA gathers ----
            // A stage holds NB blocks x 64 gathered rows x BN columns = 2048 pieces of 16 bytes.  The first HT rows of
            // every block (p.hybrid_rows: 0, 16, 32 or 48) are fetched by TMA tile::gather4 (four 128-byte row pieces per
            // instruction), the others by plain asynchronous copies: thread t copies the pieces (column piece t % CPR,
            // flattened row t / CPR + i * RPP), so a warp reads whole rows of B (512 contiguous bytes at BN = 256) and
            // writes them in the 128-byte-swizzled N-major operand layout.  Measured on B200 this path is SLOWER than the
            // TMA gather (which is therefore the default), alone and in every split: kept as an ablation.
            constexpr int NT = PB * 32;           // producer threads
            constexpr int CPR = BN / 8;           // 16-byte pieces per row of a block
            constexpr int RPP = NT / CPR;         // flattened rows covered by one pass of all threads
            constexpr int PASSES = NB * BS_ROWS / RPP;
            static_assert(NT % CPR == 0 && (NB * BS_ROWS) % RPP == 0 && PASSES >= 1, "producer threads do not tile a B stage");
            const int HT = p.hybrid_rows;         // rows per block and stage that go through TMA
            const int CR = BS_ROWS - HT;          // rows per block and stage that go through asynchronous copies
            const int t = (warp - 1) * 32 + lane;
            const int cc = t % CPR, fr0 = t / CPR;
            const int *rows_i32 = reinterpret_cast<const int *>(p.rows);
            const __half *Bg = p.B;
            // this thread's fixed share of a stage, worked out once: block, row inside the block, shared-memory offset
            int blk[PASSES], rsel[PASSES];
            uint32_t doff[PASSES];
            int passes = 0;
#pragma unroll
            for (int i = 0; i < PASSES; i++) {
                const int fr = fr0 + i * RPP;
                blk[i] = 0; rsel[i] = 0; doff[i] = 0;
                if (fr < NB * CR) {
                    const int b = fr / CR, r = HT + fr % CR;
                    blk[i] = b; rsel[i] = r;
                    doff[i] = (uint32_t)(b * T::B_BLOCK_BYTES + (cc >> 3) * T::B_CHUNK_BYTES + r * 128 + (((cc & 7) ^ (r & 7)) << 4));
                    passes = i + 1;
                }
            }
            // TMA share: HT gather4 instructions per stage (NB blocks x HT / 4 groups x CH slices), HT / PB per warp
            const int tma_per_warp = HT / PB;
            const bool tma_lane = lane < tma_per_warp;
            const int gidx = lane * PB + (warp - 1);
            const int gper_block = (HT / 4) * T::CH;
            const int gb = gper_block ? gidx / gper_block : 0, gg = gper_block ? (gidx % gper_block) / T::CH : 0, gc = gidx % T::CH;
            const bool leader = t == 0;
            if (leader && HT) tma_prefetch_desc(&tmap_rows);
            int rcur[PASSES], rnxt[PASSES];
            int4 gcur = make_int4(0, 0, 0, 0), gnxt = make_int4(0, 0, 0, 0);
            auto load_rows = [&](int tl, int l, int(&dst)[PASSES], int4 &g4) {
                int mt, nt_unused;
                tile_coords(tl, p.mtiles, p.ntiles, p.group_m, &mt, &nt_unused);
#pragma unroll
                for (int i = 0; i < PASSES; i++)
                    if (i < passes) dst[i] = __ldg(rows_i32 + ((size_t)(mt * NB + blk[i]) * p.ktiles * KT_GROUPS) * 4 + (size_t)l * BS_ROWS + rsel[i]);
                if (tma_lane) g4 = __ldg(p.rows + ((size_t)(mt * NB + gb) * p.ktiles) * KT_GROUPS + (size_t)l * BS_GROUPS + gg);
            };
            int j = 0, tile = blockIdx.x, jl = 0;
            bool valid = tile < p.total_tiles;
            if (valid) load_rows(tile, jl, rcur, gcur);
            while (valid) {
                int ntile = tile, njl = jl + 1;
                if (njl == bstages_per_tile) { njl = 0; ntile += gridDim.x; }
                const bool nvalid = ntile < p.total_tiles;
                if (nvalid) load_rows(ntile, njl, rnxt, gnxt);
                const int s = j % SB;
                if (j >= SB) {
                    const int kd = (j - SB) >> 1;  // slot s was last used by stage j - SB, a half of k-tile (j - SB) / 2
                    // one lane per warp polls: hundreds of threads spinning on a barrier slow the other roles' polls down
                    if (!wait_bounded(&kdone[kd % T::SP], (uint32_t)(kd / T::SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) break;
                }
                uint8_t *stp = b_ring + s * T::B_STAGE_BYTES;
                const uint32_t st = smem_u32(stp);
                int mt_unused, nt_cur;
                tile_coords(tile, p.mtiles, p.ntiles, p.group_m, &mt_unused, &nt_cur);
                const int n0 = nt_cur * BN;
                if (HT) {
                    if (leader) mbar_arrive_expect_tx(&b_full[s], (uint32_t)(HT * 512));  // NB * BN = 256 columns of HT rows
                    if (tma_lane) tma_gather4(stp + gb * T::B_BLOCK_BYTES + gc * T::B_CHUNK_BYTES + gg * 512, &tmap_rows, n0 + gc * 64, gcur, &b_full[s]);
                }
                const int col = n0 + cc * 8;
                const bool col_ok = col < p.N;  // N % 8 == 0: a piece lies entirely inside or outside
#pragma unroll
                for (int i = 0; i < PASSES; i++) {
                    if (i < passes) {
                        const int row = rcur[i];
                        const bool ok = col_ok && row < p.K;  // padding rows (row == K) and columns past N read as zeros
                        const __half *src = ok ? Bg + (size_t)row * p.ldb + col : Bg;
                        cp_async_16_zfill(st + doff[i], src, ok ? 16u : 0u);
                    }
                }
                cp_async_mbar_arrive_noinc(&b_full[s]);  // arrives once this thread's copies have landed
#pragma unroll
                for (int i = 0; i < PASSES; i++) rcur[i] = rnxt[i];
                gcur = gnxt;
                tile = ntile; jl = njl; valid = nvalid; ++j;
            }
            cp_async_wait_all();  // nothing of this thread is in flight when the CTA leaves (also on the abort path)
            if (*abort_flag && leader && HT) {
                for (int k = j > SB ? j - SB : 0; k < j; ++k) drain_slot(&b_full[k % SB], (uint32_t)(k / SB) & 1u, p.status);
            }
            __syncwarp();
        } else {
        const int pw = warp - 1;
        constexpr int ACTIVE = T::GATHERS / PB;  // lanes of this warp that issue gather4 loads
        const bool leader = (pw == 0 && lane == 0);
        if (leader) { tma_prefetch_desc(&tmap_rows); tma_prefetch_desc(&tmap_tile); }
        // this lane's fixed share of a stage: block b, group g, 64-column slice c
        const int idx = lane * PB + pw;
        const int gb = idx / (BS_GROUPS * T::CH);
        const int gg = (idx % (BS_GROUPS * T::CH)) / T::CH;
        const int gc = idx % T::CH;
        const bool gather_lane = (gmode == GATHER_TMA4) && lane < ACTIVE;
        const bool tile_lane = (gmode == GATHER_CONTIG) && lane == 0 && pw < NB * T::CH;
        const int tb = pw / T::CH, tc = pw % T::CH;  // CONTIG: (block, slice) of this warp
        if (gather_lane || tile_lane || leader) {
            int j = 0;
            int tile = blockIdx.x, jl = 0;
            bool valid = tile < p.total_tiles;
            auto rows_of = [&](int tl, int l) -> const int4 * {
                int mt, nt_unused;
                tile_coords(tl, p.mtiles, p.ntiles, p.group_m, &mt, &nt_unused);
                const int b = gather_lane ? gb : tb;
                return p.rows + ((size_t)(mt * NB + b) * p.ktiles) * KT_GROUPS + (size_t)l * BS_GROUPS + (gather_lane ? gg : 0);
            };
            int4 r_cur = make_int4(0, 0, 0, 0);
            if (valid && (gather_lane || tile_lane)) r_cur = __ldg(rows_of(tile, jl));
            while (valid) {
                int ntile = tile, njl = jl + 1;
                if (njl == bstages_per_tile) { njl = 0; ntile += gridDim.x; }
                const bool nvalid = ntile < p.total_tiles;
                int4 r_nxt = make_int4(0, 0, 0, 0);
                if (nvalid && (gather_lane || tile_lane)) r_nxt = __ldg(rows_of(ntile, njl));
                const int s = j % SB;
                if (j >= SB) {
                    // slot s was last used by stage j - SB, the half of k-tile (j - SB) / 2
                    const int kd = (j - SB) >> 1;
                    if (!wait_one(&kdone[kd % T::SP], (uint32_t)(kd / T::SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) break;
                }
                uint8_t *st = b_ring + s * T::B_STAGE_BYTES;
                int mt_unused, nt_cur;
                tile_coords(tile, p.mtiles, p.ntiles, p.group_m, &mt_unused, &nt_cur);
                const int n0 = nt_cur * BN;
                if (leader) {
                    if (gmode == GATHER_NONE) mbar_arrive(&b_full[s]);
                    else mbar_arrive_expect_tx(&b_full[s], T::B_STAGE_BYTES);
                }
                if (gather_lane)
                    tma_gather4(st + gb * T::B_BLOCK_BYTES + gc * T::B_CHUNK_BYTES + gg * 512, &tmap_rows, n0 + gc * 64, r_cur, &b_full[s]);
                else if (tile_lane)  // 64 consecutive rows starting at the first selected row of the stage
                    tma_load_2d(st + tb * T::B_BLOCK_BYTES + tc * T::B_CHUNK_BYTES, &tmap_tile, n0 + tc * 64, r_cur.x, &b_full[s]);
                tile = ntile; jl = njl; valid = nvalid; r_cur = r_nxt; ++j;
            }
            if (*abort_flag && leader && gmode != GATHER_NONE) {
                for (int k = j > SB ? j - SB : 0; k < j; ++k) drain_slot(&b_full[k % SB], (uint32_t)(k / SB) & 1u, p.status);
            }
        }
        __syncwarp();
        }
    } else if (warp == T::SEQ_WARP) {
        // ---------------- sequencer (one thread) ----------------
        // Takes every wait except one off the MMA issuer: per k-tile it waits for the value/metadata block,
        // copies the metadata image to tensor memory (its own tcgen05.cp, tracked by a tcgen05.commit that
        // arrives on the k-tile's "ready" barrier), waits for both B stages and arrives on the same barrier.
        if (lane == 0) {
            const uint32_t meta0 = tmem_base + T::ACC_COLS;
            const uint64_t mdesc0 = make_smem_desc(smem_u32(a_ring) + A_IMG_BYTES, 0, 128, 0);
            const int my_tiles = (p.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
            const int total_it = my_tiles * p.ktiles;
            bool alive = true;
            for (int it = 0; alive && it < total_it; ++it) {
                const int sa = it % SA;
                // the column set it & 1 was last read by the MMAs of k-tile it - 2
                if (it >= 2 && !wait_one(&kdone[(it - 2) % T::SP], (uint32_t)((it - 2) / T::SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                if (!wait_one(&a_full[sa], (uint32_t)(it / SA) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                tc_fence_after();
                // metadata image: 128 rows x 16 bytes, 8-row core matrices stored back to back
                tc_cp_128x128b(meta0 + (uint32_t)(it & 1) * 4u, mdesc0 + ((uint32_t)(sa * AM_BLOCK_BYTES) >> 4));
                tc_commit(&kready[it % T::SR]);
                for (int h = 0; h < 2; ++h) {
                    const int j = 2 * it + h;
                    if (!wait_one(&b_full[j % SB], (uint32_t)(j / SB) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                }
                if (alive) {
                    fence_proxy_async();  // stages written by per-thread asynchronous copies are read by the tensor core's proxy
                    mbar_arrive(&kready[it % T::SR]);
                }
            }
        }
        __syncwarp();
    } else if (warp == T::MMA_WARP) {
        // ---------------- MMA issuer (one thread) ----------------
        // One wait per k-tile (its "ready" barrier), 4 * NB MMAs, one tcgen05.commit that releases the
        // k-tile's A stage and both of its B stages.  Anything else on this thread would sit between two
        // MMAs: the tensor pipe accepts them nearly one at a time, so issue-side work is not hidden.
        if (lane == 0) {
            const uint32_t acc = tmem_base;
            const uint32_t meta0 = tmem_base + T::ACC_COLS;
            const uint32_t idesc0 = make_idesc_f16(TILE_M, BN, true, 0u, true);
            // descriptor templates: only the start-address field (low 14 bits, in 16-byte units) varies
            const uint64_t adesc0 = make_smem_desc(smem_u32(a_ring), 16, 1024, 2);
            const uint64_t bdesc0 = make_smem_desc(smem_u32(b_ring), T::B_CHUNK_BYTES, 1024, 2);
            const int my_tiles = (p.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
            int it = 0;
            bool alive = true;
            for (int ti = 0; alive && ti < my_tiles; ++ti) {
                // the epilogue must have read the previous tile's accumulator
                if (!wait_one(acc_empty_bar, ((uint32_t)ti & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                tc_fence_after();
                for (int kt = 0; kt < p.ktiles; ++kt, ++it) {
                    if (!wait_one(&kready[it % T::SR], (uint32_t)(it / T::SR) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t aoff = (uint32_t)((it % SA) * AM_BLOCK_BYTES) >> 4;
                    const uint32_t mcol = meta0 + (uint32_t)(it & 1) * 4u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t boff = (uint32_t)(((2 * it + h) % SB) * T::B_STAGE_BYTES) >> 4;
#pragma unroll
                        for (int b = 0; b < NB; b++) {
                            uint32_t mk[4] = {0u, 0u, 0u, 0u};  // bit set = output lane NOT written
                            if (NB == 2) {
                                mk[0] = mk[1] = (b == 0) ? 0u : 0xFFFFFFFFu;
                                mk[2] = mk[3] = (b == 0) ? 0xFFFFFFFFu : 0u;
                            } else if (NB == 4) {
                                mk[0] = (b == 0) ? 0u : 0xFFFFFFFFu;
                                mk[1] = (b == 1) ? 0u : 0xFFFFFFFFu;
                                mk[2] = (b == 2) ? 0u : 0xFFFFFFFFu;
                                mk[3] = (b == 3) ? 0u : 0xFFFFFFFFu;
                            }
#pragma unroll
                            for (int k2 = 0; k2 < 2; k2++) {
                                const int kb = h * 2 + k2;  // K=32 block inside the k-tile
                                // A: K-major, 128-byte swizzle, 8-row groups 1024 B apart; one MMA reads 32 B of each row.
                                // B: N-major, 128-byte swizzle; 8 gathered rows = 1024 B, next 64 columns = one slice further.
                                const uint64_t adesc = adesc0 + aoff + (uint32_t)(kb * 32 >> 4);
                                const uint64_t bdesc = bdesc0 + boff + (uint32_t)((b * T::B_BLOCK_BYTES + k2 * 4096) >> 4);
                                tc_mma_sp_f16(acc, adesc, bdesc, mcol + (uint32_t)(kb & ~1), idesc0 | (uint32_t)(kb & 1),
                                              (kt | kb) != 0 ? 1u : 0u, mk[0], mk[1], mk[2], mk[3]);
                            }
                        }
                    }
                    tc_commit(&kdone[it % T::SP]);
                    if (kt == p.ktiles - 1) tc_commit(acc_full_bar);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;  // tensor-memory lane quadrant this warp may read
        const int ew = warp - (3 + PB);  // 0..7: warps 0..3 drain the first half of the columns, 4..7 the second
        const int i = q * 32 + lane;
        const int arow = mma_row_to_actual(i);
        int ti = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++ti) {
            int mt, nt_cur;
            tile_coords(tile, p.mtiles, p.ntiles, p.group_m, &mt, &nt_cur);
            const int n0 = nt_cur * BN;
            const bool nm_tma = p.layout == 1 && p.nm_tma != 0;   // [N,M] through shared memory and TMA stores (the four warps of a group meet at named barriers)
            const bool got = wait_bounded(acc_full_bar, (uint32_t)ti & 1u, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE);
            if (nm_tma && !(BN / 64 < 2 && ew >= 4)) {
                if (!named_barrier_and(1 + (ew >> 2), 128, got)) break;   // the group leaves the loop together
            } else if (!got) {
                break;
            }
            tc_fence_after();
            // The tile is drained in parts of 64 columns to bound the register footprint; the
            // accumulator goes back to the MMA warp as soon as the last part is in registers.
            constexpr int PART = 64;
            const int64_t row = (int64_t)mt * TILE_M + arow;
            const bool row_ok = row < p.M;
            const bool has_bias = p.layout == 1 && p.bias != nullptr;
            const __half bias = (has_bias && row_ok) ? p.bias[row] : __ushort_as_half((unsigned short)0);
            constexpr int PARTS = BN / PART;
            constexpr int PER_GROUP = PARTS >= 2 ? PARTS / 2 : 1;  // parts per group of four warps
            const int part0 = (ew >> 2) * PER_GROUP;
            if (PARTS < 2 && ew >= 4) {  // a single part: the second group has nothing to read
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar);
                continue;
            }
#pragma unroll
            for (int pi = 0; pi < PER_GROUP; pi++) {
                const int part = part0 + pi;
                uint32_t pk[PART / 2];  // packed fp16 pairs: pk[c] = columns 2c, 2c+1 of this part
                {
                    uint32_t v0[32], v1[32];  // both loads in flight before the single wait
                    const uint32_t tcol = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(part * PART);
                    tc_ld_32x32b_x32(tcol, v0);
                    tc_ld_32x32b_x32(tcol + 32u, v1);
                    tc_wait_ld();
#pragma unroll
                    for (int jj = 0; jj < 16; jj++) {
                        __half2 h0 = __floats2half2_rn(__uint_as_float(v0[2 * jj]), __uint_as_float(v0[2 * jj + 1]));
                        __half2 h1 = __floats2half2_rn(__uint_as_float(v1[2 * jj]), __uint_as_float(v1[2 * jj + 1]));
                        pk[jj] = *reinterpret_cast<uint32_t *>(&h0);
                        pk[16 + jj] = *reinterpret_cast<uint32_t *>(&h1);
                    }
                }
                if (pi == PER_GROUP - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar);
                }
                if (nm_tma) {
                    // [N,M] + bias: the group's 128 rows x 32 columns go through 8 KiB of shared memory as [n][m] and leave
                    // as one TMA store per destination (boxes of 128 m x 32 n, clipped at M and N by the tensor map)
                    const int grp = ew >> 2;
                    uint8_t *stg = out_stage + grp * (4 * 32 * 64);
                    const bool leader = (ew & 3) == 0 && lane == 0;
#pragma unroll
                    for (int sub = 0; sub < 2; sub++) {
                        const int nsub = n0 + part * PART + sub * 32;
                        if (leader) bulk_wait_group_read0();   // the previous store has finished reading the staging buffer
                        named_barrier_sync(1 + grp, 128);
                        __half *col = reinterpret_cast<__half *>(stg) + arow;
#pragma unroll
                        for (int jj = 0; jj < 16; jj++) {
                            __half2 h = *reinterpret_cast<__half2 *>(&pk[sub * 16 + jj]);
                            __half lo = __low2half(h), hi = __high2half(h);
                            if (has_bias) { lo = __hadd(lo, bias); hi = __hadd(hi, bias); }
                            col[(2 * jj) * TILE_M] = lo;
                            col[(2 * jj + 1) * TILE_M] = hi;
                        }
                        fence_proxy_async();
                        named_barrier_sync(1 + grp, 128);
                        if (leader && nsub < p.N) {
                            tma_store_2d(&tmap_out, stg, mt * TILE_M, nsub);
                            for (int d = 1; d < p.n_out; d++) tma_store_2d(&more_out.m[d - 1], stg, mt * TILE_M, nsub);
                            bulk_commit_group();
                        }
                    }
                } else if (row_ok) {
                    const int nbase = n0 + part * PART;
                    if (p.layout == 0) {
                        // handled below, by the whole warp
                    } else {
                        __half *dst = p.out + (int64_t)nbase * p.ldo + row;
                        const int64_t step = p.ldo;
#pragma unroll
                        for (int jj = 0; jj < PART / 2; jj++) {
                            __half2 h = *reinterpret_cast<__half2 *>(&pk[jj]);
                            __half lo = __low2half(h), hi = __high2half(h);
                            if (has_bias) { lo = __hadd(lo, bias); hi = __hadd(hi, bias); }
                            if (nbase + 2 * jj < p.N) *dst = lo;
                            dst += step;
                            if (nbase + 2 * jj + 1 < p.N) *dst = hi;
                            dst += step;
                        }
                    }
                }
                if (p.layout == 0 && p.out32) {
                    // ablation (the reference's OUT_32B build, common/epilogue.h:34-61): every lane stores its own row
                    // in 32-bit words, 32 rows per instruction
                    if (row_ok) {
                        uint32_t *dst = reinterpret_cast<uint32_t *>(p.out + row * p.ldo + n0 + part * PART);
#pragma unroll
                        for (int jj = 0; jj < PART / 2; jj++)
                            if (n0 + part * PART + 2 * jj + 2 <= p.N) dst[jj] = pk[jj];
                    }
                } else if (p.layout == 0) {
                    // [M,N]: a lane holds 64 columns of ONE row, so a 16-byte store per lane would touch 32 rows with half
                    // a sector each.  The warp's 32 rows x 32 columns go through its own 2 KiB of shared memory instead
                    // (16-byte pieces XOR-swizzled, conflict-free both ways) and leave as full sectors: four lanes per row,
                    // eight rows per store instruction.
                    uint8_t *stg = out_stage + ew * (32 * 64);
                    const int slot = arow - q * 32;  // this lane's row inside the warp's 32 rows (actual order)
                    const int nbase = n0 + part * PART;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            *reinterpret_cast<uint4 *>(stg + slot * 64 + ((c ^ ((slot >> 1) & 3)) << 4)) =
                                make_uint4(pk[half * 16 + 4 * c], pk[half * 16 + 4 * c + 1], pk[half * 16 + 4 * c + 2], pk[half * 16 + 4 * c + 3]);
                        __syncwarp();
                        const int c = lane & 3;
                        const int col = nbase + half * 32 + c * 8;
#pragma unroll
                        for (int rr = 0; rr < 4; rr++) {
                            const int r = (lane >> 2) + 8 * rr;
                            const int64_t grow = (int64_t)mt * TILE_M + q * 32 + r;
                            const uint4 v = *reinterpret_cast<const uint4 *>(stg + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
                            if (grow < p.M && col + 8 <= p.N) *reinterpret_cast<uint4 *>(p.out + grow * p.ldo + col) = v;
                        }
                        __syncwarp();
                    }
                }
            }
        }
        if (p.layout == 1 && p.nm_tma != 0 && (ew & 3) == 0 && lane == 0) bulk_wait_group_read0();  // the stores have read shared memory (their global writes complete with the grid)
    }

    tc_fence_before();
    __syncthreads();
    if (warp == T::MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, T::TMEM_COLS);
    }
}

template <int BN, int NB, int SA, int SB, int PB>
cudaError_t set_attr()
{
    return cudaFuncSetAttribute(spmm_kernel<BN, NB, SA, SB, PB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Traits<BN, NB, SA, SB, PB>::SMEM_BYTES);
}

template <int BN, int NB, int SA, int SB, int PB>
cudaError_t launch_one(const SpmmConfig &cfg, const CUtensorMap &tmap_rows, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_out,
                       const OutMaps &more_out, const SpmmParams &p, cudaStream_t stream)
{
    using T = Traits<BN, NB, SA, SB, PB>;
    spmm_kernel<BN, NB, SA, SB, PB><<<(unsigned)cfg.grid, T::NUM_THREADS, T::SMEM_BYTES, stream>>>(tmap_rows, tmap_tile, tmap_out, more_out, p);
    return cudaGetLastError();
}

int g_num_sms = 0;

constexpr int kSA = 3, kSB = 4;

}  // namespace

// Tile configurations (128 rows x BN columns with NB * BN = 256, so every B stage is 32 KiB):
// V=128 -> one block per tile, BN 256; V=64 -> two blocks, BN 128; V=32 -> four blocks, BN 64.
// cfg->stages carries the number of B-producer warps (4 or 8).
bool spmm_select_config(int V, int N, int M, int producer_warps, int max_ctas, SpmmConfig *cfg)
{
    const int mtiles = (M + TILE_M - 1) / TILE_M;
    const int pb = (producer_warps == 4) ? 4 : 8;
    cfg->stages = pb;
    cfg->threads = (3 + pb + 8) * 32;
    if (V == 128) {
        cfg->bn = 256; cfg->nb = 1;
    } else if (V == 64) {
        cfg->bn = 128; cfg->nb = 2;
    } else if (V == 32) {
        cfg->bn = 64; cfg->nb = 4;
    } else {
        return false;
    }
    cfg->smem_bytes = Traits<256, 1, kSA, kSB, 8>::SMEM_BYTES;
    const long long tiles = (long long)mtiles * ((N + cfg->bn - 1) / cfg->bn);
    int sms = g_num_sms > 0 ? g_num_sms : 148;
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;  // the caller keeps some SMs free (e.g. for a collective that runs beside the product)
    cfg->grid = (int)(tiles < sms ? tiles : sms);
    return true;
}

cudaError_t spmm_init_kernels()
{
    cudaError_t e;
    if ((e = set_attr<256, 1, kSA, kSB, 8>()) != cudaSuccess) return e;
    if ((e = set_attr<128, 2, kSA, kSB, 8>()) != cudaSuccess) return e;
    if ((e = set_attr<64, 4, kSA, kSB, 8>()) != cudaSuccess) return e;
    if ((e = set_attr<256, 1, kSA, kSB, 4>()) != cudaSuccess) return e;
    if ((e = set_attr<128, 2, kSA, kSB, 4>()) != cudaSuccess) return e;
    if ((e = set_attr<64, 4, kSA, kSB, 4>()) != cudaSuccess) return e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    return cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
}

cudaError_t launch_spmm(const SpmmConfig &cfg, const CUtensorMap &tmap_rows, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_out,
                        const OutMaps &more_out, const SpmmParams &p, cudaStream_t stream)
{
    if (cfg.stages == 4) {
        if (cfg.nb == 1) return launch_one<256, 1, kSA, kSB, 4>(cfg, tmap_rows, tmap_tile, tmap_out, more_out, p, stream);
        if (cfg.nb == 2) return launch_one<128, 2, kSA, kSB, 4>(cfg, tmap_rows, tmap_tile, tmap_out, more_out, p, stream);
        if (cfg.nb == 4) return launch_one<64, 4, kSA, kSB, 4>(cfg, tmap_rows, tmap_tile, tmap_out, more_out, p, stream);
    } else {
        if (cfg.nb == 1) return launch_one<256, 1, kSA, kSB, 8>(cfg, tmap_rows, tmap_tile, tmap_out, more_out, p, stream);
        if (cfg.nb == 2) return launch_one<128, 2, kSA, kSB, 8>(cfg, tmap_rows, tmap_tile, tmap_out, more_out, p, stream);
        if (cfg.nb == 4) return launch_one<64, 4, kSA, kSB, 8>(cfg, tmap_rows, tmap_tile, tmap_out, more_out, p, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace vnm
