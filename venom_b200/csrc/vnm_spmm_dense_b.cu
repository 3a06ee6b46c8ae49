// SpMM kernel for the dense-B operand form (the V:2:m pattern re-expressed as 2:4 over all K columns).
//
// Here B is read as ordinary tiles that every row of A shares, so one CTA can reuse a B stage for two
// 128-row tiles of A: a 256 x 128 output tile with two accumulators (128 tensor-memory columns each).
// Per k-tile (128 original columns of A = 128 rows of B) the CTA streams
//     2 x 18 KiB value + metadata blocks   and   2 x 16 KiB stages of B (64 rows x 128 columns)
// = 68 KiB for eight 128 x 128 x 32 MMAs, against 82 KiB for four 128 x 256 x 32 MMAs in the gather
// kernel.  Fewer bytes per MMA clock means more k-tiles of MMA work buffered in the same shared memory,
// which is what hides the load latency.
//
// Warp roles (384 threads):
//   warp 0      A producer (one thread): two bulk copies per k-tile.
//   warp 1      B producer (one thread): two TMA tile loads (64 rows x 64 columns) per stage.
//   warp 2      sequencer (one thread): waits for the A blocks, copies both metadata images to tensor
//               memory, waits for the B stages, flips the k-tile's "ready" barrier.
//   warp 3      MMA issuer (one thread) and tensor-memory owner: one wait, eight MMAs, one commit per k-tile.
//   warps 4..11 epilogue: four warps per accumulator drain it, hand it back, store.
// Every wait is bounded: on expiry the kernel records a status bit, drains and returns.
#include "vnm_internal.h"

namespace vnm {

namespace {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at B200 clocks

#ifdef VNM_TRACE
// Debug build only: CTA 0 records clock64() stamps of its pipeline hand-offs into p.trace.
#define TRACE(slot, idx) do { if (blockIdx.x == 0 && (idx) < 4096 && p.trace) p.trace[(slot) * 4096 + (idx)] = clock64(); } while (0)
#else
#define TRACE(slot, idx) do { } while (0)
#endif

constexpr int RT = 2;            // row tiles per CTA tile
constexpr int BN = 128;          // output columns per CTA tile
constexpr int SA = 3;            // A ring: k-tiles (each RT blocks)
constexpr int SB = 5;            // B ring: stages of 64 rows x BN columns
constexpr int SP = 4;            // k-tile "done" barriers
constexpr int SR = 4;            // k-tile "ready" barriers
constexpr int META_SETS = 3;     // metadata column sets in tensor memory (4 columns per row tile each)
constexpr int B_CHUNK_BYTES = 64 * 128;            // 64 rows x 64 columns
constexpr int B_STAGE_BYTES = (BN / 64) * B_CHUNK_BYTES;  // 16 KiB
constexpr int A_STAGE_BYTES = RT * AM_BLOCK_BYTES;  // 36 KiB
constexpr int A_RING_BYTES = SA * A_STAGE_BYTES;
constexpr int B_RING_BYTES = SB * B_STAGE_BYTES;
constexpr int OUT_STAGE_BYTES = TILE_M * 128;       // 128 rows x 64 fp16 columns, staging of one TMA store
constexpr int OUT_RING_BYTES = RT * OUT_STAGE_BYTES;  // one staging buffer per accumulator
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = A_RING_BYTES + B_RING_BYTES + OUT_RING_BYTES + BAR_BYTES + 1024;
static_assert(A_RING_BYTES % 1024 == 0 && B_RING_BYTES % 1024 == 0, "swizzled staging needs 1024-byte alignment");
constexpr int NUM_THREADS = 384;  // 4 single-thread roles + 2 x 4 epilogue warps
constexpr int TMEM_COLS = 512;
constexpr int ACC_SLOTS = RT + 1;  // accumulator (tile ti, row tile rt) lives in slot (RT * ti + rt) % ACC_SLOTS
constexpr int META_COL0 = ACC_SLOTS * BN;  // first metadata column
static_assert(SP >= SA && 2 * SP >= SB + 1, "too few k-tile barriers: a waiter could miss a phase");
static_assert(META_COL0 + META_SETS * RT * 4 <= TMEM_COLS, "tensor memory overflow");
static_assert((SA + SB + SP + SR + 2 * ACC_SLOTS) * 8 + 16 <= BAR_BYTES, "barrier area too small");

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

__global__ void __launch_bounds__(NUM_THREADS, 1) spmm_dense_b_kernel(const __grid_constant__ CUtensorMap tmap_tile, const __grid_constant__ CUtensorMap tmap_out,
                                                                      const SpmmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *a_ring = smem;
    uint8_t *b_ring = smem + A_RING_BYTES;
    uint8_t *out_ring = smem + A_RING_BYTES + B_RING_BYTES;
    uint64_t *a_full = reinterpret_cast<uint64_t *>(smem + A_RING_BYTES + B_RING_BYTES + OUT_RING_BYTES);
    uint64_t *b_full = a_full + SA;
    uint64_t *kdone = b_full + SB;
    uint64_t *kready = kdone + SP;
    uint64_t *acc_full_bar = kready + SR;
    uint64_t *acc_empty_bar = acc_full_bar + ACC_SLOTS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty_bar + ACC_SLOTS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // tiles: pairs of row tiles (fastest) x column tiles
    const int mpairs = (p.mtiles + RT - 1) / RT;
    const int total_tiles = mpairs * p.ntiles;
    const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total_it = my_tiles * p.ktiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; s++) mbar_init(&a_full[s], 1);
        for (int s = 0; s < SB; s++) mbar_init(&b_full[s], 1);
        for (int s = 0; s < SP; s++) mbar_init(&kdone[s], 1);
        for (int s = 0; s < SR; s++) mbar_init(&kready[s], 2);  // metadata copies done + operands landed
        for (int s = 0; s < ACC_SLOTS; s++) {
            mbar_init(&acc_full_bar[s], 1);
            mbar_init(&acc_empty_bar[s], 4);  // the four warps that drain it
        }
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

    if (warp == 0) {
        // ---------------- A producer ----------------
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x) {
                const int mp = tile % mpairs;
                for (int kt = 0; kt < p.ktiles; ++kt, ++it) {
                    const int s = it % SA;
                    if (it >= SA) {
                        const int kd = it - SA;
                        if (!wait_one(&kdone[kd % SP], (uint32_t)(kd / SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) { alive = false; break; }
                    }
                    TRACE(0, it);
                    mbar_arrive_expect_tx(&a_full[s], A_STAGE_BYTES);
#pragma unroll
                    for (int rt = 0; rt < RT; rt++) {
                        // a missing second row tile (odd number of row tiles) re-reads the first one; its rows are never stored
                        const int mt = (mp * RT + rt < p.mtiles) ? mp * RT + rt : mp * RT;
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
    } else if (warp == 1) {
        // ---------------- B producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_tile);
            int j = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x) {
                const int n0 = (tile / mpairs) * BN;
                for (int jl = 0; jl < 2 * p.ktiles; ++jl, ++j) {
                    const int s = j % SB;
                    if (j >= SB) {
                        const int kd = (j - SB) >> 1;
                        if (!wait_one(&kdone[kd % SP], (uint32_t)(kd / SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) { alive = false; break; }
                    }
                    TRACE(1, j);
                    if (p.gather_mode != GATHER_NONE) {
                        mbar_arrive_expect_tx(&b_full[s], B_STAGE_BYTES);
                        if (p.b_nk) {
                            // B given as [N, K]: one box of 128 rows (n) x 64 k, i.e. a K-major operand tile
                            tma_load_2d(b_ring + s * B_STAGE_BYTES, &tmap_tile, jl * 64, n0, &b_full[s]);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 64; c++)
                                tma_load_2d(b_ring + s * B_STAGE_BYTES + c * B_CHUNK_BYTES, &tmap_tile, n0 + c * 64, jl * 64, &b_full[s]);
                        }
                    } else {
                        mbar_arrive(&b_full[s]);
                    }
                }
            }
            if (*abort_flag && p.gather_mode != GATHER_NONE) {
                for (int k = j > SB ? j - SB : 0; k < j; ++k) drain_slot(&b_full[k % SB], (uint32_t)(k / SB) & 1u, p.status);
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---------------- sequencer ----------------
        if (lane == 0) {
            const uint64_t mdesc0 = make_smem_desc(smem_u32(a_ring) + A_IMG_BYTES, 0, 128, 0);
            bool alive = true;
            for (int it = 0; alive && it < total_it; ++it) {
                const int sa = it % SA;
                // column set it % META_SETS was last read by the MMAs of k-tile it - META_SETS
                if (it >= META_SETS) {
                    const int kd = it - META_SETS;
                    if (!wait_one(&kdone[kd % SP], (uint32_t)(kd / SP) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                }
                if (!wait_one(&a_full[sa], (uint32_t)(it / SA) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
                tc_fence_after();
                TRACE(4, 2 * it);
                const uint32_t mcol = tmem_base + META_COL0 + (uint32_t)(it % META_SETS) * (RT * 4);
#pragma unroll
                for (int rt = 0; rt < RT; rt++)
                    tc_cp_128x128b(mcol + rt * 4, mdesc0 + ((uint32_t)(sa * A_STAGE_BYTES + rt * AM_BLOCK_BYTES) >> 4));
                tc_commit(&kready[it % SR]);
                for (int h = 0; h < 2; ++h) {
                    const int j = 2 * it + h;
                    if (!wait_one(&b_full[j % SB], (uint32_t)(j / SB) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                }
                TRACE(4, 2 * it + 1);
                if (alive) mbar_arrive(&kready[it % SR]);
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const bool b_nk = p.b_nk != 0;
            const uint32_t idesc0 = make_idesc_f16(TILE_M, BN, true, 0u, !b_nk);
            const uint64_t adesc0 = make_smem_desc(smem_u32(a_ring), 16, 1024, 2);
            // B stage: N-major (two 64-column slices, 64 k-rows of 128 B each) or K-major (128 n-rows of 128 B = 64 k)
            const uint64_t bdesc0 = b_nk ? make_smem_desc(smem_u32(b_ring), 16, 1024, 2) : make_smem_desc(smem_u32(b_ring), B_CHUNK_BYTES, 1024, 2);
            const uint32_t bstep = b_nk ? (64u >> 4) : (4096u >> 4);  // next K=32 block: 32 k = 64 B along a row, or 32 rows further
            int it = 0;
            bool alive = true;
            for (int ti = 0; alive && ti < my_tiles; ++ti) {
                // Accumulator slots rotate: row tile 0 of this tile has a slot nobody is draining, row tile 1
                // takes over the slot row tile 0 of the previous tile is being drained from.  Inside a k-tile
                // all MMAs of row tile 0 come first, so its drain also starts half a k-tile early.
                for (int kt = 0; alive && kt < p.ktiles; ++kt, ++it) {
                    TRACE(2, it);
                    if (!wait_one(&kready[it % SR], (uint32_t)(it / SR) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                    tc_fence_after();
                    TRACE(3, it);
                    const uint32_t mcol = tmem_base + META_COL0 + (uint32_t)(it % META_SETS) * (RT * 4);
#pragma unroll
                    for (int rt = 0; rt < RT; rt++) {
                        const int use = RT * ti + rt, slot = use % ACC_SLOTS;
                        if (kt == 0) {
                            if (rt == 0) TRACE(7, ti * 2);
                            if (!wait_one(&acc_empty_bar[slot], ((uint32_t)(use / ACC_SLOTS) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA)) { alive = false; break; }
                            tc_fence_after();
                            if (rt == 0) TRACE(7, ti * 2 + 1);
                        }
                        const uint32_t aoff = (uint32_t)((it % SA) * A_STAGE_BYTES + rt * AM_BLOCK_BYTES) >> 4;
#pragma unroll
                        for (int kb = 0; kb < 4; kb++) {  // K=32 blocks of the k-tile; two per B stage
                            const uint32_t boff = (uint32_t)(((2 * it + (kb >> 1)) % SB) * B_STAGE_BYTES) >> 4;
                            tc_mma_sp_f16(tmem_base + slot * BN, adesc0 + aoff + (uint32_t)(kb * 32 >> 4), bdesc0 + boff + (uint32_t)(kb & 1) * bstep,
                                          mcol + rt * 4 + (uint32_t)(kb & ~1), idesc0 | (uint32_t)(kb & 1), (kt | kb) != 0 ? 1u : 0u, 0u, 0u, 0u, 0u);
                        }
                        if (kt == p.ktiles - 1) tc_commit(&acc_full_bar[slot]);
                    }
                    if (!alive) break;
                    tc_commit(&kdone[it % SP]);
                    TRACE(5, it);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;
        const int i = q * 32 + lane;
        const int arow = mma_row_to_actual(i);
        int ti = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
            const int mp = tile % mpairs;
            const int n0 = (tile / mpairs) * BN;
            // the four warps of a group leave the loop together (they meet at named barriers below)
            const int use = RT * ti + ((warp - 4) >> 2), slot = use % ACC_SLOTS;
            const bool got = wait_warp(&acc_full_bar[slot], (uint32_t)(use / ACC_SLOTS) & 1u, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE);
            if (!named_barrier_and(1 + ((warp - 4) >> 2), 128, got)) break;
            tc_fence_after();
            if (warp == 4 && lane == 0) TRACE(6, ti * 3);
            constexpr int PART = 64;
            {
                const int rt = (warp - 4) >> 2;  // which accumulator this warp drains
                const int mt = mp * RT + rt;
                const int64_t row = (int64_t)mt * TILE_M + arow;
                const bool row_ok = mt < p.mtiles && row < p.M;
                const bool has_bias = p.layout == 1 && p.bias != nullptr;
                const __half bias = (has_bias && row_ok) ? p.bias[row] : __ushort_as_half((unsigned short)0);
                // The whole 128-column row of the accumulator goes into registers as packed halves first, so
                // that the MMA issuer gets the accumulator back before any staging or store work starts.
                uint32_t pk_all[BN / 2];
#pragma unroll
                for (int part = 0; part < BN / PART; part++) {
                    uint32_t v0[32], v1[32];
                    const uint32_t tcol = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * BN + part * PART);
                    tc_ld_32x32b_x32(tcol, v0);
                    tc_ld_32x32b_x32(tcol + 32u, v1);
                    tc_wait_ld();
#pragma unroll
                    for (int jj = 0; jj < 16; jj++) {
                        __half2 h0 = __floats2half2_rn(__uint_as_float(v0[2 * jj]), __uint_as_float(v0[2 * jj + 1]));
                        __half2 h1 = __floats2half2_rn(__uint_as_float(v1[2 * jj]), __uint_as_float(v1[2 * jj + 1]));
                        pk_all[part * (PART / 2) + jj] = *reinterpret_cast<uint32_t *>(&h0);
                        pk_all[part * (PART / 2) + 16 + jj] = *reinterpret_cast<uint32_t *>(&h1);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty_bar[slot]);
                if (warp == 4 && lane == 0) TRACE(6, ti * 3 + 1);
#pragma unroll
                for (int part = 0; part < BN / PART; part++) {
                    const uint32_t *pk = pk_all + part * (PART / 2);
                    if (p.layout == 0) {
                        // [M,N] output: stage 128 rows x 64 columns in shared memory (128-byte swizzle, rows at
                        // their actual position) and let one TMA store write full lines; it clips at M and N.
                        uint8_t *stg = out_ring + rt * OUT_STAGE_BYTES;
                        const bool leader = (warp == 4 + 4 * rt) && lane == 0;
                        if (leader) bulk_wait_group_read0();  // the previous store has finished reading the staging buffer
                        named_barrier_sync(1 + rt, 128);
#pragma unroll
                        for (int c = 0; c < 8; c++)
                            *reinterpret_cast<uint4 *>(stg + arow * 128 + ((c ^ (arow & 7)) << 4)) =
                                make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                        fence_proxy_async();
                        named_barrier_sync(1 + rt, 128);
                        if (leader && mt < p.mtiles) {
                            tma_store_2d(&tmap_out, stg, n0 + part * PART, mt * TILE_M);
                            bulk_commit_group();
                        }
                    } else {
                        // [N,M] output (+ bias): stage the transposed part, 64 rows (n) x 128 columns (m) without
                        // swizzle -- the 32 lanes of a warp write 32 consecutive m of one n -- and store it with
                        // one TMA store, which clips at N and M.
                        uint8_t *stg = out_ring + rt * OUT_STAGE_BYTES;
                        const bool leader = (warp == 4 + 4 * rt) && lane == 0;
                        if (leader) bulk_wait_group_read0();
                        named_barrier_sync(1 + rt, 128);
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
                        fence_proxy_async();
                        named_barrier_sync(1 + rt, 128);
                        if (leader && mt < p.mtiles) {
                            tma_store_2d(&tmap_out, stg, mt * TILE_M, n0 + part * PART);
                            bulk_commit_group();
                        }
                    }
                }
            }
        }
    }

    if (warp >= 4 && ((warp - 4) & 3) == 0 && lane == 0) bulk_wait_group0();  // this thread's TMA stores are complete
    tc_fence_before();
    __syncthreads();
    if (warp == 3) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

int g_num_sms_db = 0;

}  // namespace

cudaError_t spmm_dense_b_init()
{
    cudaError_t e = cudaFuncSetAttribute(spmm_dense_b_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    return cudaDeviceGetAttribute(&g_num_sms_db, cudaDevAttrMultiProcessorCount, dev);
}

void spmm_dense_b_config(int M, int N, SpmmConfig *cfg)
{
    const int mtiles = (M + TILE_M - 1) / TILE_M;
    const long long tiles = (long long)((mtiles + RT - 1) / RT) * ((N + BN - 1) / BN);
    const int sms = g_num_sms_db > 0 ? g_num_sms_db : 148;
    cfg->bn = BN;
    cfg->nb = 1;
    cfg->stages = 1;
    cfg->smem_bytes = SMEM_BYTES;
    cfg->threads = NUM_THREADS;
    cfg->grid = (int)(tiles < sms ? tiles : sms);
}

cudaError_t launch_spmm_dense_b(const SpmmConfig &cfg, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_out, const SpmmParams &p,
                                cudaStream_t stream)
{
    spmm_dense_b_kernel<<<(unsigned)cfg.grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap_tile, tmap_out, p);
    return cudaGetLastError();
}

}  // namespace vnm
