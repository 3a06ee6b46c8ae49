// V:N:M SpMM for sm_100a: C[M,N] = A_vnm[M,K] * B[K,N], fp16 in, fp32 accumulate in tensor memory.
//
// One CTA computes one 128 x BN output tile.  The 128 rows hold NB = 128/V vector blocks; each block
// has its own column-loc, hence its own gathered rows of B.  Per k-tile (64 compressed columns of A =
// 128 gathered rows of B) a stage of shared memory holds
//     [ value image 16 KiB | metadata image 2 KiB | NB gathered B tiles of 128 x BN fp16 ]
// Warp roles (192 threads):
//   warp 0      producer: one bulk copy for the value+metadata block, and TMA gather4 loads of B driven
//               by the precomputed absolute row numbers (each lane owns one group = four rows);
//   warp 1      tensor-memory allocation and MMA issue: copies the metadata image to tensor memory
//               (tcgen05.cp) and issues four K=32 tcgen05.mma.sp per block; for NB > 1 each MMA runs on
//               all 128 rows of the value tile with the output lanes of the other blocks disabled;
//   warps 2..5  epilogue: tcgen05.ld -> fp16 -> global ([M,N], or [N,M] with fused bias).
// Stages are handed over with mbarriers (full: producer -> MMA, empty: tcgen05.commit -> producer).
// Every wait is bounded: on expiry the kernel records a status bit, drains and returns.
#include "vnm_internal.h"

namespace vnm {

namespace {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at B200 clocks

template <int BN, int NB, int STAGES>
struct Traits {
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "tile N must be 64, 128, 192 or 256");
    static_assert(NB == 1 || NB == 2 || NB == 4, "128 rows hold 1, 2 or 4 vector blocks");
    static constexpr int B_BLOCK_BYTES = KT_ROWS * BN * 2;  // gathered tile of one vector block
    static constexpr int B_CHUNK_BYTES = KT_ROWS * 128;     // one 64-column slice: 128 rows x 128 B
    static constexpr int STAGE_BYTES = AM_BLOCK_BYTES + NB * B_BLOCK_BYTES;
    static_assert(STAGE_BYTES % 1024 == 0 && AM_BLOCK_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static constexpr int ACC_COLS = BN;
    static constexpr int META_COLS = 8;  // two alternating sets of four columns
    static constexpr int TMEM_COLS = (BN + META_COLS <= 32) ? 32 : (BN + META_COLS <= 64) ? 64 : (BN + META_COLS <= 128) ? 128
                                     : (BN + META_COLS <= 256) ? 256 : 512;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
    static constexpr int THREADS = 192;
};

// Whole-warp bounded wait on an mbarrier phase; lane 0 polls.  Returns false if the wait expired or
// another role already aborted.
__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = 0;
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
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

template <int BN, int NB, int STAGES>
__global__ void __launch_bounds__(192, 1) spmm_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    using T = Traits<BN, NB, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + STAGES * T::STAGE_BYTES);
    uint64_t *empty_bar = full_bar + STAGES;
    uint64_t *accum_bar = empty_bar + STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int mt = blockIdx.x % p.mtiles;  // row tiles fastest: CTAs that run together share a column panel of B
    const int nt = blockIdx.x / p.mtiles;
    const int n0 = nt * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, T::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) tma_prefetch_desc(&tmap_b);
        int issued = 0;
        for (int kt = 0; kt < p.ktiles; ++kt) {
            const int s = kt % STAGES;
            const uint32_t ph = (uint32_t)(kt / STAGES) & 1u;
            if (!wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_PRODUCER)) break;
            uint8_t *st = smem + s * T::STAGE_BYTES;
            if (lane == 0) {
                mbar_arrive_expect_tx(&full_bar[s], T::STAGE_BYTES);
                bulk_g2s(st, p.am + ((size_t)mt * p.ktiles + kt) * AM_BLOCK_BYTES, AM_BLOCK_BYTES, &full_bar[s]);
            }
            __syncwarp();
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int4 r = __ldg(p.rows + ((size_t)(mt * NB + b) * p.ktiles + kt) * KT_GROUPS + lane);
                uint8_t *dst = st + AM_BLOCK_BYTES + b * T::B_BLOCK_BYTES + lane * 512;
#pragma unroll
                for (int c = 0; c < BN / 64; c++) tma_gather4(dst + c * T::B_CHUNK_BYTES, &tmap_b, n0 + c * 64, r, &full_bar[s]);
            }
            issued = kt + 1;
        }
        if (*abort_flag) {
            // Drain: wait (bounded) until the copies of the stages still in flight have landed.
            const int first = issued > STAGES ? issued - STAGES : 0;
            for (int kt = first; kt < issued; ++kt) {
                const int s = kt % STAGES;
                const uint32_t ph = (uint32_t)(kt / STAGES) & 1u;
                int ok = 1;
                if (lane == 0) {
                    ok = 0;
                    const long long t0 = clock64();
                    while (clock64() - t0 < WAIT_LIMIT_CYCLES / 4) {
                        if (mbar_try_wait(&full_bar[s], ph)) { ok = 1; break; }
                    }
                    if (!ok) atomicOr(p.status, DEV_TIMEOUT_DRAIN);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const uint32_t acc = tmem_base;
        const uint32_t meta0 = tmem_base + T::ACC_COLS;
        for (int kt = 0; kt < p.ktiles; ++kt) {
            const int s = kt % STAGES;
            const uint32_t ph = (uint32_t)(kt / STAGES) & 1u;
            if (!wait_bounded(&full_bar[s], ph, abort_flag, p.status, DEV_TIMEOUT_MMA)) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t sbase = smem_u32(smem + s * T::STAGE_BYTES);
                const uint32_t mcol = meta0 + (uint32_t)(kt & 1) * 4u;
                // metadata image: 128 rows x 16 bytes, 8-row core matrices stored back to back
                tc_cp_128x128b(mcol, make_smem_desc(sbase + A_IMG_BYTES, 0, 128, 0));
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
                    for (int kb = 0; kb < 4; kb++) {
                        // A: K-major, 128-byte swizzle, 8-row groups 1024 B apart; one MMA reads 32 B of each row
                        const uint64_t adesc = make_smem_desc(sbase + kb * 32, 16, 1024, 2);
                        // B: N-major, 128-byte swizzle; 8 gathered rows = 1024 B, next 64 columns = one chunk further
                        const uint64_t bdesc =
                            make_smem_desc(sbase + AM_BLOCK_BYTES + b * T::B_BLOCK_BYTES + kb * 4096, T::B_CHUNK_BYTES, 1024, 2);
                        const uint32_t idesc = make_idesc_f16(TILE_M, BN, true, (uint32_t)(kb & 1), true);
                        tc_mma_sp_f16(acc, adesc, bdesc, mcol + (uint32_t)(kb & ~1), idesc, (kt | kb) != 0 ? 1u : 0u, mk[0], mk[1],
                                      mk[2], mk[3]);
                    }
                }
                tc_commit(&empty_bar[s]);
                if (kt == p.ktiles - 1) tc_commit(accum_bar);
            }
            __syncwarp();
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;  // tensor-memory lane quadrant this warp may read
        if (wait_bounded(accum_bar, 0, abort_flag, p.status, DEV_TIMEOUT_EPILOGUE)) {
            tc_fence_after();
            const int i = q * 32 + lane;
            const int64_t row = (int64_t)mt * TILE_M + mma_row_to_actual(i);
            const bool row_ok = row < p.M;
            __half bias = __ushort_as_half((unsigned short)0);
            if (p.layout == 1 && p.bias != nullptr && row_ok) bias = p.bias[row];
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tc_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                tc_wait_ld();
                if (!row_ok) continue;
                const int n = n0 + c0;
                if (p.layout == 0) {
                    __half *dst = p.out + row * p.ldo + n;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (n + j * 8 + 8 <= p.N) {
                            uint4 o;
                            __half2 h;
                            h = __floats2half2_rn(__uint_as_float(v[j * 8 + 0]), __uint_as_float(v[j * 8 + 1]));
                            o.x = *reinterpret_cast<uint32_t *>(&h);
                            h = __floats2half2_rn(__uint_as_float(v[j * 8 + 2]), __uint_as_float(v[j * 8 + 3]));
                            o.y = *reinterpret_cast<uint32_t *>(&h);
                            h = __floats2half2_rn(__uint_as_float(v[j * 8 + 4]), __uint_as_float(v[j * 8 + 5]));
                            o.z = *reinterpret_cast<uint32_t *>(&h);
                            h = __floats2half2_rn(__uint_as_float(v[j * 8 + 6]), __uint_as_float(v[j * 8 + 7]));
                            o.w = *reinterpret_cast<uint32_t *>(&h);
                            *reinterpret_cast<uint4 *>(dst + j * 8) = o;
                        }
                    }
                } else {
                    const bool has_bias = p.bias != nullptr;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (n + j < p.N) {
                            __half h = __float2half_rn(__uint_as_float(v[j]));
                            if (has_bias) h = __hadd(h, bias);
                            p.out[(int64_t)(n + j) * p.ldo + row] = h;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, T::TMEM_COLS);
    }
}

template <int BN, int NB, int STAGES>
cudaError_t set_attr()
{
    return cudaFuncSetAttribute(spmm_kernel<BN, NB, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, Traits<BN, NB, STAGES>::SMEM_BYTES);
}

template <int BN, int NB, int STAGES>
cudaError_t launch_one(const CUtensorMap &tmap_b, const SpmmParams &p, cudaStream_t stream)
{
    using T = Traits<BN, NB, STAGES>;
    const unsigned grid = (unsigned)p.mtiles * (unsigned)p.ntiles;
    spmm_kernel<BN, NB, STAGES><<<grid, T::THREADS, T::SMEM_BYTES, stream>>>(tmap_b, p);
    return cudaGetLastError();
}

}  // namespace

// Tile configurations: V=128 -> one block per tile, N tile 256 (2 stages) or 128 (4 stages) when the
// wide tile would leave most SMs idle; V=64 -> two blocks, N tile 128; V=32 -> four blocks, N tile 64.
bool spmm_select_config(int V, int N, int M, SpmmConfig *cfg)
{
    const int mtiles = (M + TILE_M - 1) / TILE_M;
    cfg->threads = 192;
    if (V == 128) {
        const long long wide_tiles = (long long)mtiles * ((N + 255) / 256);
        if (wide_tiles >= 148) {
            cfg->bn = 256; cfg->nb = 1; cfg->stages = 2; cfg->smem_bytes = Traits<256, 1, 2>::SMEM_BYTES;
        } else {
            cfg->bn = 128; cfg->nb = 1; cfg->stages = 4; cfg->smem_bytes = Traits<128, 1, 4>::SMEM_BYTES;
        }
        return true;
    }
    if (V == 64) {
        cfg->bn = 128; cfg->nb = 2; cfg->stages = 2; cfg->smem_bytes = Traits<128, 2, 2>::SMEM_BYTES;
        return true;
    }
    if (V == 32) {
        cfg->bn = 64; cfg->nb = 4; cfg->stages = 2; cfg->smem_bytes = Traits<64, 4, 2>::SMEM_BYTES;
        return true;
    }
    return false;
}

cudaError_t spmm_init_kernels()
{
    cudaError_t e;
    if ((e = set_attr<256, 1, 2>()) != cudaSuccess) return e;
    if ((e = set_attr<128, 1, 4>()) != cudaSuccess) return e;
    if ((e = set_attr<128, 2, 2>()) != cudaSuccess) return e;
    if ((e = set_attr<64, 4, 2>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_spmm(const SpmmConfig &cfg, const CUtensorMap &tmap_b, const SpmmParams &p, cudaStream_t stream)
{
    if (cfg.bn == 256 && cfg.nb == 1) return launch_one<256, 1, 2>(tmap_b, p, stream);
    if (cfg.bn == 128 && cfg.nb == 1) return launch_one<128, 1, 4>(tmap_b, p, stream);
    if (cfg.bn == 128 && cfg.nb == 2) return launch_one<128, 2, 2>(tmap_b, p, stream);
    if (cfg.bn == 64 && cfg.nb == 4) return launch_one<64, 4, 2>(tmap_b, p, stream);
    return cudaErrorInvalidValue;
}

}  // namespace vnm
