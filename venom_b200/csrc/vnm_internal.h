// Internal interface between the C ABI (vnm_capi.cu) and the kernel translation units.
#pragma once

#include "vnm_common.cuh"
#include <cuda.h>

namespace vnm {

// Device-side status word values (sticky, OR-ed): which bounded wait gave up.
enum : int {
    DEV_OK = 0,
    DEV_TIMEOUT_PRODUCER = 1,  // producer waited for a free stage
    DEV_TIMEOUT_MMA = 2,       // MMA issuer waited for a filled stage
    DEV_TIMEOUT_EPILOGUE = 4,  // epilogue waited for the accumulator
    DEV_TIMEOUT_DRAIN = 8      // drain of in-flight copies after an abort gave up
};

struct SpmmParams {
    const uint8_t *am;    // [mtiles][ktiles][AM_BLOCK_BYTES] value + metadata images
    const int4 *rows;     // [vblocks_padded][ktiles*32] absolute B rows
    const __half *bias;   // [M] or null
    __half *out;
    int64_t ldo;
    int M, N, K;
    int V;
    int mtiles, ktiles, ntiles;
    int layout;           // 0 = [M,N], 1 = [N,M] + bias
    int *status;          // device status word
    int gather_mode;      // GATHER_* below
    int total_tiles;      // mtiles * ntiles
    const __half *B;      // gather kernel, GATHER_CPASYNC: the dense operand [K, N] itself (row pieces are copied by address)
    int64_t ldb;
    int hybrid_rows;      // gather kernel, GATHER_CPASYNC: rows per block and stage fetched by TMA gather4 beside the copies (0, 16, 32, 48)
    int group_m;          // band of the tile order (tile_coords): > 0 row groups per band, < 0 column tiles per band
    uint64_t hint_a, hint_b;  // pair kernel: L2 eviction-priority policies of the A and B loads (L2_EVICT_*)
    int out32;            // gather kernel, layout MN: 32-bit stores from registers instead of staged 128-bit stores (ablation)
    int b_nk;             // dense-B kernel only: the dense operand is given as [N, K] row-major (K contiguous)
    int b_wide_ok;        // dense-B kernel only: the 4-D tensor map exists (column tiles with 256 columns inside N use one box per stage)
    int l2_ahead;         // pair kernel: k-tiles by which L2 prefetches run ahead of the loads into shared memory (0 = none)
    int nm_tma;           // gather kernel, layout NM: the result leaves through shared memory and TMA stores (tmap_out / OutMaps valid)
    int n_out;            // dense-B kernels, and the gather kernel with nm_tma: destinations of every output tile (1 = `out` only; more: the OutMaps argument, e.g. peers' buffers)
};

// Destinations 2 .. MAX_OUTS of a product whose every output tile is stored to several buffers of one geometry
// (a rank's own result buffer and the same rows of its peers' buffers): tensor maps like the first output map.
constexpr int MAX_OUTS = 8;
struct alignas(64) OutMaps {
    CUtensorMap m[MAX_OUTS - 1];
};

// How the producer warps bring the selected rows of B into shared memory.
enum : int {
    GATHER_TMA4 = 0,    // TMA tile::gather4, four rows (one group) per instruction (default for m > 4)
    GATHER_CONTIG = 1,  // plain TMA tiles of 64 consecutive rows: exact when m == 4 (every row is
                        // selected), otherwise an ablation that drops the column-loc indirection
    GATHER_NONE = 2,    // ablation only: B is not loaded at all (results are meaningless)
    GATHER_CPASYNC = 3  // per-thread 16-byte asynchronous copies of the selected rows, optionally split with TMA gather4 (ablation: measured slower)
};

struct SpmmConfig {
    int bn;      // tile N
    int nb;      // V-blocks per 128-row tile
    int stages;  // number of B-producer warps (4 or 8)
    int smem_bytes;
    int threads;
    int grid;    // persistent CTAs
};

// Host-side helpers shared by the translation units that implement C-ABI entry points (defined in vnm_capi.cu).
int set_last_error(int code, const char *msg);       // message of vnm_last_error_string() for this thread; returns code
int check_format(int M, int K, int V, int n, int m);  // VNM_OK or an error code with the message set
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn();                        // cuTensorMapEncodeTiled from the driver, or null (thread-safe)

cudaError_t launch_compress(const void *dense, int64_t ldd, const int32_t *mask, const uint32_t *colloc, int M, int K, int V, int m,
                            void *values, uint32_t *meta, unsigned long long *violations, cudaStream_t stream);
cudaError_t launch_decompress(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int m,
                              void *dense, int64_t ldd, cudaStream_t stream);
cudaError_t launch_prepare(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int m, void *am,
                           void *rows, int mtiles, int ktiles, int vblocks_padded, cudaStream_t stream);

cudaError_t launch_prepare_dense_b(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int m,
                                   void *am, void *rows, int mtiles, int ktiles, cudaStream_t stream);

cudaError_t launch_prune(const float *w, int64_t ldw, int M, int K, int V, int m, int32_t *mask, int64_t ldm, uint32_t *colloc,
                         cudaStream_t stream);

// Chooses the tile configuration for (V, N).  Returns false for an unsupported V.
bool spmm_select_config(int V, int N, int M, int producer_warps, int max_ctas, SpmmConfig *cfg);  // max_ctas: 0 = one per SM
// Opt-in to large dynamic shared memory for every kernel instance on the CURRENT device (call once per device).
cudaError_t spmm_init_kernels();
cudaError_t launch_spmm(const SpmmConfig &cfg, const CUtensorMap &tmap_rows, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_out,
                        const OutMaps &more_out, const SpmmParams &p,
                        cudaStream_t stream);

// Dense-B form: 256 x 128 tiles, two accumulators sharing every B stage (vnm_spmm_dense_b.cu).
cudaError_t spmm_dense_b_init();
cudaError_t launch_wait_expiry_selftest(int *status, cudaStream_t stream);
void spmm_dense_b_config(int M, int N, int max_ctas, SpmmConfig *cfg);  // max_ctas: 0 = one per SM
cudaError_t launch_spmm_dense_b(const SpmmConfig &cfg, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_tile2, const CUtensorMap &tmap_out, const OutMaps &more_out,
                                const SpmmParams &p, cudaStream_t stream);

// Dense-B form on pairs of SMs (clusters of two CTAs, tcgen05 cta_group::2): 512 x 240 pair tiles (vnm_spmm_dense_b2.cu).
cudaError_t spmm_dense_b_pair_init();
bool spmm_dense_b_pair_config(int M, int N, int K, int max_ctas, int force_rows, SpmmConfig *cfg);  // false: use the single-CTA kernel; force_rows: 0 auto, 1 / 2 row tiles per CTA
cudaError_t launch_spmm_dense_b_pair(const SpmmConfig &cfg, const CUtensorMap &tmap_tile, const CUtensorMap &tmap_tile2, const CUtensorMap &tmap_out, const OutMaps &more_out,
                                     const SpmmParams &p, cudaStream_t stream);

}  // namespace vnm
