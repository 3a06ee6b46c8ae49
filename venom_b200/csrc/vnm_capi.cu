// C ABI of venom_b200 (see include/venom_b200.h).  Host-side argument checking, the prepared-operand
// handle, TMA descriptor construction for the dense operand, and kernel dispatch.
#include "../../include/venom_b200.h"
#include "vnm_internal.h"
#include <mutex>

#include <cstdio>
#include <cstdlib>
#include <cstdarg>
#include <cstring>
#include <new>
#include <string>

using namespace vnm;

namespace {
thread_local std::string g_last_error;
}

namespace vnm {
// Records the message returned by vnm_last_error_string() on this thread and passes the code through.
int set_last_error(int code, const char *msg)
{
    g_last_error = msg;
    return code;
}
}  // namespace vnm

namespace {

int fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    return set_last_error(code, buf);
}

int fail_cuda(cudaError_t e, const char *what)
{
    return fail(VNM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define VNM_CUDA(call, what)                                   \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return fail_cuda(e__, what);   \
    } while (0)

}  // namespace

int vnm::check_format(int M, int K, int V, int n, int m)
{
    if (n != 2) return fail(VNM_ERR_BAD_ARG, "n must be 2 (got %d)", n);
    if (m < 4) return fail(VNM_ERR_BAD_ARG, "m must be >= 4 (got %d)", m);
    if (M <= 0 || K <= 0 || V <= 0) return fail(VNM_ERR_BAD_ARG, "M, K, V must be positive (got %d, %d, %d)", M, K, V);
    if (V % 32 != 0) return fail(VNM_ERR_BAD_ARG, "V must be a multiple of 32 (got %d)", V);
    if (M % V != 0) return fail(VNM_ERR_BAD_ARG, "M (%d) must be a multiple of V (%d)", M, V);
    if ((int64_t)K + m >= (int64_t)1 << 30) return fail(VNM_ERR_BAD_ARG, "K too large");
    return VNM_OK;
}

vnm::EncodeTiledFn vnm::get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

namespace {

// cudaFuncSetAttribute (large dynamic shared memory) applies per device: one flag per device, set under a mutex.
constexpr int kMaxDevices = 64;
bool g_kernels_ready[kMaxDevices] = {};
std::mutex g_init_mutex;
int g_strategy = 0;  // VNM_STRATEGY_*

// Opts every kernel instance into its shared-memory size on the current device (once per device).
int ensure_kernels_ready(int *device_out)
{
    int dev = -1;
    VNM_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(VNM_ERR_UNSUPPORTED, "device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_init_mutex);
    if (!g_kernels_ready[dev]) {
        VNM_CUDA(spmm_init_kernels(), "cudaFuncSetAttribute(max dynamic shared memory)");
        VNM_CUDA(spmm_dense_b_init(), "cudaFuncSetAttribute(max dynamic shared memory)");
        VNM_CUDA(spmm_dense_b_pair_init(), "cudaFuncSetAttribute(max dynamic shared memory)");
        g_kernels_ready[dev] = true;
    }
    if (device_out) *device_out = dev;
    return VNM_OK;
}

// Gather form vs dense-B form (see vnm_set_strategy in the header).  Measured on B200: the gather path is
// bound by the TMA gather rate and pays NB = 128/V times for small vector lengths, the dense-B form costs
// m/4 times the MMA work but shares B between all vector blocks.
bool choose_dense_b(int K, int V, int m, int strategy)
{
    const bool possible = (m % 4 == 0) && (K % m == 0);
    if (!possible || strategy == VNM_STRATEGY_GATHER) return false;
    if (strategy == VNM_STRATEGY_DENSE_B) return true;
    // measured on B200 (N = 16384): the dense-B kernel wins for every V at m <= 8, at m = 16 for V <= 64 and at
    // m = 32 for V = 32 (the gather kernel gathers, and multiplies with masked MMAs, once per vector block of a row tile)
    if (m <= 8) return true;
    if (V <= 64 && m <= 16) return true;
    return V == 32 && m <= 32;
}

}  // namespace

constexpr int HOST_CHUNKS_MAX = 32;   // upper bound of vnm_set_host_slices

struct vnm_prepared_s {
    int M, K, V, n, m;
    int64_t Ksp;
    int mtiles, ktiles, nb, vblocks_padded;
    int device;
    void *am;
    void *rows;
    int *status;
    // cached TMA descriptors of the last dense operand: single rows (for gather4) and 64-row tiles
    const void *tm_B;
    int64_t tm_ldb;
    int tm_N;
    int tm_nk;
    int tm_pair;             // the cached maps are the pair kernel's (half stages)
    bool tm_valid;
    CUtensorMap tmap_rows;
    CUtensorMap tmap_tile;
    CUtensorMap tmap_tile2;  // dense-B kernel: 2-D map for the ragged right edge
    bool tm_wide;            // tmap_tile is the 4-D one-box-per-stage map
    int producer_warps;
    // device staging of the host-buffer entry point
    void *stage_B;
    size_t stage_B_bytes;
    void *stage_out;
    size_t stage_out_bytes;
    void *stage_bias;
    cudaStream_t copy_in, copy_out;   // host-buffer entry point: the device's two copy streams (shared by all handles)
    cudaEvent_t ev[2 * HOST_CHUNKS_MAX + 2];
    bool host_pipe_ready;
    int host_slices;   // column slices of the host-buffer pipeline (vnm_set_host_slices)
    int gather_mode;
    int dense_b;       // 1: A re-expressed as 2:4 over all K columns, B read as plain tiles
    int out32;         // ablation: 32-bit epilogue stores (gather form, layout MN)
    int hybrid_rows;   // gather form: rows of every 64-row stage fetched by TMA gather4 beside the per-thread copies
    int nm_tma_always; // gather kernel: 1 = the [N,M] result leaves through TMA stores even for a single destination (ablation: measured 1-4 % slower)
    int l2_ahead;      // pair kernel: k-tiles of L2 prefetch ahead of the shared-memory loads (0 = none)
    int pair_rows;     // pair kernel: 0 = row tiles per CTA chosen per problem, 1 / 2 = forced where possible (ablation)
    int l2_hints;      // pair kernel: 1 = ask L2 to keep the banded operand (default), 0 = no eviction-priority hints
    int pair_mode;     // dense-B form: 1 = use the two-SM (cta_group::2) kernel where it applies (default), 0 = never
    int max_ctas;      // 0 = one persistent CTA per SM, else the cap set by vnm_set_max_ctas
};

extern "C" {

const char *vnm_last_error_string(void) { return g_last_error.c_str(); }

int vnm_version(void) { return 100; }

int vnm_sizes(int M, int K, int V, int n, int m, int64_t *ksp, int64_t *values_elems, int64_t *meta_words, int64_t *colloc_words)
{
    int rc = check_format(M, K, V, n, m);
    if (rc) return rc;
    const int64_t Ksp = ksp_of(K, m);
    if (ksp) *ksp = Ksp;
    if (values_elems) *values_elems = (int64_t)M * Ksp;
    if (meta_words) *meta_words = (int64_t)(M / 2) * (Ksp / 8);
    if (colloc_words) *colloc_words = (int64_t)(M / V) * (Ksp / 2) * 4;
    return VNM_OK;
}

int vnm_compress_f16(const void *dense, int64_t ldd, const int32_t *mask, const uint32_t *colloc, int M, int K, int V, int n, int m,
                     void *values, uint32_t *meta, unsigned long long *violations, void *stream)
{
    int rc = check_format(M, K, V, n, m);
    if (rc) return rc;
    if (!dense || !colloc || !values || !meta) return fail(VNM_ERR_BAD_ARG, "vnm_compress_f16: null pointer");
    if (ldd < K) return fail(VNM_ERR_BAD_ARG, "vnm_compress_f16: ldd (%lld) < K (%d)", (long long)ldd, K);
    if (((uintptr_t)colloc & 15) || ((uintptr_t)values & 15)) return fail(VNM_ERR_BAD_ARG, "vnm_compress_f16: colloc/values must be 16-byte aligned");
    VNM_CUDA(launch_compress(dense, ldd, mask, colloc, M, K, V, m, values, meta, violations, (cudaStream_t)stream), "compress launch");
    return VNM_OK;
}

int vnm_prune_magnitude_f32(const float *w, int64_t ldw, int M, int K, int V, int n, int m, int32_t *mask, int64_t ldm, uint32_t *colloc,
                            void *stream)
{
    int rc = check_format(M, K, V, n, m);
    if (rc) return rc;
    if (!w || !mask || !colloc) return fail(VNM_ERR_BAD_ARG, "vnm_prune_magnitude_f32: null pointer");
    if (ldw < K || ldm < K) return fail(VNM_ERR_BAD_ARG, "vnm_prune_magnitude_f32: leading dimensions must be >= K");
    if (K % m != 0) return fail(VNM_ERR_UNSUPPORTED, "vnm_prune_magnitude_f32: K (%d) must be a multiple of m (%d)", K, m);
    if ((size_t)V * m * sizeof(float) > 48 * 1024) return fail(VNM_ERR_UNSUPPORTED, "vnm_prune_magnitude_f32: V * m too large (%d x %d)", V, m);
    VNM_CUDA(launch_prune(w, ldw, M, K, V, m, mask, ldm, colloc, (cudaStream_t)stream), "prune launch");
    return VNM_OK;
}

int vnm_decompress_f16(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int n, int m,
                       void *dense, int64_t ldd, void *stream)
{
    int rc = check_format(M, K, V, n, m);
    if (rc) return rc;
    if (!dense || !colloc || !values || !meta) return fail(VNM_ERR_BAD_ARG, "vnm_decompress_f16: null pointer");
    if (ldd < K) return fail(VNM_ERR_BAD_ARG, "vnm_decompress_f16: ldd (%lld) < K (%d)", (long long)ldd, K);
    VNM_CUDA(launch_decompress(values, meta, colloc, M, K, V, m, dense, ldd, (cudaStream_t)stream), "decompress launch");
    return VNM_OK;
}

int vnm_prepared_bytes(int M, int K, int V, int n, int m, int64_t *bytes)
{
    int rc = check_format(M, K, V, n, m);
    if (rc) return rc;
    if (V != 32 && V != 64 && V != 128) return fail(VNM_ERR_UNSUPPORTED, "SpMM supports V in {32, 64, 128} (got %d)", V);
    const int64_t Ksp = ksp_of(K, m);
    const bool dense_b = choose_dense_b(K, V, m, g_strategy);
    const int64_t mtiles = (M + TILE_M - 1) / TILE_M, ktiles = dense_b ? (K + 127) / 128 : (Ksp + KT_COMP - 1) / KT_COMP;
    const int64_t nb = dense_b ? 1 : TILE_M / V;
    if (bytes) *bytes = mtiles * ktiles * AM_BLOCK_BYTES + mtiles * nb * ktiles * KT_GROUPS * 16 + 256;
    return VNM_OK;
}

int vnm_prepare(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int n, int m,
                vnm_handle_t *handle, void *stream)
{
    return vnm_prepare_as(values, meta, colloc, M, K, V, n, m, g_strategy, handle, stream);
}

int vnm_prepare_as(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int n, int m, int strategy,
                   vnm_handle_t *handle, void *stream)
{
    if (strategy != VNM_STRATEGY_AUTO && strategy != VNM_STRATEGY_GATHER && strategy != VNM_STRATEGY_DENSE_B)
        return fail(VNM_ERR_BAD_ARG, "vnm_prepare_as: unknown strategy %d", strategy);
    int rc = check_format(M, K, V, n, m);
    if (rc) return rc;
    if (!values || !meta || !colloc || !handle) return fail(VNM_ERR_BAD_ARG, "vnm_prepare: null pointer");
    if (V != 32 && V != 64 && V != 128) return fail(VNM_ERR_UNSUPPORTED, "SpMM supports V in {32, 64, 128} (got %d)", V);
    if (((uintptr_t)colloc & 15) || ((uintptr_t)values & 3)) return fail(VNM_ERR_BAD_ARG, "vnm_prepare: colloc must be 16-byte and values 4-byte aligned");
    int dev_now = -1;
    if ((rc = ensure_kernels_ready(&dev_now))) return rc;
    vnm_prepared_s *h = new (std::nothrow) vnm_prepared_s();
    if (!h) return fail(VNM_ERR_CUDA, "out of host memory");
    memset(h, 0, sizeof(*h));
    h->M = M; h->K = K; h->V = V; h->n = n; h->m = m;
    h->Ksp = ksp_of(K, m);
    h->mtiles = (M + TILE_M - 1) / TILE_M;
    h->dense_b = choose_dense_b(K, V, m, strategy) ? 1 : 0;
    if (h->dense_b) {
        h->ktiles = (K + 127) / 128;  // a k-tile covers 128 original columns
        h->nb = 1;
        h->gather_mode = GATHER_CONTIG;
    } else {
        h->ktiles = (int)((h->Ksp + KT_COMP - 1) / KT_COMP);
        h->nb = TILE_M / V;
        h->gather_mode = (m == 4) ? GATHER_CONTIG : GATHER_TMA4;  // with m == 4 every row of B is selected
    }
    h->vblocks_padded = h->mtiles * h->nb;
    h->producer_warps = 8;
    h->pair_mode = 1;
    h->l2_hints = 1;
    h->device = dev_now;
    cudaError_t e = cudaMalloc(&h->am, (size_t)h->mtiles * h->ktiles * AM_BLOCK_BYTES);
    if (e == cudaSuccess) e = cudaMalloc(&h->rows, (size_t)h->vblocks_padded * h->ktiles * KT_GROUPS * sizeof(int4));
    if (e == cudaSuccess) e = cudaMalloc((void **)&h->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemsetAsync(h->status, 0, sizeof(int), (cudaStream_t)stream);
    if (e == cudaSuccess) {
        if (h->dense_b)
            e = launch_prepare_dense_b(values, meta, colloc, M, K, V, m, h->am, h->rows, h->mtiles, h->ktiles, (cudaStream_t)stream);
        else
            e = launch_prepare(values, meta, colloc, M, K, V, m, h->am, h->rows, h->mtiles, h->ktiles, h->vblocks_padded, (cudaStream_t)stream);
    }
    if (e != cudaSuccess) {
        vnm_destroy(h);
        return fail_cuda(e, "vnm_prepare");
    }
    *handle = h;
    return VNM_OK;
}

int vnm_destroy(vnm_handle_t h)
{
    if (!h) return VNM_OK;
    cudaFree(h->am);
    cudaFree(h->rows);
    cudaFree(h->status);
    cudaFree(h->stage_B);
    cudaFree(h->stage_out);
    cudaFree(h->stage_bias);
    if (h->host_pipe_ready) {
        for (cudaEvent_t e : h->ev) cudaEventDestroy(e);
    }
    delete h;
    return VNM_OK;
}

int vnm_set_gather_mode(vnm_handle_t h, int mode)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    if (mode != GATHER_TMA4 && mode != GATHER_CONTIG && mode != GATHER_NONE && mode != GATHER_CPASYNC) return fail(VNM_ERR_BAD_ARG, "unknown gather mode %d", mode);
    if (h->dense_b && (mode == GATHER_TMA4 || mode == GATHER_CPASYNC)) return fail(VNM_ERR_BAD_ARG, "this operand was prepared in dense-B form: it has no gather");
    h->gather_mode = mode;
    return VNM_OK;
}

int vnm_set_strategy(int strategy)
{
    if (strategy != VNM_STRATEGY_AUTO && strategy != VNM_STRATEGY_GATHER && strategy != VNM_STRATEGY_DENSE_B)
        return fail(VNM_ERR_BAD_ARG, "unknown strategy %d", strategy);
    g_strategy = strategy;
    return VNM_OK;
}

int vnm_set_gather_split(vnm_handle_t h, int tma_rows)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    if (tma_rows != 0 && tma_rows != 16 && tma_rows != 32 && tma_rows != 48) return fail(VNM_ERR_BAD_ARG, "tma_rows must be 0, 16, 32 or 48 (got %d)", tma_rows);
    h->hybrid_rows = tma_rows;
    return VNM_OK;
}

int vnm_set_pair_mode(vnm_handle_t h, int mode)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    if (mode < 0 || mode > 4) return fail(VNM_ERR_BAD_ARG, "pair mode must be 0 .. 4 (got %d)", mode);
    h->pair_mode = mode != 0;
    h->l2_hints = mode != 2;
    h->pair_rows = mode == 3 ? 1 : mode == 4 ? 2 : 0;
    return VNM_OK;
}

int vnm_set_host_slices(vnm_handle_t h, int slices)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "vnm_set_host_slices: null handle");
    if (slices < 0 || slices > HOST_CHUNKS_MAX) return fail(VNM_ERR_BAD_ARG, "vnm_set_host_slices: 0 .. %d slices (got %d)", HOST_CHUNKS_MAX, slices);
    h->host_slices = slices;
    return VNM_OK;
}

int vnm_set_l2_prefetch(vnm_handle_t h, int ktiles_ahead)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "vnm_set_l2_prefetch: null handle");
    if (ktiles_ahead < 0 || ktiles_ahead > 32) return fail(VNM_ERR_BAD_ARG, "vnm_set_l2_prefetch: 0 .. 32 k-tiles (got %d)", ktiles_ahead);
    h->l2_ahead = ktiles_ahead;
    return VNM_OK;
}

int vnm_set_epilogue(vnm_handle_t h, int mode)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    if (mode < 0 || mode > 2) return fail(VNM_ERR_BAD_ARG, "unknown epilogue mode %d", mode);
    if (mode != 0 && h->dense_b) return fail(VNM_ERR_UNSUPPORTED, "the alternative epilogues exist for the V:N:M (gather) form only; this operand is held in dense-B form");
    h->out32 = mode == 1;
    h->nm_tma_always = mode == 2;
    return VNM_OK;
}

int vnm_handle_info(vnm_handle_t h, int *M, int *K, int *V, int *m, int *max_ctas)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "vnm_handle_info: null handle");
    if (M) *M = h->M;
    if (K) *K = h->K;
    if (V) *V = h->V;
    if (m) *m = h->m;
    if (max_ctas) *max_ctas = h->max_ctas;
    return VNM_OK;
}

int vnm_set_max_ctas(vnm_handle_t h, int max_ctas)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    if (max_ctas < 0) return fail(VNM_ERR_BAD_ARG, "max_ctas must be >= 0 (got %d)", max_ctas);
    h->max_ctas = max_ctas;
    return VNM_OK;
}

int vnm_set_producer_warps(vnm_handle_t h, int warps)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    if (warps != 4 && warps != 8) return fail(VNM_ERR_BAD_ARG, "producer warps must be 4 or 8 (got %d)", warps);
    h->producer_warps = warps;
    return VNM_OK;
}

int vnm_spmm_config(vnm_handle_t h, int N, int *tile_m, int *tile_n, int *stages, int *grid, int *smem_bytes)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "null handle");
    SpmmConfig cfg;
    const bool pair = h->dense_b && h->pair_mode && N >= 128 && spmm_dense_b_pair_config(h->M, N, h->K, h->max_ctas, h->pair_rows, &cfg);
    if (pair) { /* cfg filled */ }
    else if (h->dense_b) spmm_dense_b_config(h->M, N, h->max_ctas, &cfg);
    else if (!spmm_select_config(h->V, N, h->M, h->producer_warps, h->max_ctas, &cfg)) return fail(VNM_ERR_UNSUPPORTED, "unsupported V");
    if (tile_m) *tile_m = h->dense_b ? cfg.nb * TILE_M : TILE_M;  // pairs: 512 or 256, one SM per tile: 256 or 128
    if (tile_n) *tile_n = cfg.bn;
    if (stages) *stages = cfg.stages;
    if (grid) *grid = cfg.grid;
    if (smem_bytes) *smem_bytes = cfg.smem_bytes;
    return VNM_OK;
}

static int spmm_impl(vnm_handle_t h, const void *B, int64_t ldb, int N, int b_nk, const void *bias, void *out, int64_t ldo, int layout,
                     void *stream, void *const *more_outs = nullptr, int n_more = 0)
{
    if (!h || !B || !out) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: null pointer");
    if (n_more < 0 || n_more > MAX_OUTS - 1 || (n_more > 0 && !more_outs))
        return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_multi: between 1 and %d destinations", MAX_OUTS);
    if (n_more > 0 && !h->dense_b && (layout != VNM_LAYOUT_NM || ldo % 8 != 0 || ((uintptr_t)out & 15)))
        return fail(VNM_ERR_UNSUPPORTED, "vnm_spmm_f16_multi: with an operand in gather form several destinations need layout NM, ldo %% 8 == 0 and "
                                         "16-byte aligned buffers (only that epilogue leaves through TMA stores)");
    for (int d = 0; d < n_more; d++)
        if (!more_outs[d] || ((uintptr_t)more_outs[d] & 15)) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_multi: destination %d is null or not 16-byte aligned", d + 1);
    {
        // the handle's private copy, its status word and the kernel attributes belong to one device
        int dev = -1;
        VNM_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
        if (dev != h->device)
            return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: the handle was prepared on device %d but device %d is current", h->device, dev);
    }
    if (N <= 0 || N % 8 != 0) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: N (%d) must be a positive multiple of 8", N);
    if (b_nk) {
        if (!h->dense_b) return fail(VNM_ERR_UNSUPPORTED, "a [N,K] dense operand needs an operand prepared in dense-B form (see vnm_operand_form)");
        if (ldb < h->K || ldb % 8 != 0) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_nk: ldb (%lld) must be >= K and a multiple of 8", (long long)ldb);
    } else if (ldb < N || ldb % 8 != 0) {
        return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: ldb (%lld) must be >= N and a multiple of 8", (long long)ldb);
    }
    if ((uintptr_t)B & 15) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: B must be 16-byte aligned");
    if (layout == VNM_LAYOUT_MN) {
        if (bias) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: bias is only supported with layout NM");
        if (ldo < N || ldo % 8 != 0 || ((uintptr_t)out & 15))
            return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: layout MN needs ldo >= N, ldo %% 8 == 0 and a 16-byte aligned out");
    } else if (layout == VNM_LAYOUT_NM) {
        if (ldo < h->M) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: layout NM needs ldo >= M");
    } else {
        return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: unknown layout %d", layout);
    }
    SpmmConfig cfg;
    const bool pair = h->dense_b && h->pair_mode && (b_nk || N >= 128) && spmm_dense_b_pair_config(h->M, N, h->K, h->max_ctas, h->pair_rows, &cfg);
    if (pair) { /* cfg filled */ }
    else if (h->dense_b) spmm_dense_b_config(h->M, N, h->max_ctas, &cfg);
    else if (!spmm_select_config(h->V, N, h->M, h->producer_warps, h->max_ctas, &cfg)) return fail(VNM_ERR_UNSUPPORTED, "unsupported V");
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(VNM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");

    if (!h->tm_valid || h->tm_B != B || h->tm_ldb != ldb || h->tm_N != N || h->tm_nk != b_nk || h->tm_pair != (pair ? 1 : 0)) {
        cuuint32_t estr[2] = {1, 1};
        CUresult r;
        if (b_nk) {
            // B given as [N, K] (K contiguous): one box of 32 k x 256 rows (n), written with the 64-byte swizzle,
            // is the K-major operand tile of one MMA (the last 16 rows belong to the next tile and are not read).
            cuuint64_t dims[2] = {(cuuint64_t)h->K, (cuuint64_t)N};
            cuuint64_t strides[1] = {(cuuint64_t)ldb * 2};
            // the pair kernel loads each CTA's 128-row half separately, 64 k (two MMA K blocks, 128-byte rows) per box
            cuuint32_t box[2] = {pair ? 64u : 32u, pair ? 128u : 256u};
            r = enc(&h->tmap_tile, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(B), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, pair ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            h->tmap_rows = h->tmap_tile;
            h->tmap_tile2 = h->tmap_tile;
            h->tm_wide = false;
        } else {
            // B viewed as a 2-D tensor {N (contiguous), K}; one box = 64 columns (128 bytes) of one row
            // (gather4 picks four such rows) or of 64 consecutive rows (32 for the dense-B kernel), written with
            // the 128-byte swizzle the MMA's N-major operand layout expects.  Rows >= K and columns >= N read as zeros.
            cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)h->K};
            cuuint64_t strides[1] = {(cuuint64_t)ldb * 2};
            cuuint32_t box_rows[2] = {64, 1};
            cuuint32_t box_tile[2] = {64, (h->dense_b && !pair) ? 32u : 64u};
            r = enc(&h->tmap_rows, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(B), dims, strides, box_rows, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r == CUDA_SUCCESS)
                r = enc(&h->tmap_tile, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(B), dims, strides, box_tile, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            h->tmap_tile2 = h->tmap_tile;
            h->tm_wide = false;
            if (r == CUDA_SUCCESS && pair) {
                // pair kernel: a CTA's half of a stage is {64 columns, 64 rows, 2 slices} starting at any multiple of 8 columns
                // (pair tiles start at multiples of 240, the peer's half 120 columns further)
                cuuint64_t dims4[4] = {64, (cuuint64_t)h->K, 2, (cuuint64_t)((N - 128) / 8 + 1)};
                cuuint64_t strides4[3] = {(cuuint64_t)ldb * 2, 128, 16};
                cuuint32_t box4[4] = {64, 64, 2, 1};
                cuuint32_t estr4[4] = {1, 1, 1, 1};
                CUtensorMap wide;
                if (enc(&wide, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(B), dims4, strides4, box4, estr4,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
                    h->tmap_tile = wide;
                    h->tm_wide = true;
                }
            } else if (r == CUDA_SUCCESS && h->dense_b && N >= 256) {
                // dense-B kernel: {64 columns, K rows, 4 slices of 64 columns, start column / 16}.  A box {64, 32, 4, 1}
                // lands as [slice][row][64 columns], the N-major operand tile of one MMA, with a single instruction.
                // Only start columns whose 256 columns lie inside N are addressable; the ragged edge uses the 2-D map.
                cuuint64_t dims4[4] = {64, (cuuint64_t)h->K, 4, (cuuint64_t)((N - 256) / 16 + 1)};
                cuuint64_t strides4[3] = {(cuuint64_t)ldb * 2, 128, 32};
                cuuint32_t box4[4] = {64, 32, 4, 1};
                cuuint32_t estr4[4] = {1, 1, 1, 1};
                CUtensorMap wide;
                if (enc(&wide, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(B), dims4, strides4, box4, estr4,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
                    h->tmap_tile = wide;
                    h->tm_wide = true;
                }
            }
        }
        if (r != CUDA_SUCCESS) return fail(VNM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        h->tm_B = B; h->tm_ldb = ldb; h->tm_N = N; h->tm_nk = b_nk; h->tm_pair = pair ? 1 : 0; h->tm_valid = true;
    }

    SpmmParams p;
    p.am = (const uint8_t *)h->am;
    p.rows = (const int4 *)h->rows;
    p.bias = (const __half *)bias;
    p.out = (__half *)out;
    p.ldo = ldo;
    p.M = h->M; p.N = N; p.K = h->K; p.V = h->V;
    p.mtiles = h->mtiles; p.ktiles = h->ktiles; p.ntiles = (N + cfg.bn - 1) / cfg.bn;
    p.layout = layout;
    p.status = h->status;
    p.gather_mode = h->gather_mode;
    p.total_tiles = p.mtiles * p.ntiles;
    p.B = (const __half *)B;
    p.ldb = ldb;
    p.out32 = h->out32;
    {
        // Band of the tile order (tile_coords) and, for the pair kernel, which operand is asked to stay in L2.  A band
        // keeps either `g` row groups of A (18 KiB per row tile and k-tile) or `q` column panels of B (K x tile-N fp16)
        // within about 32 MB while the other operand streams past; the cheaper of the two in bytes re-read from HBM wins:
        //   row bands: A once + B once per band;   column bands: B once + A once per band.
        const int64_t rows_per_group = h->dense_b ? (int64_t)cfg.nb * TILE_M : TILE_M;   // dense-B: 256 / 128 (one SM per tile) or 512 (pairs); gather: 128
        const int64_t row_groups = (h->M + rows_per_group - 1) / rows_per_group;
        const int64_t bytes_per_group = (rows_per_group / TILE_M) * (int64_t)h->ktiles * AM_BLOCK_BYTES;
        const int64_t bytes_per_panel = (int64_t)h->K * cfg.bn * 2;
        const int64_t budget = (int64_t)32 << 20;  // measured flat between 28 and 64 MB on B200, worse at 16 and 96
        int64_t g = bytes_per_group > 0 ? budget / bytes_per_group : 1;
        g = g < 1 ? 1 : (g > 4096 ? 4096 : g);
        int64_t q = bytes_per_panel > 0 ? budget / bytes_per_panel : 1;
        q = q < 1 ? 1 : (q > 4096 ? 4096 : q);
        const double a_total = (double)row_groups * bytes_per_group, b_total = (double)p.ntiles * bytes_per_panel;
        const double cost_rows = a_total + b_total * (double)((row_groups + g - 1) / g);
        const double cost_cols = b_total + a_total * (double)((p.ntiles + q - 1) / q);
        const bool col_bands = pair && cost_cols < cost_rows;   // the one-SM and gather kernels keep row bands
        p.group_m = col_bands ? -(int)q : (int)g;
        p.hint_a = col_bands ? L2_EVICT_NORMAL : L2_EVICT_LAST;
        p.hint_b = col_bands ? L2_EVICT_LAST : L2_EVICT_NORMAL;
        if (h->l2_hints == 0) p.hint_a = p.hint_b = L2_EVICT_NORMAL;
    }
    p.hybrid_rows = h->hybrid_rows;
    p.b_nk = b_nk;
    p.b_wide_ok = h->tm_wide ? 1 : 0;
    p.l2_ahead = h->l2_ahead;
    p.n_out = 1;
    p.nm_tma = 0;
    if (h->dense_b) {
        // The result leaves through TMA stores: [M,N] as boxes of 40 columns x 128 rows, [N,M] as boxes of 128
        // columns (m) x 40 rows (n).
        if (layout == VNM_LAYOUT_NM && (ldo % 8 != 0 || ((uintptr_t)out & 15)))
            return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16: layout NM needs ldo %% 8 == 0 and a 16-byte aligned out for this operand");
        CUtensorMap tmap_out;
        OutMaps more;
        memset(&more, 0, sizeof(more));
        cuuint32_t oestr[2] = {1, 1};
        cuuint64_t ostrides[1] = {(cuuint64_t)ldo * 2};
        cuuint64_t odims[2] = {(cuuint64_t)N, (cuuint64_t)h->M};
        cuuint32_t obox[2] = {40, 128};
        if (layout == VNM_LAYOUT_NM) {
            odims[0] = (cuuint64_t)h->M; odims[1] = (cuuint64_t)N;
            obox[0] = 128; obox[1] = 40;
        }
        for (int d = 0; d <= n_more; d++) {
            CUresult r = enc(d == 0 ? &tmap_out : &more.m[d - 1], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d == 0 ? out : more_outs[d - 1], odims, ostrides, obox,
                             oestr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(VNM_ERR_CUDA, "cuTensorMapEncodeTiled (output %d) failed with CUresult %d", d, (int)r);
        }
        p.n_out = 1 + n_more;
        if (pair) VNM_CUDA(launch_spmm_dense_b_pair(cfg, h->tmap_tile, h->tmap_tile2, tmap_out, more, p, (cudaStream_t)stream), "spmm launch");
        else VNM_CUDA(launch_spmm_dense_b(cfg, h->tmap_tile, h->tmap_tile2, tmap_out, more, p, (cudaStream_t)stream), "spmm launch");
    } else {
        // Gather form: the epilogue stores from registers.  Only a [N,M] result with several destinations (or on request)
        // leaves through shared memory and TMA stores (boxes of 128 m x 32 n; needs ldo % 8 == 0 and 16-byte alignment):
        // for a single destination that path measured 1-4 % slower.
        CUtensorMap tmap_out;
        OutMaps more;
        memset(&tmap_out, 0, sizeof(tmap_out));
        memset(&more, 0, sizeof(more));
        p.nm_tma = 0;
        if (layout == VNM_LAYOUT_NM && ldo % 8 == 0 && ((uintptr_t)out & 15) == 0 && (n_more > 0 || h->nm_tma_always)) {
            cuuint32_t oestr[2] = {1, 1};
            cuuint64_t ostrides[1] = {(cuuint64_t)ldo * 2};
            cuuint64_t odims[2] = {(cuuint64_t)h->M, (cuuint64_t)N};
            cuuint32_t obox[2] = {128, 32};
            for (int d = 0; d <= n_more; d++) {
                CUresult r = enc(d == 0 ? &tmap_out : &more.m[d - 1], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d == 0 ? out : more_outs[d - 1], odims, ostrides, obox,
                                 oestr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r != CUDA_SUCCESS) return fail(VNM_ERR_CUDA, "cuTensorMapEncodeTiled (output %d) failed with CUresult %d", d, (int)r);
            }
            p.nm_tma = 1;
            p.n_out = 1 + n_more;
        } else if (n_more > 0) {
            return fail(VNM_ERR_UNSUPPORTED, "vnm_spmm_f16_multi: the register-store epilogue of the gather form writes one destination");
        }
        VNM_CUDA(launch_spmm(cfg, h->tmap_rows, h->tmap_tile, tmap_out, more, p, (cudaStream_t)stream), "spmm launch");
    }
    return VNM_OK;
}

int vnm_spmm_f16(vnm_handle_t h, const void *B, int64_t ldb, int N, const void *bias, void *out, int64_t ldo, int layout, void *stream)
{
    return spmm_impl(h, B, ldb, N, 0, bias, out, ldo, layout, stream);
}

int vnm_spmm_f16_nk(vnm_handle_t h, const void *Bt, int64_t ldbt, int N, const void *bias, void *out, int64_t ldo, int layout, void *stream)
{
    return spmm_impl(h, Bt, ldbt, N, 1, bias, out, ldo, layout, stream);
}

int vnm_spmm_f16_multi(vnm_handle_t h, const void *B, int64_t ldb, int N, const void *bias, void *const *outs, int n_outs, int64_t ldo, int layout,
                       void *stream)
{
    if (!outs || n_outs < 1 || n_outs > MAX_OUTS) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_multi: between 1 and %d destinations", MAX_OUTS);
    return spmm_impl(h, B, ldb, N, 0, bias, outs[0], ldo, layout, stream, outs + 1, n_outs - 1);
}

int vnm_operand_form(vnm_handle_t h, int *dense_b)
{
    if (!h || !dense_b) return fail(VNM_ERR_BAD_ARG, "vnm_operand_form: null pointer");
    *dense_b = h->dense_b;
    return VNM_OK;
}

static int grow(void **buf, size_t *cap, size_t need)
{
    if (*cap >= need) return VNM_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr; *cap = 0;
    cudaError_t e = cudaMalloc(buf, need);
    if (e != cudaSuccess) return fail_cuda(e, "staging cudaMalloc");
    *cap = need;
    return VNM_OK;
}

static int spmm_host_impl(vnm_handle_t h, const void *B_host, int N, const void *bias_host, void *out_host, int layout, void *stream, bool wait)
{
    if (!h || !B_host || !out_host) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_host: null pointer");
    if (N <= 0 || N % 8 != 0) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_host: N (%d) must be a positive multiple of 8", N);
    if (layout != VNM_LAYOUT_MN && layout != VNM_LAYOUT_NM) return fail(VNM_ERR_BAD_ARG, "vnm_spmm_f16_host: unknown layout %d", layout);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t b_bytes = (size_t)h->K * N * 2, o_bytes = (size_t)h->M * N * 2;
    int rc;
    if ((rc = grow(&h->stage_B, &h->stage_B_bytes, b_bytes))) return rc;
    if ((rc = grow(&h->stage_out, &h->stage_out_bytes, o_bytes))) return rc;
    if (!h->host_pipe_ready) {
        // One upload and one download stream per device for every handle: with a pair of streams per handle
        // the driver multiplexes them onto a few hardware queues and unrelated copies end up waiting for each other.
        static std::mutex mu;
        static cudaStream_t up[64], down[64];
        {
            std::lock_guard<std::mutex> lock(mu);
            const int dev = h->device >= 0 && h->device < 64 ? h->device : 0;
            if (!up[dev]) {
                VNM_CUDA(cudaStreamCreateWithFlags(&up[dev], cudaStreamNonBlocking), "cudaStreamCreate");
                VNM_CUDA(cudaStreamCreateWithFlags(&down[dev], cudaStreamNonBlocking), "cudaStreamCreate");
            }
            h->copy_in = up[dev];
            h->copy_out = down[dev];
        }
        for (cudaEvent_t &e : h->ev) VNM_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        h->host_pipe_ready = true;
    }
    // The columns are cut into slices of a multiple of 256 columns.  Slice c+1 goes up (copy engine 1) while slice c is
    // multiplied and slice c-1 comes down (copy engine 2), so the call costs about the larger of the two transfers
    // instead of their sum.  On the device every slice is its own compact matrix, [K, w] in and [M, w] or [w, M] out.
    // Equal slices, eight by default (vnm_set_host_slices).  Measured on cfg4: a schedule of growing slices (short head, long
    // rows for the later 2-D copies) changes nothing; the [M, N] result costs 70-72 ms with 4-16 slices against 60-63 ms
    // for the [N, M] result, whose slices come down as plain 1-D copies.
    int widths[HOST_CHUNKS_MAX];
    int chunks = 0;
    {
        const int slices = h->host_slices > 0 ? h->host_slices : 8;
        int nc = ((N + slices - 1) / slices + 255) / 256 * 256;
        if (nc < 1024) nc = 1024;
        for (int n0 = 0; n0 < N; n0 += nc) widths[chunks++] = N - n0 < nc ? N - n0 : nc;
    }
    cudaEvent_t ev_start = h->ev[2 * HOST_CHUNKS_MAX], ev_done = h->ev[2 * HOST_CHUNKS_MAX + 1];
    VNM_CUDA(cudaEventRecord(ev_start, s), "event record");
    VNM_CUDA(cudaStreamWaitEvent(h->copy_in, ev_start, 0), "stream wait");
    VNM_CUDA(cudaStreamWaitEvent(h->copy_out, ev_start, 0), "stream wait");
    if (bias_host) {
        if (!h->stage_bias) VNM_CUDA(cudaMalloc(&h->stage_bias, (size_t)h->M * 2), "bias cudaMalloc");
        VNM_CUDA(cudaMemcpyAsync(h->stage_bias, bias_host, (size_t)h->M * 2, cudaMemcpyHostToDevice, h->copy_in), "H2D copy of bias");
    }
    for (int c = 0, n0 = 0; c < chunks; n0 += widths[c], ++c) {
        const int w = widths[c];
        uint8_t *dB = (uint8_t *)h->stage_B + (size_t)h->K * n0 * 2;
        uint8_t *dO = (uint8_t *)h->stage_out + (size_t)h->M * n0 * 2;
        VNM_CUDA(cudaMemcpy2DAsync(dB, (size_t)w * 2, (const uint8_t *)B_host + (size_t)n0 * 2, (size_t)N * 2, (size_t)w * 2, h->K,
                                   cudaMemcpyHostToDevice, h->copy_in), "H2D copy of B");
        VNM_CUDA(cudaEventRecord(h->ev[2 * c], h->copy_in), "event record");
        VNM_CUDA(cudaStreamWaitEvent(s, h->ev[2 * c], 0), "stream wait");
        rc = vnm_spmm_f16(h, dB, w, w, bias_host ? h->stage_bias : nullptr, dO, layout == VNM_LAYOUT_MN ? w : h->M, layout, stream);
        if (rc) break;
        VNM_CUDA(cudaEventRecord(h->ev[2 * c + 1], s), "event record");
        VNM_CUDA(cudaStreamWaitEvent(h->copy_out, h->ev[2 * c + 1], 0), "stream wait");
        if (layout == VNM_LAYOUT_MN)
            VNM_CUDA(cudaMemcpy2DAsync((uint8_t *)out_host + (size_t)n0 * 2, (size_t)N * 2, dO, (size_t)w * 2, (size_t)w * 2, h->M,
                                       cudaMemcpyDeviceToHost, h->copy_out), "D2H copy of the result");
        else
            VNM_CUDA(cudaMemcpyAsync((uint8_t *)out_host + (size_t)h->M * n0 * 2, dO, (size_t)h->M * w * 2, cudaMemcpyDeviceToHost, h->copy_out),
                     "D2H copy of the result");
    }
    if (!wait) return rc;  // the caller collects the result with vnm_host_wait
    // join both copy streams back into the caller's stream, also on the error path, before returning
    cudaEventRecord(ev_done, h->copy_out);
    cudaStreamWaitEvent(s, ev_done, 0);
    cudaEventRecord(ev_start, h->copy_in);
    cudaStreamWaitEvent(s, ev_start, 0);
    cudaError_t e = cudaStreamSynchronize(s);
    if (rc) return rc;
    VNM_CUDA(e, "stream synchronize");
    return VNM_OK;
}

int vnm_spmm_f16_host(vnm_handle_t h, const void *B_host, int N, const void *bias_host, void *out_host, int layout, void *stream)
{
    return spmm_host_impl(h, B_host, N, bias_host, out_host, layout, stream, true);
}

int vnm_spmm_f16_host_async(vnm_handle_t h, const void *B_host, int N, const void *bias_host, void *out_host, int layout, void *stream)
{
    return spmm_host_impl(h, B_host, N, bias_host, out_host, layout, stream, false);
}

int vnm_host_wait(vnm_handle_t h)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "vnm_host_wait: null handle");
    if (!h->host_pipe_ready) return VNM_OK;
    VNM_CUDA(cudaStreamSynchronize(h->copy_in), "stream synchronize");
    VNM_CUDA(cudaStreamSynchronize(h->copy_out), "stream synchronize");
    return VNM_OK;
}

int vnm_selftest_wait_expiry(vnm_handle_t h, void *stream)
{
    if (!h) return fail(VNM_ERR_BAD_ARG, "vnm_selftest_wait_expiry: null handle");
    VNM_CUDA(launch_wait_expiry_selftest(h->status, (cudaStream_t)stream), "self-test launch");
    return VNM_OK;
}

int vnm_device_status(vnm_handle_t h, int *status, void *stream)
{
    if (!h || !status) return fail(VNM_ERR_BAD_ARG, "vnm_device_status: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    int v = 0;
    VNM_CUDA(cudaMemcpyAsync(&v, h->status, sizeof(int), cudaMemcpyDeviceToHost, s), "status copy");
    VNM_CUDA(cudaStreamSynchronize(s), "stream synchronize");
    if (v != 0) VNM_CUDA(cudaMemsetAsync(h->status, 0, sizeof(int), s), "status clear");
    *status = v;
    if (v != 0) return fail(VNM_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (status bits 0x%x)", v);
    return VNM_OK;
}

}  // extern "C"
