// vnm_spmm_f16_noalloc: the V:N:M product for callers that must not allocate device memory.
//
// The regular path (vnm_prepare + vnm_spmm_f16) keeps a re-packed copy of the sparse operand in memory it
// gets from cudaMalloc.  Some callers cannot do that: a serving process whose framework has already claimed
// the whole device for its own pool, a plug-in that runs inside somebody else's memory budget, or a
// latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply.
// For them this file keeps the re-packed operand in a fixed array that is part of the library image:
// every GPU that loads the library carries VNM_NOALLOC_SCRATCH_BYTES of it until the process exits.
//
// Host code must not pass the array's name to a kernel -- on the host that name is only a stand-in for the
// symbol, not a device address.  The device address is looked up once per device with
// cudaGetSymbolAddress (while that device is current) and that pointer is what the kernels receive.
#include "../../include/venom_b200.h"
#include "vnm_internal.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

using namespace vnm;

namespace {

// Scratch of the no-allocation entry point: [0,256) status word and padding, then the value/metadata
// blocks, then the row table.  Shared by every call on the device; contents persist between calls.
static __device__ __align__(256) unsigned char g_noalloc_scratch[VNM_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
constexpr size_t kHeaderBytes = 256;

struct DeviceState {
    bool ready = false;
    unsigned char *scratch = nullptr;  // device address of g_noalloc_scratch on this device
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mutex;

}  // namespace

static int nfail(int code, const char *fmt, ...)
{
    // Reports like every other entry point (return code + vnm_last_error_string()) and, because the callers of
    // this variant often run where nobody polls an error string, with one line on stderr as well.
    char msg[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    fprintf(stderr, "vnm_spmm_f16_noalloc: %s\n", msg);
    return set_last_error(code, msg);
}

extern "C" int vnm_spmm_f16_noalloc(const void *values, const uint32_t *meta, const uint32_t *colloc, int M, int K, int V, int n, int m,
                                    const void *B, int64_t ldb, int N, const void *bias, void *out, int64_t ldo, int layout, void *stream)
{
    if (!values || !meta || !colloc || !B || !out) return nfail(VNM_ERR_BAD_ARG, "null pointer");
    if (int rc = check_format(M, K, V, n, m)) return nfail(rc, "%s", vnm_last_error_string());  // same format limits as every other entry point
    if (V != 32 && V != 64 && V != 128) return nfail(VNM_ERR_UNSUPPORTED, "V must be 32, 64 or 128 (got %d)", V);
    if (N <= 0 || N % 8 != 0) return nfail(VNM_ERR_BAD_ARG, "N (%d) must be a positive multiple of 8", N);
    if (ldb < N || ldb % 8 != 0 || ((uintptr_t)B & 15)) return nfail(VNM_ERR_BAD_ARG, "B needs ldb >= N, ldb %% 8 == 0 and a 16-byte aligned base");
    if (((uintptr_t)colloc & 15) || ((uintptr_t)values & 3)) return nfail(VNM_ERR_BAD_ARG, "colloc must be 16-byte and values 4-byte aligned");
    if (layout == VNM_LAYOUT_MN) {
        if (bias) return nfail(VNM_ERR_BAD_ARG, "bias is only supported with layout NM");
        if (ldo < N || ldo % 8 != 0 || ((uintptr_t)out & 15)) return nfail(VNM_ERR_BAD_ARG, "layout MN needs ldo >= N, ldo %% 8 == 0, 16-byte aligned out");
    } else if (layout == VNM_LAYOUT_NM) {
        if (ldo < M) return nfail(VNM_ERR_BAD_ARG, "layout NM needs ldo >= M");
    } else {
        return nfail(VNM_ERR_BAD_ARG, "unknown layout %d", layout);
    }

    const int64_t Ksp = ksp_of(K, m);
    const int mtiles = (M + TILE_M - 1) / TILE_M;
    const int ktiles = (int)((Ksp + KT_COMP - 1) / KT_COMP);
    const int nb = TILE_M / V;
    const int vblocks_padded = mtiles * nb;
    const size_t am_bytes = (size_t)mtiles * ktiles * AM_BLOCK_BYTES;
    const size_t rows_bytes = (size_t)vblocks_padded * ktiles * KT_GROUPS * sizeof(int4);
    const size_t need = kHeaderBytes + am_bytes + rows_bytes;
    if (need > (size_t)VNM_NOALLOC_SCRATCH_BYTES)
        return nfail(VNM_ERR_UNSUPPORTED,
                     "sparse operand too large for the built-in scratch: its re-packed form needs %zu bytes, the limit is %d "
                     "(use vnm_prepare + vnm_spmm_f16 instead)", need, (int)VNM_NOALLOC_SCRATCH_BYTES);

    // ---- once per device: function attributes and the device address of the scratch array ----
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return nfail(VNM_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return nfail(VNM_ERR_UNSUPPORTED, "device index %d not supported", dev);
    unsigned char *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState &st = g_dev[dev];
        if (!st.ready) {
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // `dev` is current here
            if (e != cudaSuccess || p == nullptr) return nfail(VNM_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
            e = spmm_init_kernels();
            if (e != cudaSuccess) return nfail(VNM_ERR_CUDA, "kernel set-up: %s", cudaGetErrorString(e));
            st.scratch = (unsigned char *)p;
            st.ready = true;
        }
        scratch = st.scratch;
    }
    cudaStream_t s = (cudaStream_t)stream;
    int *status = (int *)scratch;
    void *am = scratch + kHeaderBytes;
    void *rows = scratch + kHeaderBytes + am_bytes;

    // The array still holds the previous call's data: the status word must start at zero; the blocks and
    // the row table are fully rewritten by the re-pack below.
    e = cudaMemsetAsync(status, 0, kHeaderBytes, s);
    if (e != cudaSuccess) return nfail(VNM_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    e = launch_prepare(values, meta, colloc, M, K, V, m, am, rows, mtiles, ktiles, vblocks_padded, s);
    if (e != cudaSuccess) return nfail(VNM_ERR_CUDA, "re-pack launch: %s", cudaGetErrorString(e));

    SpmmConfig cfg;
    if (!spmm_select_config(V, N, M, 8, 0, &cfg)) return nfail(VNM_ERR_UNSUPPORTED, "unsupported V");
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return nfail(VNM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap tmap_rows, tmap_tile;
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
    cuuint64_t strides[1] = {(cuuint64_t)ldb * 2};
    cuuint32_t box_rows[2] = {64, 1}, box_tile[2] = {64, 64}, estr[2] = {1, 1};
    CUresult r = enc(&tmap_rows, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(B), dims, strides, box_rows, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS)
        r = enc(&tmap_tile, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(B), dims, strides, box_tile, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return nfail(VNM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);

    SpmmParams p;
    p.n_out = 1;
    p.l2_ahead = 0;
    p.nm_tma = 0;
    p.am = (const uint8_t *)am;
    p.rows = (const int4 *)rows;
    p.bias = (const __half *)bias;
    p.out = (__half *)out;
    p.ldo = ldo;
    p.M = M; p.N = N; p.K = K; p.V = V;
    p.mtiles = mtiles; p.ktiles = ktiles; p.ntiles = (N + cfg.bn - 1) / cfg.bn;
    p.layout = layout;
    p.status = status;
    p.gather_mode = (m == 4) ? GATHER_CONTIG : GATHER_TMA4;
    p.total_tiles = p.mtiles * p.ntiles;
    p.B = (const __half *)B;
    p.ldb = ldb;
    p.out32 = 0;
    p.hint_a = p.hint_b = L2_EVICT_NORMAL;
    p.group_m = mtiles;  // operands this small fit in L2 whole: row tiles fastest
    p.hybrid_rows = 0;
    p.b_nk = 0;
    p.b_wide_ok = 0;
    {
        CUtensorMap no_map;   // this entry point keeps the register-store epilogue: no output tensor maps
        OutMaps no_maps;
        memset(&no_map, 0, sizeof(no_map));
        memset(&no_maps, 0, sizeof(no_maps));
        e = launch_spmm(cfg, tmap_rows, tmap_tile, no_map, no_maps, p, s);
    }
    if (e != cudaSuccess) return nfail(VNM_ERR_CUDA, "product launch: %s", cudaGetErrorString(e));

    // The status word lives in the shared scratch, so it is read back before the next call can clear it.
    int v = 0;
    e = cudaMemcpyAsync(&v, status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return nfail(VNM_ERR_CUDA, "completion: %s", cudaGetErrorString(e));
    if (v != 0) return nfail(VNM_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (status bits 0x%x)", v);
    return VNM_OK;
}
