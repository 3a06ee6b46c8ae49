// benchmark_spmm: command-line driver with the flag set and the CSV line of the reference's
// src/benchmark_spmm.cpp (flags: src/util/argparse.h:26-55,68-175; output: src/benchmark_spmm.cpp:181),
// running the sm_100a library through its C ABI.
//
//   benchmark_spmm --sparsity-type n-to-m --spmm spatha --gemm cuBlas --precision half
//       --meta-block-size 32 --block-size 4 --nn_row 2 --mm_row 8 --m 1024 --k 4096 --n 4096 --d 0.5
//       --bm 64 --bn 64 --bk 32 --wm 32 --wn 64 --wk 32 --mm 16 --mn 8 --mk 32 --nstage 2 [--random] [--check]
//
// --bm keeps its meaning (the vector length V); the other tile flags (--bn .. --nstage) are accepted and
// echoed in the CSV line but do not select kernels: the library picks its own tile per V.
// stdout: the reference's 24 columns
//   spmm_code,arch,m,k,n,meta_block_sz,block_sz,nn_row,mm_row,density,bm,bn,bk,wm,wn,wk,mm,mn,mk,nstage,
//   spmm_time,gemm_time,speedup,error
// followed by useful_tflops,hbm_gbs (algorithmic bytes / time).
// Timing protocol of the reference (src/spmm/spatha_spmm.cpp:67-72, src/cuda_utils.h:60-87): 1 + 10
// warm-up launches, then the mean of 100 launches between two CUDA events.
// Operands follow the reference's own instance generator (Format_sr_nm<T>::init / random_mask,
// src/format/format_sr_nm.cpp:31-75,151-237): per (row, group) two ascending random positions out of four,
// per (V-block, group) four ascending random column offsets out of m, values and B uniform integers in
// [-4, 4] (src/util/matrix_utils.h:93), so that every product and sum is exact and --check can use the
// reference's |a - b| <= 1.0 rule (src/benchmark_spmm.cpp:58).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cublas_v2.h>
#include <cuda_profiler_api.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "../../include/venom_b200.h"

#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e__ = (call);                                                                  \
        if (e__ != cudaSuccess) {                                                                  \
            fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e__), __FILE__, __LINE__); \
            return 2;                                                                              \
        }                                                                                          \
    } while (0)
#define VK(call)                                                                       \
    do {                                                                               \
        int r__ = (call);                                                              \
        if (r__ != 0) {                                                                \
            fprintf(stderr, "venom_b200 error %d: %s\n", r__, vnm_last_error_string()); \
            return 2;                                                                  \
        }                                                                              \
    } while (0)

static const char *kUsage =
    "Required: --sparsity-type n-to-m --spmm spatha --gemm cuBlas --precision half --m M --k K --n N --d D\n"
    "          --nn_row 2 --mm_row m --bm V [--meta-block-size 32] [--block-size 4]\n"
    "Accepted and echoed: --bn --bk --wm --wn --wk --mm --mn --mk --nstage --acc_t fp32\n"
    "Optional: --random (time-based seed), --check (compare with cuBLAS on the decompressed matrix)\n"
    "          --strategy auto|gather|dense-b   operand form (default auto: chosen per V and m)\n"
    "          --ablation none|ideal|no-b|cpasync|out32\n"
    "                                          ideal: gather form without column-loc (plain row tiles of B, the\n"
    "                                          reference's IDEAL_KERNEL build; results differ unless m = 4);\n"
    "                                          no-b: no loads of B at all (timing floor of the pipeline);\n"
    "                                          cpasync: rows gathered by per-thread cp.async copies instead of TMA tile::gather4;\n"
    "                                          out32: 32-bit epilogue stores (the reference's OUT_32B build)\n";

int main(int argc, const char **argv)
{
    int m = 0, n = 0, k = 0, bm = 0, bn = 0, bk = 0, wm = 0, wn = 0, wk = 0, mm = 0, mn = 0, mk = 0, nstage = 0, nn_row = 0, mm_row = 0;
    int block_sz = 1, meta_block_sz = 0, spmm_code = -1, gemm_code = -1, pattern_code = -1, precision_code = -1;
    float density = 0.f;
    unsigned seed = 2022;
    bool check = false;
    int strategy = VNM_STRATEGY_AUTO, ablation = 0;
    for (int i = 1; i < argc; ++i) {
        auto is = [&](const char *f) { return !strcmp(argv[i], f); };
        const bool has = i != argc - 1;
        if (is("--m") && has) m = atoi(argv[i + 1]);
        else if (is("--n") && has) n = atoi(argv[i + 1]);
        else if (is("--k") && has) k = atoi(argv[i + 1]);
        else if (is("--d") && has) density = (float)atof(argv[i + 1]);
        else if (is("--bm") && has) bm = atoi(argv[i + 1]);
        else if (is("--bn") && has) bn = atoi(argv[i + 1]);
        else if (is("--bk") && has) bk = atoi(argv[i + 1]);
        else if (is("--wm") && has) wm = atoi(argv[i + 1]);
        else if (is("--wn") && has) wn = atoi(argv[i + 1]);
        else if (is("--wk") && has) wk = atoi(argv[i + 1]);
        else if (is("--mm") && has) mm = atoi(argv[i + 1]);
        else if (is("--mn") && has) mn = atoi(argv[i + 1]);
        else if (is("--mk") && has) mk = atoi(argv[i + 1]);
        else if (is("--nstage") && has) nstage = atoi(argv[i + 1]);
        else if (is("--nn_row") && has) nn_row = atoi(argv[i + 1]);
        else if (is("--mm_row") && has) mm_row = atoi(argv[i + 1]);
        else if (is("--block-size") && has) block_sz = atoi(argv[i + 1]);
        else if (is("--meta-block-size") && has) meta_block_sz = atoi(argv[i + 1]);
        else if (is("--spmm") && has) spmm_code = !strcmp(argv[i + 1], "spatha") ? 2 : -2;
        else if (is("--gemm") && has) gemm_code = (!strcmp(argv[i + 1], "cuBlas") || !strcmp(argv[i + 1], "cuBlasLt")) ? 0 : -1;
        else if (is("--sparsity-type") && has) pattern_code = !strcmp(argv[i + 1], "n-to-m") ? 2 : -2;
        else if (is("--precision") && has) precision_code = !strcmp(argv[i + 1], "half") ? 1 : -2;
        else if (is("--check")) check = true;
        else if (is("--strategy") && has) strategy = !strcmp(argv[i + 1], "gather") ? VNM_STRATEGY_GATHER : (!strcmp(argv[i + 1], "dense-b") ? VNM_STRATEGY_DENSE_B : VNM_STRATEGY_AUTO);
        else if (is("--ablation") && has) ablation = !strcmp(argv[i + 1], "ideal") ? 1 : !strcmp(argv[i + 1], "no-b") ? 2 : !strcmp(argv[i + 1], "cpasync") ? 3 : !strcmp(argv[i + 1], "out32") ? 4 : 0;
        else if (is("--random")) seed = (unsigned)std::chrono::system_clock::now().time_since_epoch().count();
    }
    if (m == 0 || n == 0 || k == 0 || density == 0.f) {
        fprintf(stderr, "%sForget to set m,n,k,density?\n", kUsage);
        return EXIT_FAILURE;
    }
    if (pattern_code != 2 || spmm_code != 2 || precision_code != 1 || gemm_code != 0) {
        fprintf(stderr, "%sOnly --sparsity-type n-to-m --spmm spatha --gemm cuBlas --precision half are built here.\n", kUsage);
        return EXIT_FAILURE;
    }
    if (meta_block_sz == 0) meta_block_sz = 32;
    if (nn_row == 0) nn_row = 2;
    const int V = bm, M = m, K = k, N = n, mrow = mm_row;

    int64_t ksp = 0, nv = 0, nmeta = 0, ncol = 0;
    VK(vnm_sizes(M, K, V, nn_row, mrow, &ksp, &nv, &nmeta, &ncol));

    // ---- instance (host) ----
    std::mt19937 rng(seed);
    std::vector<__half> hval((size_t)nv);
    std::vector<uint32_t> hmeta((size_t)nmeta, 0u), hcol((size_t)ncol, 0u);
    std::vector<__half> hB((size_t)K * N);
    auto rnd9 = [&]() { return (float)((int)(rng() % 9u) - 4); };
    for (auto &v : hval) v = __float2half(rnd9());
    for (auto &v : hB) v = __float2half(rnd9());
    for (auto &w : hmeta) {
        uint32_t word = 0;
        for (int g = 0; g < 8; ++g) {  // 8 nibbles = 2 rows x 4 groups
            int a = (int)(rng() % 4u), b = (int)(rng() % 3u);
            if (b >= a) b++;
            const int lo = std::min(a, b), hi = std::max(a, b);
            word |= (uint32_t)(lo | (hi << 2)) << (4 * g);
        }
        w = word;
    }
    const int64_t groups = ksp / 2, full_groups = K / mrow;
    std::vector<int> perm(mrow);
    for (int64_t vb = 0; vb < M / V; ++vb)
        for (int64_t g = 0; g < groups; ++g) {
            uint32_t *c4 = &hcol[(size_t)(vb * groups + g) * 4];
            if (g < full_groups) {
                for (int i = 0; i < mrow; ++i) perm[i] = i;
                std::shuffle(perm.begin(), perm.end(), rng);
                std::sort(perm.begin(), perm.begin() + 4);
                for (int j = 0; j < 4; ++j) c4[j] = (uint32_t)perm[j];
            } else if (g == full_groups && K % mrow) {
                for (int j = 0; j < 4; ++j) c4[j] = (uint32_t)j;
            }
        }

    // ---- device ----
    __half *dval = nullptr, *dB = nullptr, *dC = nullptr, *dAd = nullptr, *dCref = nullptr;
    uint32_t *dmeta = nullptr, *dcol = nullptr;
    CK(cudaMalloc(&dval, nv * 2));
    CK(cudaMalloc(&dmeta, nmeta * 4));
    CK(cudaMalloc(&dcol, ncol * 4));
    CK(cudaMalloc(&dB, (size_t)K * N * 2));
    CK(cudaMalloc(&dC, (size_t)M * N * 2));
    CK(cudaMalloc(&dAd, (size_t)M * K * 2));
    CK(cudaMalloc(&dCref, (size_t)M * N * 2));
    CK(cudaMemcpy(dval, hval.data(), nv * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dmeta, hmeta.data(), nmeta * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dcol, hcol.data(), ncol * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dB, hB.data(), (size_t)K * N * 2, cudaMemcpyHostToDevice));
    CK(cudaMemset(dC, 0, (size_t)M * N * 2));

    vnm_handle_t h = nullptr;
    if (ablation == 1 || ablation == 3 || ablation == 4) strategy = VNM_STRATEGY_GATHER;  // switches of the V:N:M (gather) form
    VK(vnm_prepare_as(dval, dmeta, dcol, M, K, V, nn_row, mrow, strategy, &h, nullptr));
    if (ablation == 1 || ablation == 2) VK(vnm_set_gather_mode(h, ablation));
    if (ablation == 3) VK(vnm_set_gather_mode(h, 3));
    if (ablation == 4) VK(vnm_set_epilogue(h, 1));
    VK(vnm_decompress_f16(dval, dmeta, dcol, M, K, V, nn_row, mrow, dAd, K, nullptr));  // to_dense() for the cuBLAS side

    const int TIMES = 100, WARM = 11;
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    for (int i = 0; i < WARM; ++i) VK(vnm_spmm_f16(h, dB, N, N, nullptr, dC, N, VNM_LAYOUT_MN, nullptr));
    // profiler window and range around the timed launches, as the reference has them (src/benchmark_spmm.cpp:172-175)
    cudaProfilerStart();
    nvtxRangePushA("spmm");
    CK(cudaEventRecord(e0));
    for (int i = 0; i < TIMES; ++i) VK(vnm_spmm_f16(h, dB, N, N, nullptr, dC, N, VNM_LAYOUT_MN, nullptr));
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    nvtxRangePop();
    float spmm_ms = 0;
    CK(cudaEventElapsedTime(&spmm_ms, e0, e1));
    spmm_ms /= TIMES;
    int dev_status = 0;
    VK(vnm_device_status(h, &dev_status, nullptr));

    // cuBLAS: C_ref[M,N] (row-major) = A_dense * B, i.e. column-major C^T = B^T * A^T, fp32 compute
    // (the reference's call: src/gemm/cublas_gemm.cpp:54-64).
    cublasHandle_t cb;
    if (cublasCreate(&cb) != CUBLAS_STATUS_SUCCESS) { fprintf(stderr, "cublasCreate failed\n"); return 2; }
    const float alpha = 1.f, beta = 0.f;
    auto gemm = [&]() {
        return cublasGemmEx(cb, CUBLAS_OP_N, CUBLAS_OP_N, N, M, K, &alpha, dB, CUDA_R_16F, N, dAd, CUDA_R_16F, K, &beta, dCref, CUDA_R_16F, N,
                            CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    };
    for (int i = 0; i < WARM; ++i)
        if (gemm() != CUBLAS_STATUS_SUCCESS) { fprintf(stderr, "cublasGemmEx failed\n"); return 2; }
    nvtxRangePushA("gemm");
    CK(cudaEventRecord(e0));
    for (int i = 0; i < TIMES; ++i) gemm();
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    nvtxRangePop();
    cudaProfilerStop();
    float gemm_ms = 0;
    CK(cudaEventElapsedTime(&gemm_ms, e0, e1));
    gemm_ms /= TIMES;

    int error = 0;
    if (check) {
        std::vector<__half> c((size_t)M * N), r((size_t)M * N);
        CK(cudaMemcpy(c.data(), dC, c.size() * 2, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(r.data(), dCref, r.size() * 2, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < c.size(); ++i) {
            const float a = __half2float(c[i]), b = __half2float(r[i]);
            if (!(fabsf(a - b) <= 1.0f)) {
                printf("(%zu,%zu): %f vs %f\n", i / N, i % N, a, b);
                error = 1;
                break;
            }
        }
    }
    if (dev_status != 0) error = 1;

    const double useful = 2.0 * M * N * K * nn_row / mrow;
    const double bytes = 2.0 * M * ksp + 4.0 * (M / 2) * (ksp / 8) + 16.0 * (M / V) * (ksp / 2) + 2.0 * K * N + 2.0 * M * N;
    printf("%d,%s,%d,%d,%d,%d,%d,%d,%d,%g,%d,%d,%d,%d,%d,%d,%d,%d,%d,%d,%g,%g,%g,%d,%g,%g\n", spmm_code, "sm_100a", m, k, n, meta_block_sz, block_sz,
           nn_row, mm_row, (double)density, bm, bn, bk, wm, wn, wk, mm, mn, mk, nstage, spmm_ms, gemm_ms, gemm_ms / spmm_ms, error,
           useful / (spmm_ms * 1e-3) / 1e12, bytes / (spmm_ms * 1e-3) / 1e9);

    vnm_destroy(h);
    cublasDestroy(cb);
    cudaFree(dval); cudaFree(dmeta); cudaFree(dcol); cudaFree(dB); cudaFree(dC); cudaFree(dAd); cudaFree(dCref);
    return 0;
}
