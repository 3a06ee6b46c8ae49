// Thin extern "C" driver around the reference's own Spatha SpMM kernel (mma.sp, written for sm_86).
//
// TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it includes the reference headers by path
// (include/spatha/block_sparse/spmm/blockwise_op.h -> blockwise_kernel.h, blockwise_format.h) and is compiled
// for sm_100a by oracle/build_oracle.py into oracle/_ref/libvnm_ref_spatha.so.  The GPU parity tests use it as the
// second comparator ("the reference's Spatha output"); the product library and the benchmark's GPU arm never
// link or load it.
//
// Call sequence = what the reference harness does (src/spmm/spatha_spmm.cpp:24-38,60-90): BlockwiseSpMatrix
// init_sparse(brow = 4, mbrow = 32, bm = V) + transform_and_sync_device, SpmmNMInitFn / SpmmNMExecFn of one
// tile configuration per V: block V x 64 x 32, warp 32 x 64 x 32, mma 16 x 8 x 32, 2 stages -- the first
// configuration the reference's own benchmark scripts run for each V (benchmark/run_ablation2.sh:21,
// run_spmm_spatha.sh); a warp tile narrower than the block tile in N gives wrong results with the reference kernel.
// The dense operand is allocated with twice its size, as the reference's dataset does
// (src/dataset/dataset.cpp:81), because the kernel's zero-fill predicate `k > K` (blockwise_kernel.h:875)
// lets a padded group read row K.
#include "spatha/block_sparse/spmm/blockwise_op.h"
#include "spatha/block_sparse/spmm/blockwise_format.h"

#include <cstdint>
#include <cstring>
#include <vector>

using namespace spatha;

namespace {

template <int BM, int BN, int BK, int WM, int WN, int WK>
int run(BlockwiseSpMatrix<half> &spmat, int N, half *B, half *D, int repeats, float *ms)
{
    using TB = ShapeBase<BM, BN, BK>;
    using WP = ShapeBase<WM, WN, WK>;
    using MM = ShapeBase<16, 8, 32>;
    SpmmBlockwiseOpState state = SpmmNMInitFn<TB, WP, MM, 2>(spmat, N, B, D);
    if (!state.initSuccess) return 3;
    SpmmNMExecFn<TB, WP, MM, 2>(state, nullptr);
    if (cudaDeviceSynchronize() != cudaSuccess) return 4;
    if (repeats > 0 && ms) {
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0);
        for (int i = 0; i < repeats; i++) SpmmNMExecFn<TB, WP, MM, 2>(state, nullptr);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float t = 0;
        cudaEventElapsedTime(&t, e0, e1);
        *ms = t / repeats;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

}  // namespace

extern "C" {

// Host arrays in the reference format in, host result [M, N] out.  Needs N % 64 == 0 (the kernel's 128-bit
// epilogue does not handle an N residue, common/epilogue.h:64-110) and V in {32, 64, 128}.
// Returns 0, or a small positive code naming the step that failed.
int ref_spatha_spmm_f16(const uint16_t *values, const uint32_t *meta, const uint32_t *columns, int M, int K, int V, int m,
                        long values_elems, long meta_words, long col_words, const uint16_t *B_host, int N, uint16_t *D_host,
                        int repeats, float *ms)
{
    if (N % 64 != 0 || (V != 32 && V != 64 && V != 128)) return 1;
    std::vector<half> v(values_elems);
    std::memcpy(v.data(), values, values_elems * 2);
    std::vector<unsigned int> md(meta, meta + meta_words), idx(columns, columns + col_words);
    BlockwiseSpMatrix<half> spmat;
    spmat.init_sparse(M, K, /*brow*/ 4, /*n*/ 2, m, (int)values_elems, md, v, idx, 2022, /*mbrow*/ 32, /*bm*/ V);
    spmat.transform_and_sync_device();
    half *B = nullptr, *D = nullptr;
    const size_t b_bytes = (size_t)K * N * 2, d_bytes = (size_t)M * N * 2;
    if (cudaMalloc(&B, 2 * b_bytes) != cudaSuccess) return 2;
    if (cudaMalloc(&D, d_bytes) != cudaSuccess) { cudaFree(B); return 2; }
    cudaMemset(B, 0, 2 * b_bytes);
    cudaMemset(D, 0, d_bytes);
    cudaMemcpy(B, B_host, b_bytes, cudaMemcpyHostToDevice);
    int rc;
    if (V == 128) rc = run<128, 64, 32, 32, 64, 32>(spmat, N, B, D, repeats, ms);
    else if (V == 64) rc = run<64, 64, 32, 32, 64, 32>(spmat, N, B, D, repeats, ms);
    else rc = run<32, 64, 32, 32, 64, 32>(spmat, N, B, D, repeats, ms);
    if (rc == 0 && cudaMemcpy(D_host, D, d_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) rc = 6;
    cudaFree(B);
    cudaFree(D);
    return rc;
}

}
