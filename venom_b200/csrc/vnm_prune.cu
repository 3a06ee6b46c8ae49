// Magnitude pruner to the V:2:m pattern (CUDA).
//
// Follows group_n_m2 of the reference (end2end/grouped_nmv_tensor.py:81-343, driver :746-779): for every
// V x m block all C(m,4) column quadruples are scored in lexicographic order; the score of a quadruple is
// the fp32 sum, accumulated row by row (largest first, then second largest), of the two largest |w| among
// its four columns; the first quadruple with the strictly largest score wins (a block whose best score is
// not > 0 keeps nothing and gets columns {0,0,0,0}).  Inside every row of the winner the two largest
// entries are kept.
//
// One CTA per block: the V x m tile of |w| sits in shared memory, each thread scores a strided subset of
// the quadruples with the reference's sequential fp32 sum, a block reduction picks the largest score with
// the lowest quadruple index.  The result is bit-identical to the reference except in one corner: when the
// second and third largest |w| of a row of the winning quadruple are exactly equal, the reference's choice
// depends on scratch state left by all earlier blocks; here such a tie keeps the entries a freshly
// initialised partial sort would keep.  Scores, and therefore the chosen columns, never depend on ties.
#include "vnm_internal.h"

namespace vnm {

namespace {

__device__ __forceinline__ long long binom4(int n)  // C(n,4), n >= 0
{
    return n < 4 ? 0 : (long long)n * (n - 1) * (n - 2) * (n - 3) / 24;
}
__device__ __forceinline__ int binom3(int n) { return n < 3 ? 0 : n * (n - 1) * (n - 2) / 6; }
__device__ __forceinline__ int binom2(int n) { return n < 2 ? 0 : n * (n - 1) / 2; }

// idx-th 4-subset of {0..m-1} in lexicographic order.
__device__ __forceinline__ void unrank4(int idx, int m, int c[4])
{
    int a = 0;
    for (;; ++a) {
        const int cnt = binom3(m - 1 - a);  // quadruples starting with a
        if (idx < cnt) break;
        idx -= cnt;
    }
    int b = a + 1;
    for (;; ++b) {
        const int cnt = binom2(m - 1 - b);
        if (idx < cnt) break;
        idx -= cnt;
    }
    int cc = b + 1;
    for (;; ++cc) {
        const int cnt = m - 1 - cc;
        if (idx < cnt) break;
        idx -= cnt;
    }
    c[0] = a; c[1] = b; c[2] = cc; c[3] = cc + 1 + idx;
}

// std::partial_sort(idx, idx+2, idx+4, v[A] > v[B]) on a fresh idx = {0,1,2,3} (libstdc++ heap select).
__device__ __forceinline__ void top2_of4(const float v[4], int &i0, int &i1)
{
    int idx[4] = {0, 1, 2, 3};
    if (!(v[idx[1]] > v[idx[0]])) { int t = idx[0]; idx[0] = idx[1]; idx[1] = t; }
#pragma unroll
    for (int i = 2; i < 4; i++) {
        if (v[idx[i]] > v[idx[0]]) {
            const int value = idx[i];
            idx[i] = idx[0];
            idx[0] = idx[1];
            if (v[idx[0]] > v[value]) { idx[1] = idx[0]; idx[0] = value; }
            else idx[1] = value;
        }
    }
    i0 = idx[1];  // after sort_heap: largest first
    i1 = idx[0];
}

__global__ void __launch_bounds__(256) prune_kernel(const float *__restrict__ w, int64_t ldw, int M, int K, int V, int m, int64_t Ksp,
                                                    int32_t *__restrict__ mask, int64_t ldm, uint32_t *__restrict__ colloc)
{
    extern __shared__ float tile[];  // V x m magnitudes
    __shared__ float s_best[256];
    __shared__ int s_idx[256];
    __shared__ int s_cols[4];
    const int groups = K / m;
    const int bi = blockIdx.x / groups, g = blockIdx.x % groups;
    const float *src = w + (int64_t)bi * V * ldw + (int64_t)g * m;
    for (int e = threadIdx.x; e < V * m; e += blockDim.x) tile[e] = fabsf(src[(int64_t)(e / m) * ldw + (e % m)]);
    __syncthreads();

    const int ncombo = (int)binom4(m);
    float best = 0.0f;
    int best_idx = -1;
    for (int ci = threadIdx.x; ci < ncombo; ci += blockDim.x) {
        int c[4];
        unrank4(ci, m, c);
        float total = 0.0f;
        for (int r = 0; r < V; r++) {
            const float *row = tile + r * m;
            const float v0 = row[c[0]], v1 = row[c[1]], v2 = row[c[2]], v3 = row[c[3]];
            // largest and second largest of four (values only: ties do not change the sum)
            const float hi01 = fmaxf(v0, v1), lo01 = fminf(v0, v1), hi23 = fmaxf(v2, v3), lo23 = fminf(v2, v3);
            const float top1 = fmaxf(hi01, hi23);
            const float top2 = fmaxf(fminf(hi01, hi23), fmaxf(lo01, lo23));
            total += top1;
            total += top2;
        }
        if (total > best) { best = total; best_idx = ci; }  // strict: the first of equal scores stays
    }
    s_best[threadIdx.x] = best;
    s_idx[threadIdx.x] = best_idx;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ob = s_best[threadIdx.x + s];
            const int oi = s_idx[threadIdx.x + s];
            const float mb = s_best[threadIdx.x];
            const int mi = s_idx[threadIdx.x];
            // larger score wins; equal scores: the lower quadruple index (the one the sequential scan meets first)
            if (oi >= 0 && (mi < 0 || ob > mb || (ob == mb && oi < mi))) { s_best[threadIdx.x] = ob; s_idx[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int c[4] = {0, 0, 0, 0};
        if (s_idx[0] >= 0) unrank4(s_idx[0], m, c);
        for (int j = 0; j < 4; j++) {
            s_cols[j] = c[j];
            colloc[(int64_t)bi * (Ksp / 2) * 4 + (int64_t)g * 4 + j] = (uint32_t)c[j];
        }
    }
    __syncthreads();
    const bool any = s_idx[0] >= 0;
    for (int r = threadIdx.x; r < V; r += blockDim.x) {
        int32_t *mrow = mask + ((int64_t)bi * V + r) * ldm + (int64_t)g * m;
        for (int j = 0; j < m; j++) mrow[j] = 0;
        if (any) {
            const float *row = tile + r * m;
            const float v[4] = {row[s_cols[0]], row[s_cols[1]], row[s_cols[2]], row[s_cols[3]]};
            int i0, i1;
            top2_of4(v, i0, i1);
            mrow[s_cols[i0]] = 1;
            mrow[s_cols[i1]] = 1;
        }
    }
}

__global__ void zero_padded_colloc(uint32_t *colloc, int nblocks, int groups, int64_t gpad)
{
    const int64_t total = (int64_t)nblocks * (gpad - groups) * 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t per = (gpad - groups) * 4;
        const int64_t b = i / per, o = i % per;
        colloc[b * gpad * 4 + groups * 4 + o] = 0;
    }
}

}  // namespace

cudaError_t launch_prune(const float *w, int64_t ldw, int M, int K, int V, int m, int32_t *mask, int64_t ldm, uint32_t *colloc,
                         cudaStream_t stream)
{
    const int64_t Ksp = ksp_of(K, m);
    const int groups = K / m;
    const int nblocks = M / V;
    if (Ksp / 2 > groups) {
        zero_padded_colloc<<<64, 256, 0, stream>>>(colloc, nblocks, groups, Ksp / 2);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    const size_t smem = (size_t)V * m * sizeof(float);
    prune_kernel<<<(unsigned)(nblocks * groups), 256, smem, stream>>>(w, ldw, M, K, V, m, Ksp, mask, ldm, colloc);
    return cudaGetLastError();
}

}  // namespace vnm
