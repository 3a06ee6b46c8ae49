/*
 * CPU oracle for the V:N:M (VENOM) sparse format and the Spatha SpMM check path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the host algorithms of
 * the reference project (UDC-GAC/venom) that the CUDA library is compared against.
 * Nothing in the product path may call it: only the test-suite, the smoke check and
 * the CPU-baseline leg of the benchmark load this library.
 *
 * Parity status: PINNED.  Every function below is checked bit-for-bit against the
 * reference's own Format_sr_nm<__half> class (compiled from the reference sources by
 * oracle/build_oracle.py into oracle/_ref/) and against golden vectors generated from
 * that class and committed under tests/golden/.
 *
 * Notation (all follow src/format/format_sr_nm.cpp of the reference):
 *   M rows, K columns of the sparse operand A; V = vector length (bm); n:m pattern with
 *   n == 2; m_fixed = 4 candidate columns kept per group of m columns (column-loc);
 *   Ksp = ROUND_UP(ceil(K/m)*n, 16) compressed columns per row.
 *   group g covers original columns g*m .. g*m+m-1; tile t = g/4; gi = g%4;
 *   slot s in {0,1}.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) { f16 x; memcpy(&x, &h, 2); return (float)x; }
static inline uint16_t f2h(float f) { f16 x = (f16)f; uint16_t h; memcpy(&h, &x, 2); return h; }

#define CEIL_DIV(x, y) (((x) + (y) - 1) / (y))
#define ROUND_UP(x, y) (CEIL_DIV((x), (y)) * (y))

/* Sizes of the three arrays.  Reference: Format_sr_nm<T>::init,
 * src/format/format_sr_nm.cpp:53-60 (A_num_cols_sp_pad, hA_values, hA_columns, hA_metadata). */
int vnm_oracle_sizes(int M, int K, int V, int n, int m,
                     int64_t *ksp, int64_t *values_elems, int64_t *meta_words, int64_t *colloc_words)
{
    if (n != 2 || m < 4 || V <= 0 || M <= 0 || K <= 0 || (M % V) != 0 || (V % 32) != 0) return 1;
    int64_t Ksp = ROUND_UP((int64_t)(ROUND_UP(K, m) / m) * n, 16);
    if (ksp) *ksp = Ksp;
    if (values_elems) *values_elems = (int64_t)M * Ksp;
    if (colloc_words) *colloc_words = (int64_t)(M / V) * (Ksp / n) * 4;
    if (meta_words) *meta_words = (int64_t)(M / 2) * (Ksp / 8);
    return 0;
}

/* Physical index maps.  They are the closed form of the loop nests in
 * Format_sr_nm<T>::to_sparse_sr_nm (src/format/format_sr_nm.cpp:441-536) and ::to_dense (:347-414):
 *   hA_values   [bm_i*bm*Ksp + mbrow_i*mbrow*Ksp + mbrow_i2*16*Ksp + brow_i*brow*8 + mcol_i*16*8
 *                + mbrow_ii*4 + mcol_ii*8 + mbrow_iii*2 + n_i]                      (:509-518)
 *   hA_metadata [bm_i*mcol_k*bm/2 + mbrow_i*mcol_k*16 + mbrow_i2*8 + brow_i*2 + mcol_i*16 + mbrow_ii],
 *   shift = mbrow_iii*16 + mcol_ii*4 + n_i*2                                         (:527-536)
 *   hA_columns  [bm_i*col_k*16 + mcol_i*16 + col_i*4 + col_ii]                       (:447-451)
 * with row r = bm_i*bm + mbrow_i*32 + mbrow_i2*16 + brow_i*4 + mbrow_ii*2 + mbrow_iii,
 * group g = mcol_i*4 + mcol_ii (brow = 4, mbrow = 32 as every caller passes). */
static inline int64_t values_index(int64_t r, int64_t g, int s, int64_t Ksp)
{
    return (r / 16) * 16 * Ksp + (g / 4) * 128 + ((r % 16) / 4) * 32 + (g % 4) * 8 + (r % 4) * 2 + s;
}
static inline int64_t meta_index(int64_t r, int64_t g, int64_t Ksp)
{
    return (r / 32) * 16 * (Ksp / 8) + (g / 4) * 16 + (r % 32) / 2;
}
static inline int meta_shift(int64_t r, int64_t g, int s)
{
    return (int)((r & 1) * 16 + (g % 4) * 4 + s * 2);
}
static inline int64_t colloc_index(int64_t r, int64_t g, int V, int64_t Ksp)
{
    return (r / V) * (Ksp / 2) * 4 + g * 4;
}

/* Compressor + metadata packer.  Reference: Format_sr_nm<T>::to_sparse_sr_nm,
 * src/format/format_sr_nm.cpp:419-543 (value test `val != 0`, :474) and its Python twin
 * end2end/grouped_nmv_tensor.py:487-675 (mask test `nnz != 0`, :578) when `mask` is given.
 *
 * For each (row, group) the four column-loc candidates are scanned in ascending order; every kept one
 * appends (candidate position, value) to the slot list; candidates beyond column K append (0, 0) for
 * the first two positions only (:486-500).  The reference is only well defined when exactly two slots
 * are produced: with fewer it re-uses stale scratch from the previous group, with more it writes past
 * the slot.  This oracle takes the first two produced slots, zero-fills missing ones with
 * (position 0, value 0) and returns the number of (row, group) pairs that did not produce exactly two
 * -- callers must treat a non-zero return as "input violates the format contract".
 * Values and metadata must be zero-initialised by the caller exactly as init_from_dense does
 * (:136-143); this function overwrites every word and every value slot anyway. */
int64_t vnm_oracle_compress_f16(const uint16_t *dense, const int32_t *mask, const uint32_t *columns,
                                int M, int K, int V, int n, int m,
                                uint16_t *values, uint32_t *meta)
{
    int64_t Ksp, nv, nm, nc;
    if (vnm_oracle_sizes(M, K, V, n, m, &Ksp, &nv, &nm, &nc)) return -1;
    memset(values, 0, (size_t)nv * sizeof(uint16_t));
    memset(meta, 0, (size_t)nm * sizeof(uint32_t));
    int64_t G = Ksp / 2; /* groups incl. padding */
    int64_t violations = 0;
#pragma omp parallel for schedule(static) reduction(+ : violations)
    for (int64_t rp = 0; rp < M / 2; rp++) {
        for (int64_t g = 0; g < G; g++) {
            for (int h = 0; h < 2; h++) {
                int64_t r = rp * 2 + h;
                const uint32_t *c4 = columns + colloc_index(r, g, V, Ksp);
                uint16_t v[2] = {0, 0};
                uint32_t idx[2] = {0, 0};
                int pos = 0;
                for (int j = 0; j < 4; j++) {
                    int64_t col = g * m + (int64_t)c4[j];
                    if (col < K) {
                        uint16_t val = dense[r * (int64_t)K + col];
                        int keep = mask ? (mask[r * (int64_t)K + col] != 0) : (h2f(val) != 0.0f);
                        if (keep) {
                            if (pos < 2) { idx[pos] = (uint32_t)j; v[pos] = val; }
                            pos++;
                        }
                    } else if (j < 2) {
                        if (pos < 2) { idx[pos] = 0; v[pos] = 0; }
                        pos++;
                    }
                }
                if (pos != 2) violations++;
                for (int s = 0; s < 2; s++) {
                    values[values_index(r, g, s, Ksp)] = v[s];
                    /* rows 2rp and 2rp+1 share one word; this thread owns both */
                    meta[meta_index(r, g, Ksp)] |= idx[s] << meta_shift(r, g, s);
                }
            }
        }
    }
    return violations;
}

/* Decompressor.  Reference: Format_sr_nm<T>::to_dense, src/format/format_sr_nm.cpp:327-417
 * (dense is zero-filled by resize, :330; entries whose original column is >= K are skipped, :384). */
int vnm_oracle_to_dense_f16(const uint16_t *values, const uint32_t *meta, const uint32_t *columns,
                            int M, int K, int V, int n, int m, uint16_t *dense)
{
    int64_t Ksp;
    if (vnm_oracle_sizes(M, K, V, n, m, &Ksp, 0, 0, 0)) return 1;
    memset(dense, 0, (size_t)M * K * sizeof(uint16_t));
    int64_t G = Ksp / 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++) {
        for (int64_t g = 0; g < G; g++) {
            const uint32_t *c4 = columns + colloc_index(r, g, V, Ksp);
            uint32_t w = meta[meta_index(r, g, Ksp)];
            for (int s = 0; s < 2; s++) {
                uint32_t sel = (w >> meta_shift(r, g, s)) & 3u;
                int64_t col = g * m + (int64_t)c4[sel];
                if (col < K) dense[r * (int64_t)K + col] = values[values_index(r, g, s, Ksp)];
            }
        }
    }
    return 0;
}

/* Host SpMM of the check path.  The reference has no CPU SpMM: its --check compares the kernel with
 * cuBLAS run on to_dense() (src/benchmark_spmm.cpp:169-179; src/gemm/cublas_gemm.cpp:54-64: fp16
 * inputs, fp32 compute, fp16 output).  This restates that arithmetic on the host:
 *     C[r, c] = fp16( sum_k fp32(A_dense[r, k]) * fp32(B[k, c]) ),  k ascending,
 * evaluated straight from the compressed form (zeros of A_dense contribute exactly 0 for finite B).
 * layout 0: C is [M, N] row-major with leading dimension ldc (the CLI kernel);
 * layout 1: C is [N, M] row-major with leading dimension ldc and bias[r] is added after the fp16
 *           rounding, in fp16, as the torch variant's fused epilogue does
 *           (end2end/spatha_mod/block_sparse/spmm/blockwise_kernel.h:294-343).
 * Only rows listed in `rows` (nrows of them; NULL = all M rows) are computed; other rows of C are
 * left untouched, which is what the sampled check of the large configurations uses. */
int vnm_oracle_spmm_f16(const uint16_t *values, const uint32_t *meta, const uint32_t *columns,
                        int M, int K, int V, int n, int m,
                        const uint16_t *B, int N, int64_t ldb,
                        const uint16_t *bias, uint16_t *C, int64_t ldc, int layout,
                        const int32_t *rows, int nrows)
{
    int64_t Ksp;
    if (vnm_oracle_sizes(M, K, V, n, m, &Ksp, 0, 0, 0)) return 1;
    int64_t G = Ksp / 2;
    int R = rows ? nrows : M;
#pragma omp parallel
    {
        float *acc = (float *)malloc((size_t)N * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int ri = 0; ri < R; ri++) {
            int64_t r = rows ? rows[ri] : ri;
            for (int c = 0; c < N; c++) acc[c] = 0.0f;
            for (int64_t g = 0; g < G; g++) {
                const uint32_t *c4 = columns + colloc_index(r, g, V, Ksp);
                uint32_t w = meta[meta_index(r, g, Ksp)];
                /* slots are stored in ascending candidate order, so k ascends here */
                for (int s = 0; s < 2; s++) {
                    uint32_t sel = (w >> meta_shift(r, g, s)) & 3u;
                    int64_t col = g * m + (int64_t)c4[sel];
                    if (col >= K) continue;
                    float a = h2f(values[values_index(r, g, s, Ksp)]);
                    const f16 *brow = (const f16 *)(B + col * ldb);
                    for (int c = 0; c < N; c++) acc[c] += a * (float)brow[c];
                }
            }
            if (layout == 0) {
                uint16_t *crow = C + r * ldc;
                for (int c = 0; c < N; c++) crow[c] = f2h(acc[c]);
            } else {
                f16 b = 0;
                if (bias) memcpy(&b, &bias[r], 2);
                for (int c = 0; c < N; c++) {
                    f16 h = (f16)acc[c];
                    f16 o = bias ? (f16)((float)h + (float)b) : h; /* fp16 add, round-to-nearest */
                    uint16_t u; memcpy(&u, &o, 2);
                    C[(int64_t)c * ldc + r] = u;
                }
            }
        }
        free(acc);
    }
    return 0;
}

/* Dense fp32-accumulate host GEMM over a decompressed A (the literal check path: to_dense() followed
 * by a dense product, src/benchmark_spmm.cpp:169).  Used to validate vnm_oracle_spmm_f16 and as the
 * timed CPU baseline.  C is [M, N] row-major. */
int vnm_oracle_dense_gemm_f16(const uint16_t *A, const uint16_t *B, uint16_t *C,
                              int M, int K, int N, const int32_t *rows, int nrows)
{
    int R = rows ? nrows : M;
#pragma omp parallel
    {
        float *acc = (float *)malloc((size_t)N * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int ri = 0; ri < R; ri++) {
            int64_t r = rows ? rows[ri] : ri;
            for (int c = 0; c < N; c++) acc[c] = 0.0f;
            for (int64_t k = 0; k < K; k++) {
                float a = h2f(A[r * (int64_t)K + k]);
                if (a == 0.0f) continue;
                const f16 *brow = (const f16 *)(B + k * (int64_t)N);
                for (int c = 0; c < N; c++) acc[c] += a * (float)brow[c];
            }
            for (int c = 0; c < N; c++) C[r * (int64_t)N + c] = f2h(acc[c]);
        }
        free(acc);
    }
    return 0;
}

/* Result check.  Reference: check_results, src/benchmark_spmm.cpp:51-74 (abs tolerance 1.0 on integer
 * data, stops at the first mismatch).  mode 0 = the reference's rule |a-b| > abs_tol;
 * mode 1 = the build's rule |a-b| > rel_tol*(|b|+1).  Returns the number of mismatching elements and
 * stores the index of the first one (or -1). */
int64_t vnm_oracle_check(const uint16_t *got, const uint16_t *want, int64_t count,
                         int mode, float tol, int64_t *first_bad, float *max_err)
{
    int64_t bad = 0, first = -1;
    float worst = 0.0f;
    for (int64_t i = 0; i < count; i++) {
        float a = h2f(got[i]), b = h2f(want[i]);
        float d = fabsf(a - b);
        float lim = mode == 0 ? tol : tol * (fabsf(b) + 1.0f);
        if (!(d <= lim)) { if (first < 0) first = i; bad++; }
        if (d > worst || d != d) worst = d;
    }
    if (first_bad) *first_bad = first;
    if (max_err) *max_err = worst;
    return bad;
}

/* Magnitude pruner.  Reference: group_n_m2, end2end/grouped_nmv_tensor.py:81-343 (driver :746-779).
 * Per V x m block every 4-column combination (lexicographic) is scored by the sum over rows of the two
 * largest of the four |w|; the first combination with the strictly largest fp32 score wins.  Inside a
 * row the two largest are picked by a partial sort whose index scratch persists between rows and
 * combinations (:112-113,:151-152), so ties are resolved by that scratch's current order; this
 * restatement keeps the same persistent scratch and the same libstdc++ partial_sort steps for
 * 4 elements / 2 selected (heap-select over the first two, then compare-and-swap of the rest).
 * absw: [M, K] fp32 magnitudes.  mask: [M, K] int32 out.  columns: column-loc out (sorted ascending).
 * Only K % m == 0 is restated (every published configuration); a ragged K returns 2. */
static void psort2_of4(uint64_t idx[4], const float v[4])
{
    /* std::partial_sort(first, first+2, last, comp) with comp(A,B) = v[A] > v[B]:
     * make_heap on [0,2) (a "max-heap" w.r.t. comp, i.e. the *smallest* v on top), then for each i in
     * [2,4): if comp(idx[i], idx[0]) pop-replace; finally sort_heap.  For two elements this is: */
    /* make_heap of 2 = __adjust_heap(hole 0, len 2, value idx[0]): idx[1] moves up, then __push_heap
     * puts the old idx[0] back on top only if comp(idx[1], idx[0]); so the pair is swapped unless
     * v[idx[1]] > v[idx[0]] (ties swap). */
    if (!(v[idx[1]] > v[idx[0]])) { uint64_t t = idx[0]; idx[0] = idx[1]; idx[1] = t; }
    for (int i = 2; i < 4; i++) {
        if (v[idx[i]] > v[idx[0]]) {
            /* __pop_heap(first, middle, i): value = idx[i]; idx[i] = idx[0]; adjust heap of size 2
             * with hole at 0 and then push value */
            uint64_t value = idx[i];
            idx[i] = idx[0];
            /* __adjust_heap(first, hole=0, len=2, value): secondChild loop does not run for len 2
             * ((len-1)/2 = 0); since len is even and secondChild == (len-2)/2 == 0: move child 1 up */
            idx[0] = idx[1];
            /* __push_heap(first, hole=1, top=0, value): parent 0; while comp(idx[parent], value) */
            if (v[idx[0]] > v[value]) { idx[1] = idx[0]; idx[0] = value; }
            else idx[1] = value;
        }
    }
    /* sort_heap on 2 elements: pop_heap -> swap(idx[0], idx[1]) then heap of size 1 */
    { uint64_t t = idx[0]; idx[0] = idx[1]; idx[1] = t; }
}

int vnm_oracle_prune(const float *absw, int M, int K, int V, int n, int m, int32_t *mask, uint32_t *columns)
{
    int64_t Ksp;
    if (vnm_oracle_sizes(M, K, V, n, m, &Ksp, 0, 0, 0)) return 1;
    if (K % m != 0) return 2;
    memset(mask, 0, (size_t)M * K * sizeof(int32_t));
    int64_t ncol_words = (int64_t)(M / V) * (Ksp / 2) * 4;
    for (int64_t i = 0; i < ncol_words; i++) columns[i] = 0;
    int groups = K / m;
    uint64_t indices[4] = {0, 1, 2, 3}; /* persists over everything, as in the reference (:112-113) */
    int32_t *best_mask = (int32_t *)malloc((size_t)V * m * sizeof(int32_t));
    int32_t *cur_mask = (int32_t *)malloc((size_t)V * m * sizeof(int32_t));
    for (int bi = 0; bi < M / V; bi++) {
        for (int g = 0; g < groups; g++) {
            float best = 0.0f;
            int best_cols[4] = {0, 0, 0, 0};
            memset(best_mask, 0, (size_t)V * m * sizeof(int32_t));
            int vx[4];
            for (vx[0] = 0; vx[0] < m; vx[0]++)
            for (vx[1] = vx[0] + 1; vx[1] < m; vx[1]++)
            for (vx[2] = vx[1] + 1; vx[2] < m; vx[2]++)
            for (vx[3] = vx[2] + 1; vx[3] < m; vx[3]++) {
                float total = 0.0f;
                memset(cur_mask, 0, (size_t)V * m * sizeof(int32_t));
                for (int row = 0; row < V; row++) {
                    const float *w = absw + ((int64_t)bi * V + row) * K + (int64_t)g * m;
                    float v[4] = {w[vx[0]], w[vx[1]], w[vx[2]], w[vx[3]]};
                    psort2_of4(indices, v);
                    for (int id = 0; id < 2; id++) {
                        total += w[vx[indices[id]]];
                        cur_mask[row * m + vx[indices[id]]] = 1;
                    }
                }
                if (total > best) {
                    best = total;
                    memcpy(best_mask, cur_mask, (size_t)V * m * sizeof(int32_t));
                    for (int j = 0; j < 4; j++) best_cols[j] = vx[j];
                }
            }
            for (int row = 0; row < V; row++)
                for (int j = 0; j < m; j++)
                    mask[((int64_t)bi * V + row) * K + (int64_t)g * m + j] = best_mask[row * m + j];
            for (int j = 0; j < 4; j++)
                columns[(int64_t)bi * (Ksp / 2) * 4 + (int64_t)g * 4 + j] = (uint32_t)best_cols[j];
        }
    }
    free(best_mask);
    free(cur_mask);
    return 0;
}

/* Sets the number of OpenMP threads of the host routines explicitly (launchers such as torchrun export
 * OMP_NUM_THREADS=1, which would otherwise silently make the timed CPU baseline single-threaded). */
void vnm_oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int vnm_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
