// Small program against include/venom_b200_spatha.hpp, written the way a harness uses the reference's classes:
// build a V:N:M instance from a dense matrix, round-trip it, multiply, compare with a host fp32 loop.
// Compiled by tests/test_cpp_shim.py; prints "shim ok" and returns 0 on success.
#include <cuda_fp16.h>

#include <cmath>
#include <cstdio>
#include <vector>

#include "venom_b200_spatha.hpp"

int main()
{
    const int M = 256, K = 512, N = 128, V = 128, n = 2, m = 8;
    int64_t ksp = 0, nv = 0, nm = 0, nc = 0;
    if (vnm_sizes(M, K, V, n, m, &ksp, &nv, &nm, &nc)) return 2;
    // column-loc {1,2,5,6} for every block; every row keeps two of them, chosen by (row + group) parity
    std::vector<unsigned int> columns(nc);
    const unsigned int sel[4] = {1, 2, 5, 6};
    for (int64_t i = 0; i < nc; i++) columns[i] = sel[i % 4];
    std::vector<__half> dense((size_t)M * K, __float2half(0.f));
    for (int r = 0; r < M; r++)
        for (int g = 0; g < K / m; g++) {
            const int a = (r + g) & 1, b = 2 + ((r + g) >> 1 & 1);
            dense[(size_t)r * K + g * m + sel[a]] = __float2half((float)((r * 7 + g * 3) % 9 - 4 ? (r * 7 + g * 3) % 9 - 4 : 1));
            dense[(size_t)r * K + g * m + sel[b]] = __float2half((float)((r * 5 + g) % 7 - 3 ? (r * 5 + g) % 7 - 3 : 2));
        }
    std::vector<__half> B((size_t)K * N);
    for (size_t i = 0; i < B.size(); i++) B[i] = __float2half((float)((int)(i * 2654435761u >> 28) - 8));

    venom_b200::Format_sr_nm<__half> f;
    f.init_from_dense(M, K, (float)n / m, 0, n, m, 4, 32, V, dense, columns);
    if ((int64_t)f.get_hA_val().size() != nv || (int64_t)f.get_hA_metadata().size() != nm || f.get_A_nnz() != nv) return 3;
    std::vector<__half> &back = f.to_dense();
    for (size_t i = 0; i < dense.size(); i++)
        if (__half2float(back[i]) != __half2float(dense[i])) { std::printf("round trip differs at %zu\n", i); return 4; }

    venom_b200::Spatha<__half, __half> op(f, B, N);
    const float ms = op.spmm(3, V, 64, 32, 32, 64, 32, 16, 8, 32, 2);
    std::vector<__half> &C = op.get_result();
    for (int r = 0; r < M; r++)
        for (int c = 0; c < N; c++) {
            float acc = 0.f;
            for (int k = 0; k < K; k++) acc += __half2float(dense[(size_t)r * K + k]) * __half2float(B[(size_t)k * N + c]);
            const float got = __half2float(C[(size_t)r * N + c]), want = __half2float(__float2half(acc));
            if (std::fabs(got - want) > 1e-2f * (std::fabs(want) + 1.f)) { std::printf("C[%d,%d] = %g, expected %g\n", r, c, got, want); return 5; }
        }
    std::printf("shim ok (%.4f ms per launch)\n", ms);
    return 0;
}
