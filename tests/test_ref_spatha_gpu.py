"""Second comparator: the reference's own Spatha SpMM kernel, compiled for sm_100a from the reference checkout
(oracle/_ref/libvnm_ref_spatha.so, test-only) and run on the same seeded operands as this library.

Bar: |C - C_spatha| <= 1e-2 * (|C_spatha| + 1) elementwise on uniform data; identical bits on small-integer data
(every partial sum is exact in fp32, so the summation order cannot matter).  The reference kernel's time on this
GPU is printed as context only: it is the legacy mma.sp path, not a target.
The tests skip where the comparator library was never built (it needs the reference checkout at build time).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


@pytest.fixture(scope="module")
def spatha_ref():
    from oracle.oracle import RefSpatha
    ref = RefSpatha.load(build=False)
    if ref is None:
        pytest.skip("oracle/_ref/libvnm_ref_spatha.so is not built")
    return ref


@pytest.fixture(scope="module")
def capi():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from venom_b200 import capi
    capi.lib()
    return capi


def _operands(oracle, M, K, V, m, N, seed, ints):
    from venom_b200.synth import random_dense_b, random_vnm_dense
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=seed, integer_values=ints)
    ov, om, bad = oracle.compress(dense, cols, V, m)
    assert bad == 0
    return ov, om, cols, random_dense_b(K, N, seed=seed + 1, integer_values=ints)


def _ours(capi, ov, om, cols, M, K, V, m, B, strategy):
    import torch
    prep = capi.Prepared(torch.from_numpy(ov).cuda(), torch.from_numpy(om.view(np.int32)).cuda(), torch.from_numpy(cols.view(np.int32)).cuda(),
                         M, K, V, m, strategy=strategy)
    out = prep.spmm(torch.from_numpy(B).cuda()).cpu().numpy()
    assert prep.device_status() == 0
    return out


# the first case is deliberately tiny; then the single-SpMM configuration and three points of the layer-shape sweep
CASES = [(128, 256, 128, 8, 64), (1024, 4096, 64, 8, 4096), (1024, 1024, 32, 4, 16384), (4096, 1024, 128, 16, 16384),
         (1024, 4096, 64, 32, 16384)]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "%dx%d_V%d_2:%d_N%d" % c)
def test_matches_reference_spatha_kernel(capi, oracle, spatha_ref, case):
    M, K, V, m, N = case
    for ints in (True, False):
        ov, om, cols, B = _operands(oracle, M, K, V, m, N, seed=M + K + V + m, ints=ints)
        want, ms = spatha_ref.spmm(ov, om, cols, M, K, V, m, B, repeats=0 if ints else 5)
        for strategy in (capi.STRATEGY_GATHER, capi.STRATEGY_DENSE_B):
            if strategy == capi.STRATEGY_DENSE_B and (m % 4 or K % m):
                continue
            got = _ours(capi, ov, om, cols, M, K, V, m, B, strategy)
            if ints:
                assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), "integer data must match the reference kernel bit for bit"
            else:
                bad, first, worst = oracle.check(got, want, mode=1, tol=REL_TOL)
                assert bad == 0, "%d mismatches against the reference kernel, first at %d, max abs err %g" % (bad, first, worst)
        if ms is not None:
            print("reference Spatha kernel (mma.sp) %dx%dx%d V=%d 2:%d: %.3f ms = %.1f useful TFLOP/s" %
                  (M, K, N, V, m, ms, 2.0 * M * N * K * 2 / m / (ms * 1e-3) / 1e12))
