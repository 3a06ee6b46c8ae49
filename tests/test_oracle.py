"""CPU tests: the C restatement (oracle/vnm_oracle.c) against the golden vectors produced by the
reference's own Format_sr_nm<__half> / group_n_m2, and against the reference library itself where it
is available."""
import numpy as np
import pytest

from oracle.oracle import sizes
from venom_b200.synth import random_dense_b, random_vnm_dense, vnm_sizes

N_FMT = 10
N_RND = 3
N_PRN = 4


def _u16(a):
    return np.ascontiguousarray(a).view(np.uint16)


def test_sizes_match_reference_formulas():
    # cfg0 / cfg4 figures quoted from the reference's init (format_sr_nm.cpp:53-60)
    assert sizes(1024, 4096, 64, 8) == (1024, 1024 * 1024, 512 * 128, 16 * 512 * 4)
    assert sizes(49152, 12288, 128, 8) == (3072, 49152 * 3072, 24576 * 384, 384 * 1536 * 4)
    assert sizes(128, 280, 64, 10)[0] == 64            # 28 groups -> 56 -> padded to 64
    assert vnm_sizes(128, 280, 64, 10) == sizes(128, 280, 64, 10)
    with pytest.raises(ValueError):
        sizes(100, 64, 64, 8)


@pytest.mark.parametrize("i", range(N_FMT))
def test_compress_matches_golden(oracle, golden_format, i):
    p = "fmt%d_" % i
    M, K, V, m = (int(x) for x in golden_format[p + "shape"])
    dense = golden_format[p + "dense"].view(np.float16).reshape(M, K)
    cols = golden_format[p + "columns"]
    values, meta, bad = oracle.compress(dense, cols, V, m)
    assert bad == 0
    assert np.array_equal(_u16(values), golden_format[p + "values"])
    assert np.array_equal(meta, golden_format[p + "meta"])
    back = oracle.to_dense(values, meta, cols, M, K, V, m)
    assert np.array_equal(_u16(back).reshape(-1), golden_format[p + "to_dense"].reshape(-1))


@pytest.mark.parametrize("i", range(N_RND))
def test_to_dense_matches_golden_reference_random_instances(oracle, golden_format, i):
    p = "rnd%d_" % i
    M, K, V, m = (int(x) for x in golden_format[p + "shape"])
    values = golden_format[p + "values"].view(np.float16)
    back = oracle.to_dense(values, golden_format[p + "meta"], golden_format[p + "columns"], M, K, V, m)
    assert np.array_equal(_u16(back).reshape(-1), golden_format[p + "to_dense"].reshape(-1))


@pytest.mark.parametrize("i", range(N_PRN))
def test_prune_matches_golden(oracle, golden_prune, i):
    p = "prn%d_" % i
    M, K, V, m = (int(x) for x in golden_prune[p + "shape"])
    mask, cols = oracle.prune(np.abs(golden_prune[p + "w"]), V, m)
    assert np.array_equal(mask.astype(np.int8), golden_prune[p + "mask"])
    assert np.array_equal(cols, golden_prune[p + "columns"])


@pytest.mark.parametrize("shape", [(128, 256, 64, 8), (256, 384, 128, 12), (96, 512, 32, 32), (64, 99, 32, 8)])
def test_against_live_reference(oracle, reference, shape):
    if reference is None:
        pytest.skip("reference checkout not available on this host")
    M, K, V, m = shape
    dense, cols, mask = random_vnm_dense(M, K, V, m, seed=11)
    v, me, bad = oracle.compress(dense, cols, V, m)
    rv, rme = reference.compress(dense, cols, V, m)
    assert bad == 0
    assert np.array_equal(_u16(v), _u16(rv)) and np.array_equal(me, rme)
    assert np.array_equal(_u16(oracle.to_dense(v, me, cols, M, K, V, m)),
                          _u16(reference.to_dense(rv, rme, cols, M, K, V, m)))


def test_mask_mode_keeps_exact_zeros(oracle):
    # Python-twin semantics (grouped_nmv_tensor.py:578): kept entries are identified by the mask, so a
    # kept value that is exactly zero survives; the value-based mode reports it as a violation.
    M, K, V, m = 64, 64, 32, 8
    dense, cols, mask = random_vnm_dense(M, K, V, m, seed=3)
    r, c = np.argwhere(mask)[5]
    dense[r, c] = 0
    v, me, bad = oracle.compress(dense, cols, V, m, mask=mask)
    assert bad == 0
    assert np.array_equal(_u16(oracle.to_dense(v, me, cols, M, K, V, m)), _u16(dense))
    _, _, bad2 = oracle.compress(dense, cols, V, m)
    assert bad2 == 1


def test_spmm_oracle_equals_dense_check_path(oracle):
    M, K, V, m, N = 128, 256, 64, 8, 72
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=21)
    B = random_dense_b(K, N, seed=22)
    v, me, _ = oracle.compress(dense, cols, V, m)
    c_sp = oracle.spmm(v, me, cols, M, K, V, m, B)
    c_de = oracle.dense_gemm(dense, B)
    assert np.array_equal(_u16(c_sp), _u16(c_de))
    ref = dense.astype(np.float32) @ B.astype(np.float32)
    bad, first, worst = oracle.check(c_sp, ref.astype(np.float16))
    assert bad == 0
    # integer data: the reference's own check rule (|a-b| <= 1.0, benchmark_spmm.cpp:58) is exact
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=23, integer_values=True)
    B = random_dense_b(K, N, seed=24, integer_values=True)
    v, me, _ = oracle.compress(dense, cols, V, m)
    c_sp = oracle.spmm(v, me, cols, M, K, V, m, B)
    exact = (dense.astype(np.float64) @ B.astype(np.float64))
    assert np.array_equal(c_sp.astype(np.float64), exact.astype(np.float16).astype(np.float64))
    assert oracle.check(c_sp, exact.astype(np.float16), mode=0, tol=1.0)[0] == 0


def test_spmm_oracle_transposed_layout_and_row_subset(oracle):
    M, K, V, m, N = 64, 128, 32, 16, 40
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=31)
    B = random_dense_b(K, N, seed=32)
    bias = np.random.default_rng(33).uniform(-1, 1, M).astype(np.float16)
    v, me, _ = oracle.compress(dense, cols, V, m)
    c0 = oracle.spmm(v, me, cols, M, K, V, m, B)
    c1 = oracle.spmm(v, me, cols, M, K, V, m, B, bias=bias, layout=1)
    want = (c0.astype(np.float32) + bias[:, None].astype(np.float32)).astype(np.float16).T
    assert np.array_equal(_u16(c1), _u16(want))
    rows = np.array([3, 17, 63], dtype=np.int32)
    cs = oracle.spmm(v, me, cols, M, K, V, m, B, rows=rows)
    assert np.array_equal(_u16(cs[rows]), _u16(c0[rows]))
    assert not cs[0].any()
