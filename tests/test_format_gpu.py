"""GPU parity tests of the format kernels (compressor + metadata packer, decompressor) through the C
ABI, bit-exact against the CPU oracle and the golden vectors of the reference."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [
    # (M, K, V, m)
    (64, 64, 32, 4), (64, 128, 64, 8), (128, 256, 128, 16), (256, 512, 128, 32), (128, 280, 64, 10),
    (64, 140, 32, 7), (64, 100, 32, 8), (64, 99, 32, 8), (64, 98, 32, 8), (1024, 4096, 64, 8),
    (4096, 1024, 128, 4), (1024, 1024, 32, 32), (512, 2000, 64, 20), (256, 4000, 128, 100),
]


def _u16(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.fixture(scope="module")
def capi():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from venom_b200 import capi
    capi.lib()
    return capi


def _random_format_shapes(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        V = 32 * int(rng.integers(1, 6))                  # 32 .. 160, not only the three the SpMM takes
        M = V * int(rng.integers(1, 5))
        m = int(rng.choice([4, 5, 6, 7, 8, 9, 12, 16, 24, 32, 48, 100, 130]))
        K = int(rng.integers(m, 30 * m))                   # any K >= m, aligned or not
        if K % m == 1:
            K += 1      # with one column in the last group the reference's to_dense drops a value: no round trip to check
        out.append((M, K, V, m))
    return out


@pytest.mark.parametrize("shape", SHAPES + _random_format_shapes(24, seed=7))
def test_compress_decompress_bit_exact(capi, oracle, shape):
    import torch
    from venom_b200.synth import random_vnm_dense
    M, K, V, m = shape
    dense, cols, mask = random_vnm_dense(M, K, V, m, seed=hash(shape) % 1000)
    ov, om, obad = oracle.compress(dense, cols, V, m)
    assert obad == 0
    d = torch.from_numpy(dense).cuda()
    c = torch.from_numpy(cols.view(np.int32)).cuda()
    v, me, bad = capi.compress(d, c, V, m)
    assert bad == 0
    assert np.array_equal(_u16(v.cpu().numpy()), _u16(ov))
    assert np.array_equal(me.cpu().numpy().view(np.uint32), om)
    # mask mode (Python-twin semantics) gives the same arrays on contract-conforming input
    v2, me2, bad2 = capi.compress(d, c, V, m, mask=torch.from_numpy(mask).cuda())
    assert bad2 == 0 and torch.equal(v2, v) and torch.equal(me2, me)
    back = capi.decompress(v, me, c, M, K, V, m)
    assert np.array_equal(_u16(back.cpu().numpy()), _u16(oracle.to_dense(ov, om, cols, M, K, V, m)))
    assert np.array_equal(_u16(back.cpu().numpy()), _u16(dense))


@pytest.mark.parametrize("i", range(10))
def test_compress_matches_reference_golden(capi, golden_format, i):
    import torch
    p = "fmt%d_" % i
    M, K, V, m = (int(x) for x in golden_format[p + "shape"])
    d = torch.from_numpy(golden_format[p + "dense"].view(np.float16).reshape(M, K).copy()).cuda()
    c = torch.from_numpy(golden_format[p + "columns"].view(np.int32).copy()).cuda()
    v, me, bad = capi.compress(d, c, V, m)
    assert bad == 0
    assert np.array_equal(_u16(v.cpu().numpy()), golden_format[p + "values"])
    assert np.array_equal(me.cpu().numpy().view(np.uint32), golden_format[p + "meta"])
    back = capi.decompress(v, me, c, M, K, V, m)
    assert np.array_equal(_u16(back.cpu().numpy()).reshape(-1), golden_format[p + "to_dense"].reshape(-1))


@pytest.mark.parametrize("i", range(3))
def test_decompress_reference_random_instances(capi, golden_format, i):
    import torch
    p = "rnd%d_" % i
    M, K, V, m = (int(x) for x in golden_format[p + "shape"])
    v = torch.from_numpy(golden_format[p + "values"].view(np.float16).copy()).cuda()
    me = torch.from_numpy(golden_format[p + "meta"].view(np.int32).copy()).cuda()
    c = torch.from_numpy(golden_format[p + "columns"].view(np.int32).copy()).cuda()
    back = capi.decompress(v, me, c, M, K, V, m)
    assert np.array_equal(_u16(back.cpu().numpy()).reshape(-1), golden_format[p + "to_dense"].reshape(-1))


def test_violations_are_counted_and_mask_mode_keeps_zeros(capi, oracle):
    import torch
    from venom_b200.synth import random_vnm_dense
    M, K, V, m = 128, 256, 64, 8
    dense, cols, mask = random_vnm_dense(M, K, V, m, seed=5)
    kept = np.argwhere(mask)
    for r, c in kept[[3, 500, 4000]]:
        dense[r, c] = 0                       # three kept entries become exact zeros
    d = torch.from_numpy(dense).cuda()
    c = torch.from_numpy(cols.view(np.int32)).cuda()
    v, me, bad = capi.compress(d, c, V, m)
    ov, om, obad = oracle.compress(dense, cols, V, m)
    assert bad == obad == 3
    assert np.array_equal(_u16(v.cpu().numpy()), _u16(ov)) and np.array_equal(me.cpu().numpy().view(np.uint32), om)
    v2, me2, bad2 = capi.compress(d, c, V, m, mask=torch.from_numpy(mask).cuda())
    ov2, om2, obad2 = oracle.compress(dense, cols, V, m, mask=mask)
    assert bad2 == obad2 == 0
    assert np.array_equal(_u16(v2.cpu().numpy()), _u16(ov2)) and np.array_equal(me2.cpu().numpy().view(np.uint32), om2)


def test_compress_strided_dense(capi, oracle):
    import torch
    from venom_b200.synth import random_vnm_dense
    M, K, V, m = 128, 256, 32, 16
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=9)
    big = torch.zeros((M, K + 64), dtype=torch.float16, device="cuda")
    big[:, :K] = torch.from_numpy(dense).cuda()
    v, me, bad = capi.compress(big[:, :K], torch.from_numpy(cols.view(np.int32)).cuda(), V, m)
    ov, om, _ = oracle.compress(dense, cols, V, m)
    assert bad == 0 and np.array_equal(_u16(v.cpu().numpy()), _u16(ov)) and np.array_equal(me.cpu().numpy().view(np.uint32), om)


@pytest.mark.parametrize("use_mask", [False, True])
def test_column_offsets_outside_their_group_count_as_violations(capi, use_mask):
    """A corrupt column-loc entry (offset >= m) is never dereferenced: the (row, group) pairs it touches are reported as
    violations and every other group still compresses to the same bits (register form without a mask, tiled form with one)."""
    import torch
    from venom_b200.synth import random_vnm_dense
    M, K, V, m = 128, 512, 64, 8
    dense, cols, mask = random_vnm_dense(M, K, V, m, seed=21)
    d = torch.from_numpy(dense).cuda()
    mk = torch.from_numpy(mask).cuda() if use_mask else None
    good_v, good_m, bad0 = capi.compress(d, torch.from_numpy(cols.view(np.int32)).cuda(), V, m, mask=mk)
    assert bad0 == 0
    broken = cols.copy().reshape(M // V, -1, 4)
    broken[1, 5, 3] = 4000000000                      # second vector block, group 5: far outside the group
    v, me, bad = capi.compress(d, torch.from_numpy(broken.reshape(-1).view(np.int32)).cuda(), V, m, mask=mk)
    assert bad == V                                   # one violation per row of the vector block
    gv, bv = good_v.cpu().numpy().view(np.uint16).copy(), v.cpu().numpy().view(np.uint16).copy()
    from venom_b200.synth import vnm_sizes
    ksp = vnm_sizes(M, K, V, m)[0]
    # compare everything except the compressed columns of group 5 (2 halves per row) of rows V .. 2V-1
    rows = np.arange(M)[:, None]
    j = np.arange(ksp)[None, :]
    idx = (rows // 16) * 16 * ksp + (j // 8) * 128 + ((rows % 16) // 4) * 32 + ((j // 2) % 4) * 8 + (rows % 4) * 2 + (j % 2)
    keep = ~((rows >= V) & (rows < 2 * V) & (j // 2 == 5))
    assert np.array_equal(gv[idx[keep]], bv[idx[keep]])
    assert np.all(bv[idx[~keep]] == 0)                # the affected slots are zero-filled
