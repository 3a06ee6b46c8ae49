"""GPU parity at the sizes the benchmark configurations name, through the C ABI, against the CPU oracle.

The small-shape tests elsewhere give every CTA one tile.  Here every launch has far more tiles than the GPU has
SMs and many k-tiles per tile, so the persistent paths of both kernels are exercised: accumulator hand-off
between consecutive tiles, producers running ahead into the next tile, and barrier phases that wrap many times.
Operands are drawn and compressed on the GPU (the compressor is compared with the oracle bit for bit in
test_format_gpu.py / test_large_gpu.py); the oracle then decodes the same three reference-format arrays on
the host and multiplies a seeded sample of rows in fp32.  Tolerance: |C - C_ref| <= 1e-2 * (|C_ref| + 1).
A checksum of checksums, (1^T A) B == 1^T C, covers the rows that were not sampled.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2
SHAPES = [(1024, 1024), (4096, 1024), (1024, 4096)]
CFG1 = [(M, K, V, m, 16384) for (M, K) in SHAPES for V in (32, 64, 128) for m in (4, 8, 16, 32)]


@pytest.fixture(scope="module")
def capi():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from venom_b200 import capi
    capi.lib()
    return capi


def _operands(capi, M, K, V, m, N, seed):
    import torch
    from venom_b200.synth import random_vnm_dense_cuda
    dense, colloc = random_vnm_dense_cuda(M, K, V, m, seed=seed)
    values, meta, bad = capi.compress(dense, colloc, V, m)
    assert bad == 0
    g = torch.Generator(device="cuda")
    g.manual_seed(seed + 1)
    B = (torch.rand((K, N), device="cuda", generator=g) * 2 - 1).half()
    return dense, colloc, values, meta, B


def _check_rows(oracle, out, layout, values, meta, colloc, M, K, V, m, B, bias=None, nrows=48, seed=1):
    import torch
    rows = np.sort(np.random.default_rng(seed).choice(M, size=min(nrows, M), replace=False)).astype(np.int32)
    hv = values.cpu().numpy()
    hm = meta.cpu().numpy().view(np.uint32)
    hc = colloc.cpu().numpy().view(np.uint32)
    hb = None if bias is None else bias.cpu().numpy()
    want = oracle.spmm(hv, hm, hc, M, K, V, m, B.cpu().numpy(), bias=hb, layout=layout, rows=rows)
    ridx = torch.from_numpy(rows).long().cuda()
    if layout == 0:
        got, ref = out[ridx].cpu().numpy(), want[rows]
    else:
        got, ref = out[:, ridx].cpu().numpy(), want[:, rows]
    bad, first, worst = oracle.check(got, ref, mode=1, tol=REL_TOL)
    assert bad == 0, "%d mismatches in the sampled rows, first at %d, max abs err %g" % (bad, first, worst)


def _check_column_sums(dense, B, out, layout, bias=None):
    """(1^T A) B == 1^T C up to the fp16 rounding of the M entries of C that each sum adds up."""
    import torch
    M = dense.shape[0]
    want = (dense.float().sum(0, keepdim=True) @ B.float()).flatten()
    if bias is not None:
        want = want + bias.float().sum()
    got = (out.float().sum(0) if layout == 0 else out.float().sum(1)).flatten()
    # every stored element carries a rounding error of at most 2^-11 relative; the errors add up like a random walk
    scale = float(out.float().abs().max()) * (2.0 ** -11) * (M ** 0.5) * 8 + 1e-3
    err = float((got - want).abs().max())
    assert err <= scale, "column sums differ by %g (allowed %g)" % (err, scale)


@pytest.mark.parametrize("point", CFG1, ids=lambda p: "%dx%d_V%d_2:%d" % p[:4])
def test_cfg1_sweep_point_sampled_rows(capi, oracle, point):
    """All 36 points of the N:M / V sweep at BERT-large layer shapes, N = 16384, in whichever operand form the
    library picks (V = 128 at m >= 16 and V = 64 at m = 32 run the V:N:M gather kernel with 512-2048 tiles)."""
    M, K, V, m, N = point
    dense, colloc, values, meta, B = _operands(capi, M, K, V, m, N, seed=M + K + 7 * V + m)
    prep = capi.Prepared(values, meta, colloc, M, K, V, m)
    out = prep.spmm(B)
    assert prep.device_status() == 0
    _check_rows(oracle, out, 0, values, meta, colloc, M, K, V, m, B)
    _check_column_sums(dense, B, out, 0)


FORCED_GATHER = [(1024, 4096, 64, 8, 4096), (4096, 4096, 128, 8, 4096), (1024, 1024, 32, 8, 16384), (4096, 1024, 64, 16, 16384),
                 (1024, 4096, 128, 4, 16384), (4096, 1024, 32, 32, 16384)]


@pytest.mark.parametrize("shape", FORCED_GATHER, ids=lambda p: "%dx%d_V%d_2:%d_N%d" % p)
def test_gather_form_forced_at_benchmark_sizes(capi, oracle, shape):
    """The V:N:M gather kernel at shapes where the automatic choice would take the dense-B form (2:8 above all):
    one, two and four vector blocks per row tile, many tiles per CTA, both layouts."""
    import torch
    M, K, V, m, N = shape
    dense, colloc, values, meta, B = _operands(capi, M, K, V, m, N, seed=3 * M + K + V + m)
    prep = capi.Prepared(values, meta, colloc, M, K, V, m, strategy=capi.STRATEGY_GATHER)
    assert not prep.dense_b_form()
    out = prep.spmm(B)
    _check_rows(oracle, out, 0, values, meta, colloc, M, K, V, m, B)
    _check_column_sums(dense, B, out, 0)
    bias = (torch.rand(M, device="cuda") - 0.5).half()
    outT = prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM)
    _check_rows(oracle, outT, 1, values, meta, colloc, M, K, V, m, B, bias=bias)
    assert prep.device_status() == 0
    # both operand forms give the same product up to fp32 summation order
    other = capi.Prepared(values, meta, colloc, M, K, V, m, strategy=capi.STRATEGY_DENSE_B).spmm(B)
    assert float((other.float() - out.float()).abs().max()) <= REL_TOL * (float(out.float().abs().max()) + 1)


# the four linear layers of a GPT-3-175B-shaped block (M = out features, K = in features), V = 128, 2:16
GPT3_LAYERS = [(36864, 12288), (12288, 12288), (49152, 12288), (12288, 49152)]


@pytest.mark.parametrize("mk", GPT3_LAYERS, ids=lambda p: "%dx%d" % p)
def test_gpt3_layer_shapes_one_sequence_shard(capi, oracle, mk):
    """128:2:16 at hidden 12288 / FFN 49152 on one sequence's column shard (N = 2048): up to 96 k-tiles per tile
    in the gather kernel, 768-3072 tiles, [M,N] and [N,M] + bias."""
    import torch
    M, K = mk
    V, m, N = 128, 16, 2048
    dense, colloc, values, meta, B = _operands(capi, M, K, V, m, N, seed=M // 64 + K // 32)
    prep = capi.Prepared(values, meta, colloc, M, K, V, m)
    assert not prep.dense_b_form()
    out = prep.spmm(B)
    assert prep.device_status() == 0
    _check_rows(oracle, out, 0, values, meta, colloc, M, K, V, m, B, nrows=32)
    _check_column_sums(dense, B, out, 0)
    bias = (torch.rand(M, device="cuda") - 0.5).half()
    outT = prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM)
    assert prep.device_status() == 0
    _check_rows(oracle, outT, 1, values, meta, colloc, M, K, V, m, B, bias=bias, nrows=32, seed=2)
    _check_column_sums(dense, B, outT, 1, bias=bias)


PAIR_CASES = [(1024, 1024, 64, 8, 17000), (2048, 512, 128, 4, 9000), (512, 4096, 32, 16, 18000), (4096, 1024, 128, 8, 4808),
              (1024, 4096, 64, 8, 4096),      # the single-SpMM configuration: 256-row pair tiles (one row tile per CTA)
              (768, 1024, 128, 8, 8200)]      # six row tiles: 256-row pair tiles, ragged N


@pytest.mark.parametrize("shape", PAIR_CASES, ids=lambda p: "%dx%d_V%d_2:%d_N%d" % p)
def test_two_sm_kernel_matches_single_sm_kernel_and_oracle(capi, oracle, shape):
    """Dense-B form on pairs of SMs (cta_group::2, each CTA loading half of every B stage) against the single-SM kernel:
    same MMAs in the same order, so the bits must be identical -- [M,N], [N,M] + bias, and the [N,K] dense operand --
    with a ragged last column tile; and against the CPU oracle on sampled rows."""
    import torch
    M, K, V, m, N = shape
    dense, colloc, values, meta, B = _operands(capi, M, K, V, m, N, seed=M + 2 * K + N)
    prep = capi.Prepared(values, meta, colloc, M, K, V, m, strategy=capi.STRATEGY_DENSE_B)
    assert prep.dense_b_form()
    assert prep.config(N)["stages"] == 2, "the pair kernel was expected to be chosen for this shape"   # stages: 2 = SM pairs
    bias = (torch.rand(M, device="cuda") - 0.5).half()
    bt = B.t().contiguous()
    pair = [prep.spmm(B), prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM), prep.spmm_nk(bt, bias=bias, layout=capi.VNM_LAYOUT_NM),
            prep.spmm_nk(bt, layout=capi.VNM_LAYOUT_MN)]
    assert prep.device_status() == 0
    # one and two row tiles per CTA (256- and 512-row pair tiles; the first alternates two accumulators between tiles)
    for mode, tile_m in ((3, 256), (4, 512)):
        prep.set_pair_mode(mode)
        if prep.config(N)["stages"] == 2 and prep.config(N)["tile_m"] == tile_m:
            assert torch.equal(prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM), pair[1])
            assert torch.equal(prep.spmm_nk(bt, layout=capi.VNM_LAYOUT_MN), pair[3])
            assert prep.device_status() == 0
    prep.set_pair_mode(0)
    assert prep.config(N)["stages"] == 1
    single = [prep.spmm(B), prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM), prep.spmm_nk(bt, bias=bias, layout=capi.VNM_LAYOUT_NM),
              prep.spmm_nk(bt, layout=capi.VNM_LAYOUT_MN)]
    assert prep.device_status() == 0
    for a, b in zip(pair, single):
        assert torch.equal(a, b)
    _check_rows(oracle, pair[0], 0, values, meta, colloc, M, K, V, m, B)
    _check_rows(oracle, pair[1], 1, values, meta, colloc, M, K, V, m, B, bias=bias)
    _check_column_sums(dense, B, pair[0], 0)


@pytest.mark.parametrize("shape", [(1024, 1024, 64, 8, 17000), (768, 1024, 128, 8, 8200), (384, 512, 128, 4, 1000)],
                         ids=lambda p: "%dx%d_V%d_2:%d_N%d" % p)
def test_product_stored_to_several_destinations(capi, shape):
    """vnm_spmm_f16_multi: every output tile is stored to each destination (the store side of the peer-store gathered
    product, here with all destinations on one GPU).  Both dense-B kernels, both layouts; every copy must carry the bits
    of the single-destination product, and memory outside the destinations' rows must stay untouched."""
    import torch
    M, K, V, m, N = shape
    dense, colloc, values, meta, B = _operands(capi, M, K, V, m, N, seed=5 * M + K + N)
    prep = capi.Prepared(values, meta, colloc, M, K, V, m, strategy=capi.STRATEGY_DENSE_B)
    bias = (torch.rand(M, device="cuda") - 0.5).half()
    for pair_mode in (1, 0):
        prep.set_pair_mode(pair_mode)
        for layout, b in ((capi.VNM_LAYOUT_MN, None), (capi.VNM_LAYOUT_NM, bias)):
            want = prep.spmm(B, bias=b, layout=layout)
            rows = want.shape[0]
            # destinations are row blocks of larger buffers, as a rank's rows are inside the gathered result
            bufs = [torch.full((rows + 16, want.shape[1]), 7.0, dtype=torch.float16, device="cuda") for _ in range(3)]
            outs = [buf[8:8 + rows] for buf in bufs]
            prep.spmm_multi(B, outs, bias=b, layout=layout)
            assert prep.device_status() == 0
            for buf, o in zip(bufs, outs):
                assert torch.equal(o, want)
                assert bool((buf[:8] == 7.0).all()) and bool((buf[8 + rows:] == 7.0).all())
    with pytest.raises(capi.VenomError):
        prep.spmm_multi(B, [torch.empty_like(want)] * 9, layout=capi.VNM_LAYOUT_NM)
    # gather form: several destinations only where its epilogue leaves through TMA stores, i.e. layout NM
    gather = capi.Prepared(values, meta, colloc, M, K, V, m, strategy=capi.STRATEGY_GATHER)
    with pytest.raises(capi.VenomError):
        gather.spmm_multi(B, [torch.empty((M, N), dtype=torch.float16, device="cuda")] * 2)
    want = gather.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM)
    bufs = [torch.full((N + 16, M), 7.0, dtype=torch.float16, device="cuda") for _ in range(3)]
    outs = [buf[8:8 + N] for buf in bufs]
    gather.spmm_multi(B, outs, bias=bias, layout=capi.VNM_LAYOUT_NM)
    assert gather.device_status() == 0
    for buf, o in zip(bufs, outs):
        assert torch.equal(o, want)
        assert bool((buf[:8] == 7.0).all()) and bool((buf[8 + N:] == 7.0).all())


@pytest.mark.parametrize("shape", [(1024, 1024, 128, 16, 16384), (192, 512, 64, 32, 1000), (96, 256, 32, 8, 4104), (4096, 1024, 64, 32, 8200),
                                   (256, 2048, 128, 8, 72)], ids=lambda p: "%dx%d_V%d_2:%d_N%d" % p)
def test_gather_form_nm_epilogues_give_identical_bits(capi, oracle, shape):
    """[N,M] + bias from the gather kernel: through shared memory and TMA stores (`set_epilogue(2)`; what a product with
    several destinations uses) against fp16 stores from registers (default), bit for bit, with ragged N, a last row tile that is partly outside M, one to four vector
    blocks per tile, and against the CPU oracle; a leading dimension that TMA cannot take falls back to register stores."""
    import torch
    M, K, V, m, N = shape
    dense, colloc, values, meta, B = _operands(capi, M, K, V, m, N, seed=M + 3 * K + N)
    prep = capi.Prepared(values, meta, colloc, M, K, V, m, strategy=capi.STRATEGY_GATHER)
    bias = (torch.rand(M, device="cuda") - 0.5).half()
    regs = prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM)
    assert prep.device_status() == 0
    prep.set_epilogue(2)
    canvas = torch.full((N + 2, M), 3.0, dtype=torch.float16, device="cuda")
    tma = prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM, out=canvas[1:N + 1])
    assert prep.device_status() == 0
    assert bool((canvas[0] == 3.0).all()) and bool((canvas[N + 1] == 3.0).all())
    assert torch.equal(tma, regs)
    _check_rows(oracle, tma, 1, values, meta, colloc, M, K, V, m, B, bias=bias, nrows=32)
    # ldo = M + 4 is not a multiple of 8: the same request silently takes the register path
    wide = torch.zeros((N, M + 4), dtype=torch.float16, device="cuda")
    prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM, out=wide[:, :M])
    assert torch.equal(wide[:, :M], regs) and bool((wide[:, M:] == 0).all())
