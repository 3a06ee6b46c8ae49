"""GPU parity tests of the V:N:M SpMM through the C ABI against the CPU oracle.

Tolerance (stated by the task for this path): |C - C_ref| <= 1e-2 * (|C_ref| + 1) elementwise against the
fp32-accumulate host reference; integer-valued inputs (the reference's own `rand()%9-4` data,
src/format/format_sr_nm.cpp:65) must match exactly, which is stricter than the reference's |a-b| <= 1.0
check (src/benchmark_spmm.cpp:58)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2

# (M, K, V, m, N)
SMALL = [
    (128, 256, 128, 8, 256),     # one tile, one k-tile
    (128, 512, 128, 4, 256),     # pure 2:4, two k-tiles
    (256, 1024, 128, 16, 512),   # several tiles / k-tiles, wide N tile
    (128, 1024, 64, 8, 128),     # two vector blocks per tile
    (192, 768, 64, 8, 200),      # ragged row tile (M % 128 != 0) and ragged N
    (128, 1024, 32, 8, 64),      # four vector blocks per tile
    (96, 512, 32, 32, 72),       # ragged everything
    (128, 280, 64, 10, 128),     # padded Ksp (56 -> 64 compressed columns)
    (64, 99, 32, 8, 64),         # ragged last group (K % m != 0)
    (256, 2000, 128, 20, 264),   # m not a power of two
    (128, 4000, 128, 100, 128),  # very sparse
]


@pytest.fixture(scope="module")
def capi():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from venom_b200 import capi
    capi.lib()
    return capi


def _setup(capi, oracle, M, K, V, m, N, seed, ints):
    import torch
    from venom_b200.synth import random_dense_b, random_vnm_dense
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=seed, integer_values=ints)
    B = random_dense_b(K, N, seed=seed + 1, integer_values=ints)
    ov, om, bad = oracle.compress(dense, cols, V, m)
    assert bad == 0
    v = torch.from_numpy(ov).cuda()
    me = torch.from_numpy(om.view(np.int32)).cuda()
    c = torch.from_numpy(cols.view(np.int32)).cuda()
    prep = capi.Prepared(v, me, c, M, K, V, m)
    return prep, torch.from_numpy(B).cuda(), (ov, om, cols, B)


def _check(oracle, got, want):
    bad, first, worst = oracle.check(got, want, mode=1, tol=REL_TOL)
    assert bad == 0, "%d mismatches, first at %d, max abs err %g" % (bad, first, worst)


@pytest.mark.parametrize("shape", SMALL)
@pytest.mark.parametrize("ints", [True, False])
def test_spmm_matches_oracle(capi, oracle, shape, ints):
    M, K, V, m, N = shape
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=M + K + N, ints=ints)
    out = prep.spmm(Bd)
    assert prep.device_status() == 0
    want = oracle.spmm(ov, om, cols, M, K, V, m, B)
    got = out.cpu().numpy()
    if ints:
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    else:
        _check(oracle, got, want)


@pytest.mark.parametrize("shape", SMALL[:7])
def test_spmm_transposed_output_with_bias(capi, oracle, shape):
    import torch
    M, K, V, m, N = shape
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=7 * M + N, ints=False)
    bias = np.random.default_rng(M).uniform(-1, 1, M).astype(np.float16)
    out = prep.spmm(Bd, bias=torch.from_numpy(bias).cuda(), layout=capi.VNM_LAYOUT_NM)
    assert tuple(out.shape) == (N, M)
    want = oracle.spmm(ov, om, cols, M, K, V, m, B, bias=bias, layout=1)
    _check(oracle, out.cpu().numpy(), want)
    out2 = prep.spmm(Bd, layout=capi.VNM_LAYOUT_NM)       # bias is optional in this library
    _check(oracle, out2.cpu().numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B, layout=1))


def test_spmm_is_deterministic_and_handles_strided_operands(capi, oracle):
    import torch
    M, K, V, m, N = 256, 1024, 64, 8, 384
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=77, ints=False)
    a = prep.spmm(Bd)
    b = prep.spmm(Bd)
    assert torch.equal(a, b)
    wide = torch.zeros((K, N + 64), dtype=torch.float16, device="cuda")
    wide[:, :N] = Bd
    outw = torch.full((M, N + 8), 7.0, dtype=torch.float16, device="cuda")
    prep.spmm(wide[:, :N], out=outw[:, :N])
    assert torch.equal(outw[:, :N], a)
    assert bool((outw[:, N:] == 7.0).all())                # canary columns untouched


def test_spmm_host_buffers_end_to_end(capi, oracle):
    import torch
    M, K, V, m, N = 128, 512, 128, 8, 256
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=123, ints=True)
    Bh = torch.from_numpy(B).pin_memory()
    oh = torch.empty((M, N), dtype=torch.float16).pin_memory()
    prep.spmm_host(Bh, oh)
    want = oracle.spmm(ov, om, cols, M, K, V, m, B)
    assert np.array_equal(oh.numpy().view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("cfg", [(256, 512, 64, 8, 2568, True), (128, 256, 128, 16, 1536, False)])
def test_spmm_host_buffers_in_slices(capi, oracle, cfg):
    """Host-buffer call whose columns go through in several slices (the last one ragged), both layouts, with
    bias, from pinned and from pageable memory: equal to the device-buffer call bit for bit."""
    import torch
    M, K, V, m, N, pinned = cfg
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=5, ints=False)
    bias = np.random.default_rng(9).uniform(-1, 1, M).astype(np.float16)
    Bh = torch.from_numpy(B)
    o_mn, o_nm = torch.empty((M, N), dtype=torch.float16), torch.empty((N, M), dtype=torch.float16)
    if pinned:
        Bh, o_mn, o_nm = Bh.pin_memory(), o_mn.pin_memory(), o_nm.pin_memory()
    prep.spmm_host(Bh, o_mn)
    prep.spmm_host(Bh, o_nm, bias_host=torch.from_numpy(bias), layout=capi.VNM_LAYOUT_NM)
    assert torch.equal(o_mn, prep.spmm(Bd).cpu())
    assert torch.equal(o_nm, prep.spmm(Bd, bias=torch.from_numpy(bias).cuda(), layout=capi.VNM_LAYOUT_NM).cpu())
    _check(oracle, o_nm.numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B, bias=bias, layout=1))


def test_spmm_host_async_calls_overlap_and_match(capi, oracle):
    """Three products queued without waiting (different handles, pinned buffers), collected afterwards."""
    import torch
    cases = [(128, 512, 128, 8, 1280), (256, 256, 64, 8, 2048), (128, 1024, 128, 16, 1024)]
    jobs = []
    for i, (M, K, V, m, N) in enumerate(cases):
        prep, Bd, _ = _setup(capi, oracle, M, K, V, m, N, seed=40 + i, ints=False)
        jobs.append((prep, Bd, Bd.cpu().pin_memory(), torch.empty((M, N), dtype=torch.float16).pin_memory()))
    for prep, Bd, Bh, oh in jobs:
        prep.spmm_host_async(Bh, oh)
    for prep, Bd, Bh, oh in jobs:
        prep.host_wait()
    for prep, Bd, Bh, oh in jobs:
        assert torch.equal(oh, prep.spmm(Bd).cpu())


def test_serialised_weight_loads_and_multiplies(capi, oracle, tmp_path):
    """A compressed weight written to a file and loaded back gives the same product bit for bit."""
    import torch
    from venom_b200 import serialize
    M, K, V, m, N = 256, 512, 64, 8, 264
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=321, ints=False)
    path = tmp_path / "w.vnm"
    path.write_bytes(serialize.dumps(ov, om, cols, M, K, V, m))
    prep2, hdr = serialize.load_prepared(str(path))
    assert (hdr["M"], hdr["K"], hdr["V"], hdr["m"]) == (M, K, V, m)
    assert torch.equal(prep2.spmm(Bd), prep.spmm(Bd))


def test_bounded_wait_expiry_is_reported_and_the_handle_stays_usable(capi, oracle):
    """Failure detection without a fault: a wait on a barrier that nothing signals runs out, the kernel returns,
    the host reads the status, and the next product on the same handle is correct."""
    import torch
    M, K, V, m, N = 128, 512, 128, 8, 256
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=9, ints=True)
    before = prep.spmm(Bd)
    assert prep.device_status() == 0
    prep.selftest_wait_expiry()
    with pytest.raises(capi.VenomError, match="bounded device-side wait"):
        prep.device_status()
    assert prep.device_status() == 0                       # reading the status cleared it
    assert torch.equal(prep.spmm(Bd), before)              # the context and the handle are intact


def test_bad_arguments_raise(capi, oracle):
    import torch
    M, K, V, m, N = 128, 256, 128, 8, 64
    prep, Bd, _ = _setup(capi, oracle, M, K, V, m, N, seed=1, ints=True)
    with pytest.raises(capi.VenomError):
        prep.spmm(Bd[:, :60].contiguous())                # N % 8 != 0
    with pytest.raises(capi.VenomError):
        prep.spmm(torch.zeros((K + 1, N), dtype=torch.float16, device="cuda"))
    with pytest.raises(capi.VenomError):
        prep.spmm(Bd, bias=torch.zeros(M, dtype=torch.float16, device="cuda"))   # bias needs layout NM
    with pytest.raises(capi.VenomError, match="unsupported|supports"):
        from venom_b200.synth import vnm_sizes
        ksp, nv, nm, nc = vnm_sizes(192, 64, 96, 8)
        capi.Prepared(torch.zeros(nv, dtype=torch.float16, device="cuda"), torch.zeros(nm, dtype=torch.int32, device="cuda"),
                      torch.zeros(nc, dtype=torch.int32, device="cuda"), 192, 64, 96, 8)


@pytest.mark.parametrize("shape", [(1024, 4096, 64, 8, 4096), (1024, 1024, 128, 4, 16384), (4096, 1024, 32, 16, 2048)])
def test_spmm_baseline_shapes_sampled_rows(capi, oracle, shape):
    """Headline-sized shapes: a seeded sample of output rows is checked against the oracle, and the
    whole result against linearity (A*(B1+B2) on exactly representable integer data)."""
    import torch
    M, K, V, m, N = shape
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=2024, ints=False)
    out = prep.spmm(Bd).cpu().numpy()
    rows = np.sort(np.random.default_rng(1).choice(M, size=48, replace=False)).astype(np.int32)
    want = oracle.spmm(ov, om, cols, M, K, V, m, B, rows=rows)
    _check(oracle, out[rows], want[rows])
    # linearity on small integers (every partial sum exact): A*B1 + A*B2 == A*(B1+B2)
    prep_i, B1, (iv, im, icols, Bi) = _setup(capi, oracle, M, K, V, m, 256, seed=99, ints=True)
    B2 = torch.roll(B1, 1, dims=0)
    s = prep_i.spmm(B1).float() + prep_i.spmm(B2).float()
    t = prep_i.spmm(B1 + B2).float()
    assert torch.equal(s, t)


def test_gather_modes_agree_when_every_row_is_selected(capi, oracle):
    """m == 4: the 64-row tile loads (default) and the gather4 loads must give identical bits; both
    producer-warp counts too."""
    import torch
    M, K, V, m, N = 256, 1024, 128, 4, 512
    capi.set_strategy(capi.STRATEGY_GATHER)          # the gather-mode switch belongs to the V:N:M form
    try:
        prep, Bd, _ = _setup(capi, oracle, M, K, V, m, N, seed=5, ints=False)
    finally:
        capi.set_strategy(capi.STRATEGY_AUTO)
    a = prep.spmm(Bd)
    prep.set_gather_mode(0)
    b = prep.spmm(Bd)
    prep.set_producer_warps(4)
    c = prep.spmm(Bd)
    assert prep.device_status() == 0
    assert torch.equal(a, b) and torch.equal(a, c)


@pytest.mark.parametrize("shape", [(256, 1024, 128, 8, 512), (256, 2048, 64, 16, 384), (128, 1024, 32, 8, 72), (96, 520, 32, 10, 200),
                                   (2048, 2048, 128, 16, 4096)])
def test_gather_paths_give_identical_bits(capi, oracle, shape):
    """The selected rows of B reach shared memory by per-thread cp.async copies (default), by TMA gather4, or by any
    split of the two; the MMAs and their order do not change, so every variant must produce the same bits."""
    import torch
    M, K, V, m, N = shape
    capi.set_strategy(capi.STRATEGY_GATHER)
    try:
        prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=11 * M + K, ints=False)
    finally:
        capi.set_strategy(capi.STRATEGY_AUTO)
    assert not prep.dense_b_form()
    ref = prep.spmm(Bd)                                   # default: TMA gather4
    if M * N <= 1 << 20:
        _check(oracle, ref.cpu().numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B))
    else:
        rows = np.arange(0, M, 97, dtype=np.int32)
        want = oracle.spmm(ov, om, cols, M, K, V, m, B, rows=rows)
        _check(oracle, ref.cpu().numpy()[rows], want[rows])
    prep.set_gather_mode(3)                               # per-thread cp.async copies, alone and split with TMA gather4
    for split in (0, 16, 32, 48):
        prep.set_gather_split(split)
        assert torch.equal(prep.spmm(Bd), ref), "cp.async + TMA split %d differs" % split
    assert prep.device_status() == 0


@pytest.mark.parametrize("shape", [(128, 512, 128, 4, 256), (256, 1024, 128, 8, 512), (192, 768, 64, 8, 200), (128, 1024, 32, 16, 64),
                                   (96, 512, 32, 32, 72), (256, 2048, 64, 16, 384),
                                   (128, 1000, 64, 8, 520),      # K ends inside a 128-column k-tile; N ends inside the third column tile
                                   (384, 200, 128, 4, 1024)])    # three row tiles (odd), one short k-tile
@pytest.mark.parametrize("strategy", ["gather", "dense_b"])
def test_both_operand_forms_match_oracle(capi, oracle, shape, strategy):
    """The V:N:M gather form and the dense-B form (2:4 over all K columns) are interchangeable."""
    M, K, V, m, N = shape
    capi.set_strategy(capi.STRATEGY_GATHER if strategy == "gather" else capi.STRATEGY_DENSE_B)
    try:
        for ints in (True, False):
            prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=3 * M + K, ints=ints)
            out = prep.spmm(Bd)
            assert prep.device_status() == 0
            want = oracle.spmm(ov, om, cols, M, K, V, m, B)
            if ints:
                assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
            else:
                _check(oracle, out.cpu().numpy(), want)
            import torch
            bias = np.random.default_rng(7).uniform(-1, 1, M).astype(np.float16)
            outT = prep.spmm(Bd, bias=torch.from_numpy(bias).cuda(), layout=capi.VNM_LAYOUT_NM)
            _check(oracle, outT.cpu().numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B, bias=bias, layout=1))
    finally:
        capi.set_strategy(capi.STRATEGY_AUTO)


@pytest.mark.parametrize("shape", [(256, 1024, 64, 8, 384), (384, 512, 128, 4, 200), (128, 2048, 32, 16, 72), (128, 1000, 64, 8, 520)])
def test_transposed_dense_operand_and_tma_store_layouts(capi, oracle, shape):
    """Dense-B form: B given as [N,K] (no transpose copy) must equal the [K,N] call, in both output layouts."""
    import torch
    M, K, V, m, N = shape
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=11 * M + N, ints=False)
    assert prep.dense_b_form()
    bias = np.random.default_rng(3).uniform(-1, 1, M).astype(np.float16)
    bt = Bd.t().contiguous()
    a = prep.spmm(Bd, bias=torch.from_numpy(bias).cuda(), layout=capi.VNM_LAYOUT_NM)
    b = prep.spmm_nk(bt, bias=torch.from_numpy(bias).cuda(), layout=capi.VNM_LAYOUT_NM)
    assert torch.equal(a, b)
    _check(oracle, b.cpu().numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B, bias=bias, layout=1))
    c = prep.spmm_nk(bt, layout=capi.VNM_LAYOUT_MN)
    assert torch.equal(c, prep.spmm(Bd))
    wide = torch.full((N, M + 8), 3.0, dtype=torch.float16, device="cuda")
    prep.spmm_nk(bt, layout=capi.VNM_LAYOUT_NM, out=wide[:, :M])
    assert torch.equal(wide[:, :M], prep.spmm(Bd, layout=capi.VNM_LAYOUT_NM)) and bool((wide[:, M:] == 3.0).all())


def _random_cases(count, seed):
    rng = np.random.default_rng(seed)
    cases = []
    while len(cases) < count:
        V = int(rng.choice([32, 64, 128]))
        M = V * int(rng.integers(1, 7))
        m = int(rng.choice([4, 5, 6, 8, 10, 12, 16, 24, 32, 40, 64]))
        K = int(rng.integers(1, 40)) * m + int(rng.choice([0, 0, 0, 1, 3]))     # mostly K % m == 0, sometimes a ragged last group
        N = 8 * int(rng.integers(1, 90))
        cases.append((M, K, V, m, N))
    return cases


@pytest.mark.parametrize("case", _random_cases(28, seed=2025))
def test_random_shapes_match_oracle(capi, oracle, case):
    """Seeded random shapes, small enough for the CPU oracle: tiny N, K shorter than a k-tile, odd m, single
    vector block ... in both output layouts with bias, whichever operand form the library picks."""
    import torch
    M, K, V, m, N = case
    prep, Bd, (ov, om, cols, B) = _setup(capi, oracle, M, K, V, m, N, seed=M + 3 * K + N, ints=False)
    _check(oracle, prep.spmm(Bd).cpu().numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B))
    bias = np.random.default_rng(M + N).uniform(-1, 1, M).astype(np.float16)
    if not prep.dense_b_form() or M % 8 == 0:
        outT = prep.spmm(Bd, bias=torch.from_numpy(bias).cuda(), layout=capi.VNM_LAYOUT_NM)
        _check(oracle, outT.cpu().numpy(), oracle.spmm(ov, om, cols, M, K, V, m, B, bias=bias, layout=1))
    if prep.dense_b_form() and K % 8 == 0:
        assert torch.equal(prep.spmm_nk(Bd.t().contiguous(), layout=capi.VNM_LAYOUT_MN), prep.spmm(Bd))
    assert prep.device_status() == 0
