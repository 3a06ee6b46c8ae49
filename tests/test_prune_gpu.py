"""GPU parity of the magnitude pruner (vnm_prune_magnitude_f32) against the CPU oracle and the golden
vectors produced by the reference's group_n_m2."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    import torch
    assert torch.cuda.is_available()
    from venom_b200 import capi
    capi.lib()
    return capi


@pytest.mark.parametrize("shape", [(128, 256, 64, 8), (256, 128, 128, 16), (64, 128, 32, 4), (64, 64, 64, 32), (128, 280, 64, 10)])
def test_prune_matches_oracle_on_continuous_weights(capi, oracle, shape):
    import torch
    M, K, V, m = shape
    w = np.random.default_rng(M + K).normal(0, 0.02, (M, K)).astype(np.float32)
    mask, cols = capi.prune_magnitude(torch.from_numpy(w).cuda(), V, m)
    omask, ocols = oracle.prune(np.abs(w), V, m)
    assert np.array_equal(cols.cpu().numpy().view(np.uint32), ocols)
    assert np.array_equal(mask.cpu().numpy(), omask)
    # the pruned matrix compresses without violations and round-trips
    dense = (torch.from_numpy(w).cuda() * mask).half()
    dense[(dense == 0) & (mask != 0)] = 6e-8          # kept entries that underflow in fp16 stay representable
    values, meta, bad = capi.compress(dense, cols, V, m, mask=mask)
    assert bad == 0
    assert torch.equal(capi.decompress(values, meta, cols, M, K, V, m), dense)


@pytest.mark.parametrize("i", range(4))
def test_prune_matches_reference_golden(capi, golden_prune, i):
    """Golden vectors from the reference pruner; cases 1-3 contain many exact ties.  Columns must always
    match; the mask may differ only in rows whose candidates tie (see the kernel's header)."""
    import torch
    p = "prn%d_" % i
    M, K, V, m = (int(x) for x in golden_prune[p + "shape"])
    w = golden_prune[p + "w"]
    mask, cols = capi.prune_magnitude(torch.from_numpy(w).cuda(), V, m)
    assert np.array_equal(cols.cpu().numpy().view(np.uint32), golden_prune[p + "columns"])
    got = mask.cpu().numpy()
    want = golden_prune[p + "mask"].astype(np.int32)
    assert got.sum() == want.sum()
    diff_rows, diff_groups = np.nonzero((got != want).reshape(M, K // m, m).any(axis=2))
    a = np.abs(w).reshape(M, K // m, m)
    for r, g in zip(diff_rows, diff_groups):
        c4 = golden_prune[p + "columns"].reshape(M // V, -1, 4)[r // V, g]
        v = np.sort(a[r, g, c4])[::-1]
        assert v[1] == v[2], "mask differs from the reference in a row without a tie"
    if i == 0:
        assert len(diff_rows) == 0


def test_magnitude_sparsifier_feeds_the_spmm(capi, oracle):
    import torch
    from venom_b200.nmv import MagnitudeSparsifier
    torch.manual_seed(1)
    W = (torch.randn(256, 512, device="cuda") * 0.02)
    t = MagnitudeSparsifier(2, 8, 64)(W)
    assert t.violations == 0
    dense = t.to_dense()
    kept = (dense != 0).float().mean().item()
    assert abs(kept - 0.25) < 0.01
    x = (torch.rand(512, 128, device="cuda") - 0.5).half()
    out = t.prepared().spmm(x)
    assert torch.allclose(out.float(), dense.float() @ x.float(), rtol=1e-2, atol=1e-2)
    # magnitude pruning keeps at least as much |w| as the fixed pattern
    from venom_b200.nmv import NMVectorSparsifier
    fixed = NMVectorSparsifier(2, 8, 64)(W).to_dense()
    assert dense.float().abs().sum() >= fixed.float().abs().sum()
