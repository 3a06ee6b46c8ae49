"""The largest configuration named for this path: M=49152, K=12288, V=128, 2:8 -- the compressor over the whole
matrix, bit for bit against the CPU oracle, and the product on one rank's column shard (N = 32768 / 8)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from venom_b200 import capi
    capi.lib()
    return capi


def test_largest_matrix_compressor_bit_exact_and_shard_product(capi, oracle):
    import torch
    from venom_b200.synth import random_vnm_dense_cuda, vnm_sizes
    M, K, V, m, N = 49152, 12288, 128, 8, 4096
    dense, colloc = random_vnm_dense_cuda(M, K, V, m, seed=4)
    values, meta, bad = capi.compress(dense, colloc, V, m)
    assert bad == 0
    # the round trip is the size-independent property; the oracle comparison is the full-size bit check
    assert torch.equal(capi.decompress(values, meta, colloc, M, K, V, m), dense)
    dense_h = dense.cpu().numpy()
    cols_h = colloc.cpu().numpy().view(np.uint32)
    ov, om, obad = oracle.compress(dense_h, cols_h, V, m)
    assert obad == 0
    assert np.array_equal(values.cpu().numpy().view(np.uint16), ov.view(np.uint16))
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), om)

    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    B = (torch.rand((K, N), device="cuda", generator=g) * 2 - 1).half()
    prep = capi.Prepared(values, meta, colloc, M, K, V, m)
    out = prep.spmm(B)
    rows = np.sort(np.random.default_rng(2).choice(M, size=32, replace=False)).astype(np.int32)
    want = oracle.spmm(ov, om, cols_h, M, K, V, m, B.cpu().numpy(), rows=rows)
    bad, first, worst = oracle.check(out[torch.from_numpy(rows).long().cuda()].cpu().numpy(), want[rows], mode=1, tol=1e-2)
    assert bad == 0, (bad, first, worst)
    # a checksum of checksums over ALL rows: (1^T A) B == 1^T C up to the fp16 rounding of C
    colsum = dense.float().sum(0, keepdim=True) @ B.float()
    got = out.float().sum(0, keepdim=True)
    assert torch.allclose(got, colsum, rtol=2e-3, atol=8.0), float((got - colsum).abs().max())
    assert prep.device_status() == 0
