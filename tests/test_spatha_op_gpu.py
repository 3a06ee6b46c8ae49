"""GPU tests of the reference-facing surfaces: the `spatha` torch extension, the SrnmSpmm module that
replaces torch.nn.Linear, and the benchmark_spmm command line."""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def spatha():
    import torch
    assert torch.cuda.is_available()
    import venom_b200
    return venom_b200.spatha_module()


@pytest.mark.parametrize("cfg", [(768, 768, 128, 8, 512), (1024, 1024, 64, 8, 1024), (512, 1024, 32, 16, 256), (256, 512, 128, 4, 128)])
def test_spatha_spmm_matches_dense_product_plus_bias(spatha, oracle, cfg):
    """The reference's only op-level check (end2end/tests.ipynb cells 24-28):
    spatha.spmm(...).T == dense @ rhs + bias."""
    import torch
    from venom_b200.synth import random_dense_b, random_vnm_dense
    M, K, V, m, N = cfg
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=M + N)
    B = random_dense_b(K, N, seed=3)
    ov, om, _ = oracle.compress(dense, cols, V, m)
    values = torch.from_numpy(ov).cuda()
    meta = torch.from_numpy(om.view(np.int32)).cuda()
    idx = torch.from_numpy(cols.view(np.int32)).cuda()
    bias = torch.full((M,), 2.0, dtype=torch.float16, device="cuda")
    rhs = torch.from_numpy(B).cuda()
    out = spatha.spmm(meta, idx, values, rhs, bias, M, K, N, V, 2, m, values.numel(), 0, 32, 4)
    assert tuple(out.shape) == (N, M) and out.dtype == torch.float16
    want = oracle.spmm(ov, om, cols, M, K, V, m, B, bias=bias.cpu().numpy(), layout=1)
    bad, first, worst = oracle.check(out.cpu().numpy(), want, mode=1, tol=1e-2)
    assert bad == 0, (bad, first, worst)
    ref = torch.from_numpy(dense).cuda().float() @ rhs.float() + 2.0
    assert torch.allclose(out.T.float(), ref, rtol=1e-2, atol=1e-2)
    # second call hits the prepared-operand cache and a non-default stream works
    n0 = spatha.cache_size()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        out2 = spatha.spmm(meta, idx, values, rhs, bias, M, K, N, V, 2, m, values.numel(), 0, 32, 4)
    s.synchronize()
    assert spatha.cache_size() == n0 and torch.equal(out, out2)
    # the end-to-end scripts pass `flattened_input.T` (end2end/bert_pytorch.py:133): a transposed view of a
    # [tokens, features] activation must give the same result whether or not the op has to copy it
    act = rhs.t().contiguous()
    out3 = spatha.spmm(meta, idx, values, act.t(), bias, M, K, N, V, 2, m, values.numel(), 0, 32, 4)
    assert torch.equal(out, out3)


def test_spatha_spmm_rejects_bad_arguments(spatha):
    import torch
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    v = torch.zeros(8, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        spatha.spmm(z, z, v, torch.zeros((64, 64), dtype=torch.float16, device="cuda"), None, 64, 64, 64, 32, 2, 8, 8, 0, 32, 4)


def test_srnm_spmm_module_replaces_linear(spatha):
    import torch
    from venom_b200.nmv import SrnmSpmm, linear_to_spmm
    torch.manual_seed(0)
    lin = torch.nn.Linear(1024, 512).half().cuda()
    sp = SrnmSpmm(lin, n=2, m=8, v=64)
    x = (torch.rand((4, 96, 1024), device="cuda") - 0.5).half()
    y = sp(x)
    assert tuple(y.shape) == (4, 96, 512)
    # fixed pattern of the reference sparsifier: columns 0 and 2 of every group of 8
    mask = torch.zeros(1024, device="cuda")
    mask[0::8] = 1
    mask[2::8] = 1
    want = torch.nn.functional.linear(x.float(), lin.weight.float() * mask, lin.bias.float())
    assert torch.allclose(y.float(), want, rtol=2e-2, atol=2e-2)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 256)).half().cuda()
    linear_to_spmm(model, 2, 8, 128)
    assert isinstance(model[0], SrnmSpmm) and isinstance(model[2], SrnmSpmm)
    assert tuple(model(x[..., :256]).shape) == (4, 96, 256)


@pytest.mark.parametrize("flags", [
    "--m 1024 --k 4096 --n 4096 --bm 64 --mm_row 8",
    "--m 1024 --k 1024 --n 2048 --bm 128 --mm_row 4",
    "--m 512 --k 2000 --n 1024 --bm 32 --mm_row 20",
    "--m 1024 --k 1024 --n 2048 --bm 128 --mm_row 8 --strategy gather",
    "--m 1024 --k 1024 --n 2048 --bm 128 --mm_row 16 --strategy dense-b",
    "--m 1024 --k 1024 --n 2048 --bm 128 --mm_row 4 --ablation ideal",
    "--m 1024 --k 2048 --n 2048 --bm 128 --mm_row 16 --ablation cpasync",     # rows gathered by per-thread cp.async instead of TMA gather4
    "--m 1024 --k 2048 --n 2056 --bm 64 --mm_row 8 --ablation out32",         # 32-bit epilogue stores, ragged N
])
def test_benchmark_spmm_cli_check(flags):
    exe = os.path.join(ROOT, "venom_b200", "benchmark_spmm")
    assert os.path.exists(exe), "CLI not built: python -m venom_b200.build"
    cmd = (exe + " --sparsity-type n-to-m --spmm spatha --gemm cuBlas --precision half --meta-block-size 32 --block-size 4 "
           "--nn_row 2 --d 0.5 --bn 64 --bk 32 --wm 32 --wn 64 --wk 32 --mm 16 --mn 8 --mk 32 --nstage 2 --check " + flags)
    r = subprocess.run(cmd.split(), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    cols = r.stdout.strip().splitlines()[-1].split(",")
    assert len(cols) == 26 and cols[0] == "2" and cols[1] == "sm_100a"
    assert cols[23] == "0", "check failed: " + r.stdout
    assert float(cols[20]) > 0 and float(cols[21]) > 0


def test_bert_encoder_harness_small(spatha):
    """Two BERT-large-shaped encoder layers, magnitude-pruned to 64:2:8: the sparse model must agree with a
    dense model whose linear weights were masked the same way."""
    import torch
    from venom_b200 import e2e_bert
    from venom_b200.nmv import SrnmSpmm
    torch.manual_seed(0)
    dense = e2e_bert.build_model(2).half().cuda()
    sparse = e2e_bert.build_model(2).half().cuda()
    sparse.load_state_dict(dense.state_dict())
    assert e2e_bert.sparsify_encoder(sparse, 2, 8, 64) == 12
    # mask the dense twin's weights with what the sparse modules kept
    for (name, mod) in sparse.named_modules():
        if isinstance(mod, SrnmSpmm):
            from venom_b200 import capi
            kept = capi.decompress(mod.values, mod.metadata, mod.columns, mod.nrows_sp, mod.ncols_sp, mod.v, mod.m)
            dict(dense.named_modules())[name].weight.data.copy_(kept)
    ids = torch.randint(0, 30522, (2, 128), device="cuda")
    with torch.no_grad():
        a = dense(ids).last_hidden_state.float()
        b = sparse(ids).last_hidden_state.float()
    assert torch.allclose(a, b, rtol=3e-2, atol=3e-2), (a - b).abs().max()


def test_transposed_view_prepares_dense_b_form_at_high_sparsity(spatha, oracle):
    """At 128:2:32 the automatic choice is the gather form; an activation that arrives as a transposed view
    makes the op prepare the dense-B form instead (read in place).  Both must agree with the oracle."""
    import torch
    from venom_b200 import capi
    from venom_b200.synth import random_dense_b, random_vnm_dense
    M, K, V, m, N = 256, 1024, 128, 32, 512
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=77)
    B = random_dense_b(K, N, seed=78)
    ov, om, _ = oracle.compress(dense, cols, V, m)
    values = torch.from_numpy(ov).cuda()
    meta = torch.from_numpy(om.view(np.int32)).cuda()
    idx = torch.from_numpy(cols.view(np.int32)).cuda()
    act = torch.from_numpy(np.ascontiguousarray(B.T)).cuda()          # [N, K]
    spatha.clear_cache()
    out = spatha.spmm(meta, idx, values, act.t(), None, M, K, N, V, 2, m, values.numel(), 0, 32, 4)
    want = oracle.spmm(ov, om, cols, M, K, V, m, B, layout=1)
    bad, first, worst = oracle.check(out.cpu().numpy(), want, mode=1, tol=1e-2)
    assert bad == 0, (bad, first, worst)
    auto = capi.Prepared(values, meta, idx, M, K, V, m)
    forced = capi.Prepared(values, meta, idx, M, K, V, m, strategy=capi.STRATEGY_DENSE_B)
    assert not auto.dense_b_form() and forced.dense_b_form()
    assert torch.equal(forced.spmm_nk(act, layout=capi.VNM_LAYOUT_NM), out)


def test_gpt_block_sparse_equals_masked_dense_twin(spatha):
    """One GPT-shaped decoder layer pruned by magnitude to 128:2:16: the block whose linears run through the op
    must agree with a dense block whose weights were masked with exactly what the sparse modules kept."""
    import torch
    from venom_b200 import capi, e2e_gpt
    from venom_b200.nmv import SrnmSpmm
    torch.manual_seed(0)
    hidden, heads, ffn = 512, 8, 2048
    with torch.device("cuda"):
        dense = e2e_gpt.build_block(2, hidden, heads, ffn).half()
        sparse = e2e_gpt.build_block(2, hidden, heads, ffn).half()
    sparse.load_state_dict(dense.state_dict())
    assert e2e_gpt.sparsify(sparse, 2, 16, 128, magnitude=True) == 8
    twins = dict(dense.named_modules())
    for name, mod in sparse.named_modules():
        if isinstance(mod, SrnmSpmm):
            kept = capi.decompress(mod.values, mod.metadata, mod.columns, mod.nrows_sp, mod.ncols_sp, mod.v, mod.m)
            assert int((kept != 0).sum()) == mod.nrows_sp * mod.ncols_sp // 8      # 2 of every 16
            twins[name].weight.data.copy_(kept)
    x = torch.randn((2, 256, hidden), device="cuda").half()
    with torch.no_grad():
        a = dense(x).float()
        b = sparse(x).float()
    assert torch.allclose(a, b, rtol=3e-2, atol=3e-2), float((a - b).abs().max())


def test_gpt_block_harness_small(spatha):
    """The decoder-block harness on a small shape: sparse and dense forwards run and print the reference's lines."""
    from venom_b200 import e2e_gpt
    d, s_ = e2e_gpt.main(["-m", "16", "-v", "128", "--layers", "1", "--hidden", "512", "--heads", "8", "--ffn", "2048", "--batch", "2",
                          "--seq", "128", "--repeats", "2"])
    assert d > 0 and s_ > 0


def test_cache_does_not_outlive_the_operand_it_was_built_from(spatha, oracle):
    """A weight is freed and a DIFFERENT one of the same shape lands on the same device addresses (torch's caching
    allocator hands the blocks straight back): the op must multiply with the new weight, not the cached old one."""
    import torch
    from venom_b200.synth import random_dense_b, random_vnm_dense
    M, K, V, m, N = 256, 1024, 64, 8, 256
    B = random_dense_b(K, N, seed=5)
    Bd = torch.from_numpy(B).cuda()
    spatha.clear_cache()
    seen = []
    for seed in (1, 2):
        dense, cols, _ = random_vnm_dense(M, K, V, m, seed=seed)
        ov, om, _ = oracle.compress(dense, cols, V, m)
        values = torch.from_numpy(ov).cuda()
        meta = torch.from_numpy(om.view(np.int32)).cuda()
        idx = torch.from_numpy(cols.view(np.int32)).cuda()
        seen.append((values.data_ptr(), meta.data_ptr(), idx.data_ptr()))
        out = spatha.spmm(meta, idx, values, Bd, None, M, K, N, V, 2, m, values.numel(), 0, 32, 4)
        want = oracle.spmm(ov, om, cols, M, K, V, m, B, layout=1)
        bad, first, worst = oracle.check(out.cpu().numpy(), want, mode=1, tol=1e-2)
        assert bad == 0, "seed %d: %d mismatches (max abs err %g)" % (seed, bad, worst)
        del values, meta, idx, out
    if seen[0] != seen[1]:
        pytest.skip("the allocator did not hand the same addresses back: the stale-entry case was not exercised")
    assert spatha.cache_size() == 1     # the dead entry was released when the new operand arrived
