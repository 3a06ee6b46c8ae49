"""The no-allocation entry point, vnm_spmm_f16_noalloc, against the regular vnm_prepare + vnm_spmm_f16 path.

Who needs it: callers that are not allowed to grow device memory -- a serving process whose framework has
taken the whole GPU for its own pool, a plug-in inside another component's memory budget, a loop that cannot
accept the device-wide synchronisation that cudaMalloc / cudaFree bring.  The entry point keeps the re-packed
sparse operand in an array built into the library, so this test calls it twice in a row with different
operands (the array is shared and keeps old contents) and compares each result with the regular path, which
is itself checked against the CPU oracle elsewhere, and with the CPU oracle's product of the same operands.
"Allocates nothing" is checked where it can be seen from outside the library: the device's free memory
(cudaMemGetInfo, which also sees a cudaMalloc made inside the library) is the same before and after each
call once a first call has done the per-device set-up.  The file name makes pytest collect it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, values, meta, cols, M, K, V, m, B, out, bias=None, layout=0):
    import torch
    lib.vnm_spmm_f16_noalloc.restype = C.c_int
    lib.vnm_spmm_f16_noalloc.argtypes = ([C.c_void_p] * 3 + [C.c_int] * 5 + [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int, C.c_void_p])
    return lib.vnm_spmm_f16_noalloc(values.data_ptr(), meta.data_ptr(), cols.data_ptr(), M, K, V, 2, m, B.data_ptr(), B.stride(0),
                                    B.shape[1], None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0), layout,
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))


def _operands(oracle, M, K, V, m, N, seed):
    import torch
    from venom_b200.synth import random_dense_b, random_vnm_dense
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=seed)
    ov, om, bad = oracle.compress(dense, cols, V, m)
    assert bad == 0
    B = random_dense_b(K, N, seed + 1)
    return (torch.from_numpy(ov).cuda(), torch.from_numpy(om.view(np.int32)).cuda(), torch.from_numpy(cols.view(np.int32)).cuda(),
            torch.from_numpy(B).cuda(), (ov, om, cols, B))


def test_noalloc_matches_regular_path_on_two_calls_in_a_row(oracle):
    import torch
    assert torch.cuda.is_available()
    from venom_b200 import capi
    lib = capi.lib()
    # two different operands back to back: the second call must not see anything of the first
    cases = [(512, 2048, 64, 8, 384, 0), (256, 1024, 128, 16, 264, 1), (512, 2048, 64, 8, 384, 0)]
    for i, (M, K, V, m, N, layout) in enumerate(cases):
        values, meta, cols, B, (ov, om, hcols, hB) = _operands(oracle, M, K, V, m, N, seed=M + N)
        bias = (torch.rand(M, device="cuda") - 0.5).half() if layout == 1 else None
        # the built-in-scratch entry point always uses the gather form of the operand; ask the regular
        # path for the same form so that the two results can be compared bit for bit
        capi.set_strategy(capi.STRATEGY_GATHER)
        try:
            want = capi.Prepared(values, meta, cols, M, K, V, m).spmm(B, bias=bias, layout=layout)
        finally:
            capi.set_strategy(capi.STRATEGY_AUTO)
        got = torch.full_like(want, float("nan"))
        if i == 0:
            # the first call on a device looks up the scratch array's address and sets kernel attributes
            assert _call_noalloc(lib, values, meta, cols, M, K, V, m, B, got, bias=bias, layout=layout) == 0
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = _call_noalloc(lib, values, meta, cols, M, K, V, m, B, got, bias=bias, layout=layout)
        free_after, _ = torch.cuda.mem_get_info()
        assert rc == 0
        assert free_after == free_before, "the call changed the device's free memory by %d bytes" % (free_before - free_after)
        # same kernel, same re-pack: the results are required to be identical, which is within the
        # |C - C_ref| <= 1e-2 * (|C_ref| + 1) tolerance the SpMM tests use
        assert torch.equal(got, want)
        # and against the CPU oracle's product of the same operands
        ref = oracle.spmm(ov, om, hcols, M, K, V, m, hB, bias=None if bias is None else bias.cpu().numpy(), layout=layout)
        bad, _, worst = oracle.check(got.cpu().numpy(), ref, mode=1, tol=1e-2)
        assert bad == 0, "%d mismatches against the CPU oracle (max abs err %g)" % (bad, worst)


def test_noalloc_rejects_operands_beyond_the_built_in_scratch(oracle, capfd):
    import torch
    from venom_b200 import capi
    lib = capi.lib()
    M, K, V, m, N = 4096, 4096, 128, 4, 64          # re-packed form is about 19 MB > 8 MiB
    from venom_b200.synth import vnm_sizes
    ksp, nv, nm, nc = vnm_sizes(M, K, V, m)
    values = torch.zeros(nv, dtype=torch.float16, device="cuda")
    meta = torch.zeros(nm, dtype=torch.int32, device="cuda")
    cols = torch.zeros(nc, dtype=torch.int32, device="cuda")
    B = torch.zeros((K, N), dtype=torch.float16, device="cuda")
    out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    rc = _call_noalloc(lib, values, meta, cols, M, K, V, m, B, out)
    assert rc == 3                                   # VNM_ERR_UNSUPPORTED
    err = capfd.readouterr().err
    assert "too large" in err and "8388608" in err
    assert b"too large" in lib.vnm_last_error_string()   # the same message through the library's error string
