"""CPU tests of the boundary: the shared library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments with the documented codes (no compute calls)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from venom_b200 import build
    build.build_lib()
    from venom_b200 import capi
    return capi.lib()


def test_every_declared_symbol_is_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "venom_b200.h")).read()
    names = set(re.findall(r"\b(vnm_[a-z0-9_]+)\s*\(", hdr))
    assert {"vnm_sizes", "vnm_compress_f16", "vnm_decompress_f16", "vnm_prepare", "vnm_spmm_f16", "vnm_spmm_f16_host",
            "vnm_destroy", "vnm_last_error_string"} <= names
    for n in names:
        assert hasattr(lib, n), n


def test_sizes_and_argument_errors(lib):
    from venom_b200 import capi
    from venom_b200.synth import vnm_sizes
    for shape in [(1024, 4096, 64, 8), (49152, 12288, 128, 8), (128, 280, 64, 10), (64, 99, 32, 8)]:
        assert capi.sizes(*shape) == vnm_sizes(*shape)
    with pytest.raises(capi.VenomError, match="multiple of V"):
        capi.sizes(100, 64, 64, 8)
    with pytest.raises(capi.VenomError, match="n must be 2"):
        capi.sizes(128, 64, 64, 8, n=1)
    # null pointers are rejected before any CUDA call
    rc = lib.vnm_compress_f16(None, 64, None, None, 64, 64, 32, 2, 8, None, None, None, None)
    assert rc == 1 and b"null" in lib.vnm_last_error_string()
    h = C.c_void_p()
    rc = lib.vnm_prepare(None, None, None, 64, 64, 32, 2, 8, C.byref(h), None)
    assert rc == 1
    out = C.c_int64()
    assert lib.vnm_prepared_bytes(192, 64, 96, 2, 8, C.byref(out)) == 3      # valid format, unsupported by the SpMM
    assert lib.vnm_prepared_bytes(128, 4096, 128, 2, 8, C.byref(out)) == 0 and out.value > 128 * 1024 * 2


def test_cpu_tensors_are_rejected():
    import torch
    from venom_b200 import capi
    with pytest.raises(capi.VenomError, match="no CPU path"):
        capi.compress(torch.zeros(64, 64, dtype=torch.float16), torch.zeros(64, dtype=torch.int32), 32, 8)


def test_handle_setters_and_launcher_entry_points_reject_bad_arguments_without_a_gpu(lib):
    """Every switch and every vnm_mgpu_* entry point checks its arguments before touching CUDA or NCCL."""
    import ctypes as C
    for name in ("vnm_set_gather_mode", "vnm_set_gather_split", "vnm_set_pair_mode", "vnm_set_l2_prefetch", "vnm_set_host_slices", "vnm_set_epilogue", "vnm_set_max_ctas",
                 "vnm_set_producer_warps"):
        fn = getattr(lib, name)
        fn.argtypes = [C.c_void_p, C.c_int]
        fn.restype = C.c_int
        assert fn(None, 0) == 1 and b"null handle" in lib.vnm_last_error_string(), name
    lo, hi = C.c_int(), C.c_int()
    assert lib.vnm_mgpu_shard(64, 2, 1, 8, C.byref(lo), C.byref(hi)) == 0 and (lo.value, hi.value) == (32, 64)
    assert lib.vnm_mgpu_shard(60, 2, 1, 8, C.byref(lo), C.byref(hi)) == 1
    ctx = C.c_void_p()
    assert lib.vnm_mgpu_create(None, 2, 0, C.byref(ctx)) == 1
    assert lib.vnm_mgpu_create_from_comm(None, C.byref(ctx)) == 1
    assert lib.vnm_mgpu_unique_id(None) == 1
    assert lib.vnm_mgpu_destroy(None) == 0
    assert lib.vnm_mgpu_spmm_gathered(None, None, None, 0, 64, None, None, 0, 4, None) == 1
    assert lib.vnm_mgpu_broadcast_operand(None, None, None, None, 64, 64, 32, 2, 8, 0, None) == 1
    assert lib.vnm_mgpu_register_output(None, None, 0) == 1
    assert lib.vnm_mgpu_unregister_output(None, None) == 1
    assert lib.vnm_mgpu_spmm_gathered_p2p(None, None, None, 0, 64, None, None, 0, None) == 1
    assert lib.vnm_spmm_f16_multi(None, None, 0, 64, None, None, 0, 0, 0, None) == 1
