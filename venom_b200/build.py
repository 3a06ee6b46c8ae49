"""In-tree build of the CUDA library (sm_100a only).

    python -m venom_b200.build [--force] [--verbose]

Produces venom_b200/libvenom_b200.so (the C ABI of include/venom_b200.h) with nvcc.  The torch
extension `spatha` and the `benchmark_spmm` CLI are thin wrappers that link against it; they are built
by build_spatha() / build_cli().
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libvenom_b200.so")
CLI = os.path.join(PKG, "benchmark_spmm")

NVCC_BASE = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
NVCC_FLAGS = NVCC_BASE + ["--use_fast_math"]
# Translation units whose floating-point results are compared bit for bit with the reference are built WITHOUT
# --use_fast_math: the magnitude pruner sums fp32 scores, and flush-to-zero would change them for denormal weights.
EXACT_FP_UNITS = {"vnm_prune.cu"}
OBJ_DIR = os.path.join(PKG, "build")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources():
    cu = [os.path.join(CSRC, f) for f in ("vnm_format.cu", "vnm_prune.cu", "vnm_spmm.cu", "vnm_spmm_dense_b.cu", "vnm_spmm_dense_b2.cu", "vnm_capi.cu", "vnm_noalloc.cu", "vnm_mgpu.cu")]
    hdr = [os.path.join(CSRC, f) for f in ("vnm_common.cuh", "vnm_internal.h")] + [os.path.join(ROOT, "include", "venom_b200.h")]
    return cu, hdr


def build_lib(force=False, verbose=False):
    """Compiles every translation unit to an object file (in parallel, only the stale ones) and links them."""
    from concurrent.futures import ThreadPoolExecutor
    cu, hdr = _sources()
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs, objs = [], []
    for src in cu:
        name = os.path.basename(src)
        obj = os.path.join(OBJ_DIR, name[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdr):
            flags = NVCC_BASE if name in EXACT_FP_UNITS else NVCC_FLAGS
            jobs.append(["nvcc"] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            list(ex.map(subprocess.check_call, jobs))
    if jobs or not os.path.exists(LIB) or _stale(LIB, objs):
        subprocess.check_call(["nvcc"] + NVCC_BASE + ["-shared", "-o", LIB] + objs + ["-lcudart", "-ldl"])
    return LIB


def build_cli(force=False):
    src = os.path.join(CSRC, "benchmark_spmm.cpp")
    if not os.path.exists(src):
        return None
    build_lib(force)
    if not force and not _stale(CLI, [src, LIB]):
        return CLI
    cmd = ["nvcc"] + NVCC_FLAGS + ["-x", "cu", "-o", CLI, src, "-L" + PKG, "-lvenom_b200", "-lcublas", "-lcudart",
                                    "-Xlinker", "-rpath=$ORIGIN"]
    subprocess.check_call(cmd)
    return CLI


def build_spatha(force=False):
    """pybind torch extension `spatha` (same module name and spmm() signature as the reference's
    end2end/spatha_mod extension).  Built in-tree next to this file."""
    src = os.path.join(CSRC, "spatha_torch.cpp")
    if not os.path.exists(src):
        return None
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    build_lib(force)
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(PKG, "spatha" + suffix)
    if not force and not _stale(out, [src, LIB]):
        return out
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include"]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", abi, "-DTORCH_EXTENSION_NAME=spatha",
           "-DTORCH_API_INCLUDE_EXTENSION_H"] + inc + ["-o", out, src, "-L" + PKG, "-lvenom_b200",
           "-L" + tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
           "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    subprocess.check_call(cmd)
    return out


def build_all(force=False, verbose=False):
    outs = [build_lib(force, verbose)]
    outs.append(build_cli(force))
    outs.append(build_spatha(force))
    return outs


if __name__ == "__main__":
    print(build_all("--force" in sys.argv, "--verbose" in sys.argv))
