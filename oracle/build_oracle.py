"""Build the CPU oracle.

* ``oracle/libvnm_oracle.so`` -- the C restatement in ``vnm_oracle.c`` (gcc, OpenMP, F16C).
* ``oracle/_ref/libvnm_ref.so`` -- the reference's own ``Format_sr_nm<__half>`` class, compiled from
  the reference checkout where it lies (only when that checkout is present), with the small
  ``ref_driver.cu`` wrapper.  The reference's host-only format code lives in CUDA-language translation
  units (it includes cuda_fp16.h and calls cudaMalloc in one method), so nvcc is the compiler; C++14
  because it uses std::random_shuffle.

* ``oracle/_ref/libvnm_ref_spatha.so`` -- the reference's own Spatha SpMM kernel (header-only templates under
  ``include/spatha/block_sparse``; legacy ``mma.sp``), compiled for sm_100a with ``ref_spatha_driver.cu``: three
  tile configurations from the reference's instantiation list, one per V.  Used on the GPU box as the second
  comparator of the SpMM parity tests.

All are test infrastructure; the product library never links or loads them.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: VENOM_REFERENCE_DIR, else a directory "reference" next to this repository
REF = os.environ.get("VENOM_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_restatement(force=False):
    src = os.path.join(HERE, "vnm_oracle.c")
    out = os.path.join(HERE, "libvnm_oracle.so")
    if not force and _newer(out, [src]):
        return out
    cmd = ["gcc", "-O3", "-fopenmp", "-mf16c", "-mavx2", "-mfma", "-shared", "-fPIC", "-std=gnu11",
           "-o", out, src, "-lm"]
    subprocess.check_call(cmd)
    return out


def build_reference(force=False):
    """Returns the path of libvnm_ref.so, or None when the reference checkout is absent and no
    prebuilt copy exists."""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libvnm_ref.so")
    fmt = os.path.join(REF, "src", "format")
    srcs = [os.path.join(HERE, "ref_driver.cu"), os.path.join(fmt, "format.cpp"),
            os.path.join(fmt, "format_sr_nm.cpp")]
    if not all(os.path.exists(s) for s in srcs):
        return out if os.path.exists(out) else None
    if not force and _newer(out, srcs):
        return out
    os.makedirs(out_dir, exist_ok=True)
    cmd = ["nvcc", "-std=c++14", "-w", "-O2", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-shared", "-I", os.path.join(REF, "src"), "-o", out] + srcs
    subprocess.check_call(cmd)
    return out


def build_reference_spatha(force=False):
    """Returns the path of libvnm_ref_spatha.so, or None when the reference checkout is absent and no prebuilt copy
    exists.  The reference's CMake build is not used (it needs cuSPARSELt and empty submodules)."""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libvnm_ref_spatha.so")
    inc = os.path.join(REF, "include")
    hdrs = [os.path.join(inc, "spatha", "block_sparse", "spmm", f) for f in ("blockwise_op.h", "blockwise_kernel.h", "blockwise_format.h")]
    src = os.path.join(HERE, "ref_spatha_driver.cu")
    if not all(os.path.exists(s) for s in hdrs + [src]):
        return out if os.path.exists(out) else None
    if not force and _newer(out, hdrs + [src]):
        return out
    os.makedirs(out_dir, exist_ok=True)
    cmd = ["nvcc", "-std=c++14", "-w", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-shared",
           "-I", inc, "-o", out, src]
    subprocess.check_call(cmd, stderr=subprocess.DEVNULL)   # ptxas prints one advisory per mma.sp instruction
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_restatement(force))
    print(build_reference(force))
    print(build_reference_spatha(force))
