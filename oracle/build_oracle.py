"""Build the CPU oracle.

* ``oracle/libvnm_oracle.so`` -- the C restatement in ``vnm_oracle.c`` (gcc, OpenMP, F16C).
* ``oracle/_ref/libvnm_ref.so`` -- the reference's own ``Format_sr_nm<__half>`` class, compiled from
  the reference checkout where it lies (only when that checkout is present), with the small
  ``ref_driver.cu`` wrapper.  The reference's host-only format code lives in CUDA-language translation
  units (it includes cuda_fp16.h and calls cudaMalloc in one method), so nvcc is the compiler; C++14
  because it uses std::random_shuffle.

Both are test infrastructure; the product library never links or loads them.
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


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_restatement(force))
    print(build_reference(force))
