"""The header-only C++ shim (include/venom_b200_spatha.hpp): compiles against the C ABI on any host, runs on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "venom_b200")
EXE = os.path.join(PKG, "build", "shim_check")


def _build():
    from venom_b200 import build
    build.build_lib()
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    src = os.path.join(ROOT, "tests", "shim_check.cpp")
    hdrs = [os.path.join(ROOT, "include", h) for h in ("venom_b200_spatha.hpp", "venom_b200.h")]
    if os.path.exists(EXE) and all(os.path.getmtime(p) <= os.path.getmtime(EXE) for p in [src] + hdrs):
        return EXE
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include", "-o", EXE, src,
           "-L" + PKG, "-lvenom_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + PKG, "-Wl,-rpath,/usr/local/cuda/lib64"]
    subprocess.check_call(cmd)
    return EXE


def test_shim_compiles_and_links_with_a_plain_host_compiler():
    assert os.path.exists(_build())


@pytest.mark.gpu
def test_shim_program_runs_on_the_gpu():
    exe = EXE if os.path.exists(EXE) else _build()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "shim ok" in r.stdout, (r.returncode, r.stdout, r.stderr)
