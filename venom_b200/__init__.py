"""venom_b200: a Blackwell (sm_100a) implementation of the V:N:M sparse x dense product (Spatha),
its dense->V:N:M compressor and an N-sharded multi-GPU launcher, behind a C ABI."""
import importlib
import os
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))


def spatha_module():
    """The `spatha` torch extension (same name and spmm() signature as the reference's).  Built in-tree
    by `python -m venom_b200.build`; importing it fails loudly if it is missing."""
    if "spatha" in sys.modules:
        return sys.modules["spatha"]
    import torch  # noqa: F401  (libtorch must be loaded first)
    if _PKG not in sys.path:
        sys.path.insert(0, _PKG)
    try:
        return importlib.import_module("spatha")
    except ImportError as e:
        raise ImportError("the `spatha` extension is not built: run `python -m venom_b200.build` (%s)" % e)
