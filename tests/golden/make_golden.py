"""Generate the golden vectors under tests/golden/ from the REFERENCE implementation.

Run in a container where the reference checkout is mounted:
    python tests/golden/make_golden.py
It needs (a) oracle/_ref/libvnm_ref.so, built by oracle/build_oracle.py from the reference's
src/format/{format,format_sr_nm}.cpp, for the compressor / decompressor vectors and (b) the reference's
end2end/grouped_nmv_tensor.py (imported from the checkout) for the magnitude-pruner vectors.
Inputs come from venom_b200.synth (seeded numpy), outputs from the reference; both are stored so the
tests need neither the reference nor this script at run time.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("VENOM_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))

from oracle.oracle import Reference  # noqa: E402
from venom_b200.synth import random_vnm_dense  # noqa: E402

# (M, K, V, m, integer_values): small shapes covering V in {32,64,128}, m in {4,7,8,10,16,32},
# a padded Ksp (280/10 -> 56 -> 64) and ragged last groups (K % m in {1? no, 2,3,4}).
FORMAT_CASES = [
    (64, 64, 32, 4, False),
    (64, 128, 64, 8, False),
    (128, 256, 64, 8, True),
    (128, 256, 128, 16, False),
    (256, 512, 128, 32, False),
    (128, 280, 64, 10, False),
    (64, 140, 32, 7, True),
    (64, 100, 32, 8, False),
    (64, 99, 32, 8, False),
    (64, 98, 32, 8, False),
]
PRUNE_CASES = [(64, 64, 32, 8, False), (128, 128, 64, 8, True), (128, 64, 128, 16, True), (64, 32, 32, 4, True)]


def main():
    ref = Reference.load()
    assert ref is not None, "reference library not built"
    out = {}
    for i, (M, K, V, m, ints) in enumerate(FORMAT_CASES):
        dense, cols, mask = random_vnm_dense(M, K, V, m, seed=1000 + i, integer_values=ints)
        values, meta = ref.compress(dense, cols, V, m)
        back = ref.to_dense(values, meta, cols, M, K, V, m)
        p = "fmt%d_" % i
        out[p + "shape"] = np.array([M, K, V, m], dtype=np.int32)
        out[p + "dense"] = dense.view(np.uint16)
        out[p + "columns"] = cols
        out[p + "values"] = values.view(np.uint16)
        out[p + "meta"] = meta
        out[p + "to_dense"] = back.view(np.uint16)
    # the reference's own random instances (libc rand stream after srand(seed))
    for i, (M, K, V, m) in enumerate([(128, 256, 64, 8), (128, 280, 64, 10), (64, 512, 32, 16)]):
        values, meta, cols = ref.random_init(M, K, V, m, 2022 + i)
        back = ref.to_dense(values, meta, cols, M, K, V, m)
        p = "rnd%d_" % i
        out[p + "shape"] = np.array([M, K, V, m], dtype=np.int32)
        out[p + "values"] = values.view(np.uint16)
        out[p + "meta"] = meta
        out[p + "columns"] = cols
        out[p + "to_dense"] = back.view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "format_golden.npz"), **out)

    sys.path.insert(0, os.path.join(REF, "end2end"))
    import tempfile
    import torch
    # the reference pruner JIT-compiles its embedded C++ into ./.compile_cache: keep that out of this repository
    os.chdir(tempfile.mkdtemp(prefix="vnm_golden_"))
    import grouped_nmv_tensor as G
    out = {}
    for i, (M, K, V, m, quant) in enumerate(PRUNE_CASES):
        rng = np.random.default_rng(500 + i)
        w = rng.normal(0, 0.02, (M, K)).astype(np.float32)
        if quant:
            w = (np.round(w * 100) / 100).astype(np.float32)      # many exact ties
        masks, cols = G.nm_vector_mask_sparsify(torch.from_numpy(w), 2, m, V)
        p = "prn%d_" % i
        out[p + "shape"] = np.array([M, K, V, m], dtype=np.int32)
        out[p + "w"] = w
        out[p + "mask"] = masks.numpy().astype(np.int8)
        out[p + "columns"] = cols.numpy().astype(np.uint32)
    np.savez_compressed(os.path.join(HERE, "prune_golden.npz"), **out)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
