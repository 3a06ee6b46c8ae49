"""Serialised compressed-weight files: round trip, reference-format sizes, corruption detection (CPU only)."""
import numpy as np
import pytest

from venom_b200 import serialize
from venom_b200.synth import random_vnm_dense, vnm_sizes


@pytest.mark.parametrize("shape", [(64, 128, 32, 8), (128, 280, 64, 10), (256, 512, 128, 16)])
def test_round_trip_is_bit_exact(oracle, shape):
    M, K, V, m = shape
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=5)
    values, meta, bad = oracle.compress(dense, cols, V, m)
    blob = serialize.dumps(values, meta, cols, M, K, V, m)
    ksp, nv, nm, nc = vnm_sizes(M, K, V, m)
    assert len(blob) == serialize.HEADER_BYTES + sum(-(-x // 16) * 16 for x in (2 * nv, 4 * nm, 4 * nc))
    v2, m2, c2, hdr = serialize.loads(blob)
    assert hdr == dict(M=M, K=K, V=V, n=2, m=m, Ksp=ksp)
    assert np.array_equal(v2.view(np.uint16), values.view(np.uint16))
    assert np.array_equal(m2, meta) and np.array_equal(c2, cols)
    # the arrays still decompress to the original matrix
    assert np.array_equal(oracle.to_dense(v2, m2, c2, M, K, V, m).view(np.uint16), dense.view(np.uint16))


def test_bad_files_are_rejected(oracle):
    M, K, V, m = 64, 128, 32, 8
    dense, cols, _ = random_vnm_dense(M, K, V, m, seed=6)
    values, meta, _ = oracle.compress(dense, cols, V, m)
    blob = bytearray(serialize.dumps(values, meta, cols, M, K, V, m))
    with pytest.raises(ValueError, match="not a V:N:M"):
        serialize.loads(b"garbage" + bytes(blob))
    with pytest.raises(ValueError, match="truncated"):
        serialize.loads(bytes(blob[:-16]))
    flipped = bytearray(blob)
    flipped[serialize.HEADER_BYTES + 40] ^= 0x10
    with pytest.raises(ValueError, match="checksum"):
        serialize.loads(bytes(flipped))
    with pytest.raises(ValueError, match="sizes"):
        serialize.dumps(values[:-1], meta, cols, M, K, V, m)
