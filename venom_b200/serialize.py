"""Serialised form of a V:N:M compressed weight: one file = header + values | metadata | column-loc.

The three arrays are the reference's format bit for bit (src/format/format_sr_nm.cpp:53-60 for the sizes,
:441-536 for the element order), so a file written here can be consumed by the reference's device upload
(which concatenates metadata and column-loc the same way, format_sr_nm.cpp:262-284) and vice versa.  Loading
re-packs once into the kernel-private layout (`capi.Prepared`); nothing is re-compressed at start-up.

Layout (little endian):
    0   8 bytes   magic  b"VNMSRNM1"
    8   9 x int64  M, K, V, n, m, Ksp, values_elems, meta_words, colloc_words
    80  uint64     CRC-32 (zlib) of the payload, zero-extended
    88  40 bytes   reserved (zero)
    128 payload    values (fp16) | metadata (uint32) | column-loc (uint32), each padded to 16 bytes
"""
import struct
import zlib

import numpy as np

from .synth import vnm_sizes

MAGIC = b"VNMSRNM1"
HEADER_BYTES = 128


def _pad16(n):
    return -(-n // 16) * 16


def _checksum(data):
    return zlib.crc32(data) & 0xFFFFFFFF


def dumps(values, metadata, columns, M, K, V, m, n=2):
    """values fp16 [M*Ksp], metadata / columns 32-bit; numpy arrays or anything np.asarray accepts."""
    ksp, nv, nm, nc = vnm_sizes(M, K, V, m, n)
    v = np.ascontiguousarray(np.asarray(values).reshape(-1)).view(np.uint16)
    me = np.ascontiguousarray(np.asarray(metadata).reshape(-1)).view(np.uint32)
    co = np.ascontiguousarray(np.asarray(columns).reshape(-1)).view(np.uint32)
    if v.size != nv or me.size != nm or co.size != nc:
        raise ValueError("array sizes do not match the format (%d, %d, %d expected)" % (nv, nm, nc))
    parts = []
    for a in (v, me, co):
        raw = a.tobytes()
        parts.append(raw + b"\0" * (_pad16(len(raw)) - len(raw)))
    payload = b"".join(parts)
    header = MAGIC + struct.pack("<9q", M, K, V, n, m, ksp, nv, nm, nc) + struct.pack("<Q", _checksum(payload))
    return header + b"\0" * (HEADER_BYTES - len(header)) + payload


def loads(blob):
    """Returns (values fp16, metadata uint32, columns uint32, dict(M, K, V, n, m, Ksp)); raises ValueError on a bad file."""
    if len(blob) < HEADER_BYTES or blob[:8] != MAGIC:
        raise ValueError("not a V:N:M weight file")
    M, K, V, n, m, ksp, nv, nm, nc = struct.unpack("<9q", blob[8:80])
    (check,) = struct.unpack("<Q", blob[80:88])
    if (ksp, nv, nm, nc) != vnm_sizes(M, K, V, m, n):
        raise ValueError("header sizes do not match the format")
    o1 = HEADER_BYTES
    o2 = o1 + _pad16(nv * 2)
    o3 = o2 + _pad16(nm * 4)
    end = o3 + _pad16(nc * 4)
    if len(blob) != end:
        raise ValueError("truncated or oversized file: %d bytes, expected %d" % (len(blob), end))
    if _checksum(blob[HEADER_BYTES:]) != check:
        raise ValueError("checksum mismatch")
    values = np.frombuffer(blob, dtype=np.float16, count=nv, offset=o1).copy()
    metadata = np.frombuffer(blob, dtype=np.uint32, count=nm, offset=o2).copy()
    columns = np.frombuffer(blob, dtype=np.uint32, count=nc, offset=o3).copy()
    return values, metadata, columns, dict(M=M, K=K, V=V, n=n, m=m, Ksp=ksp)


def save(path, tensor):
    """tensor: an nmv.SrNMTensor (or any object with values / metadata / columns / nrows / ncols / tileM / m / n)."""
    blob = dumps(tensor.values.detach().cpu().numpy(), tensor.metadata.cpu().numpy(), tensor.columns.cpu().numpy(),
                 tensor.nrows, tensor.ncols, tensor.tileM, tensor.m, tensor.n)
    with open(path, "wb") as f:
        f.write(blob)


def load_prepared(path, device="cuda", strategy=None):
    """Reads a file and re-packs it once for the kernels: returns (capi.Prepared, header dict)."""
    import torch
    from . import capi
    with open(path, "rb") as f:
        values, metadata, columns, hdr = loads(f.read())
    v = torch.from_numpy(values).to(device)
    me = torch.from_numpy(metadata.view(np.int32)).to(device)
    co = torch.from_numpy(columns.view(np.int32)).to(device)
    return capi.Prepared(v, me, co, hdr["M"], hdr["K"], hdr["V"], hdr["m"], hdr["n"], strategy=strategy), hdr
