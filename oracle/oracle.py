"""ctypes front-end of the CPU oracle.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline legs of
bench.py.  The product package (venom_b200) never imports this module.

``Oracle``   -- the C restatement (oracle/vnm_oracle.c).
``Reference``-- the reference's own Format_sr_nm<__half> class compiled from the reference checkout
                (oracle/_ref/libvnm_ref.so); available only where that library was built.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

_i64p = C.POINTER(C.c_int64)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def sizes(M, K, V, m, n=2):
    """(Ksp, values_elems, meta_words, colloc_words); format_sr_nm.cpp:53-60 of the reference."""
    if n != 2 or m < 4 or M % V or V % 32:
        raise ValueError("unsupported V:N:M shape")
    ksp = -(-(-(-K // m) * 2) // 16) * 16
    return ksp, M * ksp, (M // 2) * (ksp // 8), (M // V) * (ksp // 2) * 4


class Oracle:
    def __init__(self, build=True):
        path = os.path.join(HERE, "libvnm_oracle.so")
        if build:
            from . import build_oracle
            path = build_oracle.build_restatement()
        self.lib = C.CDLL(path)
        L = self.lib
        L.vnm_oracle_compress_f16.restype = C.c_int64
        L.vnm_oracle_compress_f16.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5 + [C.c_void_p] * 2
        L.vnm_oracle_to_dense_f16.restype = C.c_int
        L.vnm_oracle_to_dense_f16.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5 + [C.c_void_p]
        L.vnm_oracle_spmm_f16.restype = C.c_int
        L.vnm_oracle_spmm_f16.argtypes = ([C.c_void_p] * 3 + [C.c_int] * 5 + [C.c_void_p, C.c_int, C.c_int64,
                                          C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int])
        L.vnm_oracle_dense_gemm_f16.restype = C.c_int
        L.vnm_oracle_dense_gemm_f16.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p, C.c_int]
        L.vnm_oracle_check.restype = C.c_int64
        L.vnm_oracle_check.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_float, _i64p,
                                       C.POINTER(C.c_float)]
        L.vnm_oracle_prune.restype = C.c_int
        L.vnm_oracle_prune.argtypes = [C.c_void_p] + [C.c_int] * 5 + [C.c_void_p] * 2
        L.vnm_oracle_num_threads.restype = C.c_int

    def num_threads(self):
        return int(self.lib.vnm_oracle_num_threads())

    def set_num_threads(self, n):
        """Explicit OpenMP thread count (overrides an inherited OMP_NUM_THREADS); returns the count in effect."""
        self.lib.vnm_oracle_set_num_threads(int(n))
        return self.num_threads()

    def compress(self, dense, columns, V, m, mask=None):
        """dense: [M,K] float16; columns: uint32 column-loc.  Returns (values f16, meta u32, violations)."""
        M, K = dense.shape
        ksp, nv, nm, nc = sizes(M, K, V, m)
        dense = np.ascontiguousarray(dense, dtype=np.float16)
        columns = np.ascontiguousarray(columns, dtype=np.uint32)
        assert columns.size == nc
        if mask is not None:
            mask = np.ascontiguousarray(mask, dtype=np.int32)
        values = np.empty(nv, dtype=np.float16)
        meta = np.empty(nm, dtype=np.uint32)
        bad = self.lib.vnm_oracle_compress_f16(_ptr(dense), _ptr(mask), _ptr(columns), M, K, V, 2, m,
                                               _ptr(values), _ptr(meta))
        if bad < 0:
            raise ValueError("bad shape")
        return values, meta, int(bad)

    def to_dense(self, values, meta, columns, M, K, V, m):
        dense = np.empty((M, K), dtype=np.float16)
        rc = self.lib.vnm_oracle_to_dense_f16(_ptr(values), _ptr(meta), _ptr(columns), M, K, V, 2, m, _ptr(dense))
        assert rc == 0
        return dense

    def spmm(self, values, meta, columns, M, K, V, m, B, bias=None, layout=0, rows=None, out=None):
        """B: [K,N] float16.  layout 0 -> C [M,N]; layout 1 -> C [N,M] (+bias).  rows: optional subset."""
        B = np.ascontiguousarray(B, dtype=np.float16)
        N = B.shape[1]
        if out is None:
            out = np.zeros((M, N) if layout == 0 else (N, M), dtype=np.float16)
        ldc = N if layout == 0 else M
        r = None if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
        if bias is not None:
            bias = np.ascontiguousarray(bias, dtype=np.float16)
        rc = self.lib.vnm_oracle_spmm_f16(_ptr(values), _ptr(meta), _ptr(columns), M, K, V, 2, m, _ptr(B), N, N,
                                          _ptr(bias), _ptr(out), ldc, layout, _ptr(r), 0 if r is None else r.size)
        assert rc == 0
        return out

    def dense_gemm(self, A, B, rows=None):
        A = np.ascontiguousarray(A, dtype=np.float16)
        B = np.ascontiguousarray(B, dtype=np.float16)
        M, K = A.shape
        N = B.shape[1]
        out = np.zeros((M, N), dtype=np.float16)
        r = None if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
        rc = self.lib.vnm_oracle_dense_gemm_f16(_ptr(A), _ptr(B), _ptr(out), M, K, N, _ptr(r), 0 if r is None else r.size)
        assert rc == 0
        return out

    def check(self, got, want, mode=1, tol=1e-2):
        """mode 1: |got-want| <= tol*(|want|+1); mode 0: the reference's |got-want| <= tol (tol=1.0).
        Returns (mismatches, first_bad_index, max_abs_err)."""
        got = np.ascontiguousarray(got, dtype=np.float16)
        want = np.ascontiguousarray(want, dtype=np.float16)
        assert got.size == want.size
        first = C.c_int64(-1)
        worst = C.c_float(0)
        bad = self.lib.vnm_oracle_check(_ptr(got), _ptr(want), got.size, mode, tol, C.byref(first), C.byref(worst))
        return int(bad), int(first.value), float(worst.value)

    def prune(self, absw, V, m):
        absw = np.ascontiguousarray(absw, dtype=np.float32)
        M, K = absw.shape
        ksp, nv, nm, nc = sizes(M, K, V, m)
        mask = np.empty((M, K), dtype=np.int32)
        cols = np.empty(nc, dtype=np.uint32)
        rc = self.lib.vnm_oracle_prune(_ptr(absw), M, K, V, 2, m, _ptr(mask), _ptr(cols))
        if rc:
            raise ValueError("prune: unsupported shape (rc=%d)" % rc)
        return mask, cols


class Reference:
    """The reference's own compressor / decompressor (None-safe: use Reference.load())."""

    @staticmethod
    def load(build=True):
        path = os.path.join(HERE, "_ref", "libvnm_ref.so")
        if build:
            from . import build_oracle
            path = build_oracle.build_reference()
        if not path or not os.path.exists(path):
            return None
        return Reference(path)

    def __init__(self, path):
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_compress_f16.restype = C.c_int
        L.ref_compress_f16.argtypes = [C.c_void_p] * 2 + [C.c_int] * 4 + [C.c_void_p] * 2 + [C.c_long] * 3
        L.ref_to_dense_f16.restype = C.c_int
        L.ref_to_dense_f16.argtypes = [C.c_void_p] * 3 + [C.c_int] * 4 + [C.c_long] * 3 + [C.c_void_p]
        L.ref_random_init_f16.restype = C.c_int
        L.ref_random_init_f16.argtypes = [C.c_int] * 4 + [C.c_uint] + [C.c_void_p] * 3 + [C.c_long] * 3

    def compress(self, dense, columns, V, m):
        M, K = dense.shape
        ksp, nv, nm, nc = sizes(M, K, V, m)
        dense = np.ascontiguousarray(dense, dtype=np.float16)
        columns = np.ascontiguousarray(columns, dtype=np.uint32)
        values = np.empty(nv, dtype=np.float16)
        meta = np.empty(nm, dtype=np.uint32)
        rc = self.lib.ref_compress_f16(_ptr(dense), _ptr(columns), M, K, V, m, _ptr(values), _ptr(meta), nv, nm, nc)
        assert rc == 0
        return values, meta

    def to_dense(self, values, meta, columns, M, K, V, m):
        ksp, nv, nm, nc = sizes(M, K, V, m)
        dense = np.empty((M, K), dtype=np.float16)
        rc = self.lib.ref_to_dense_f16(_ptr(values), _ptr(meta), _ptr(columns), M, K, V, m, nv, nm, nc, _ptr(dense))
        assert rc == 0
        return dense

    def random_init(self, M, K, V, m, seed):
        ksp, nv, nm, nc = sizes(M, K, V, m)
        values = np.empty(nv, dtype=np.float16)
        meta = np.empty(nm, dtype=np.uint32)
        cols = np.empty(nc, dtype=np.uint32)
        rc = self.lib.ref_random_init_f16(M, K, V, m, seed, _ptr(values), _ptr(meta), _ptr(cols), nv, nm, nc)
        assert rc == 0
        return values, meta, cols


class RefSpatha:
    """The reference's own Spatha SpMM kernel (legacy mma.sp, compiled for sm_100a from the reference checkout by
    build_oracle.build_reference_spatha): the second comparator of the GPU parity tests.  Needs a CUDA device.
    None-safe: use RefSpatha.load(), which returns None where the library was never built."""

    @staticmethod
    def load(build=True):
        path = os.path.join(HERE, "_ref", "libvnm_ref_spatha.so")
        if build:
            from . import build_oracle
            path = build_oracle.build_reference_spatha()
        if not path or not os.path.exists(path):
            return None
        return RefSpatha(path)

    def __init__(self, path):
        self.lib = C.CDLL(path)
        f = self.lib.ref_spatha_spmm_f16
        f.restype = C.c_int
        f.argtypes = [C.c_void_p] * 3 + [C.c_int] * 4 + [C.c_long] * 3 + [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_float)]

    def spmm(self, values, meta, columns, M, K, V, m, B, repeats=0):
        """Host arrays in the reference format, B [K,N] float16 (N % 64 == 0).  Returns (C [M,N] float16, ms per launch
        or None)."""
        ksp, nv, nm, nc = sizes(M, K, V, m)
        values = np.ascontiguousarray(values, dtype=np.float16)
        meta = np.ascontiguousarray(meta, dtype=np.uint32)
        columns = np.ascontiguousarray(columns, dtype=np.uint32)
        B = np.ascontiguousarray(B, dtype=np.float16)
        N = B.shape[1]
        out = np.empty((M, N), dtype=np.float16)
        ms = C.c_float(0)
        rc = self.lib.ref_spatha_spmm_f16(_ptr(values), _ptr(meta), _ptr(columns), M, K, V, m, nv, nm, nc, _ptr(B), N, _ptr(out),
                                          repeats, C.byref(ms))
        if rc:
            raise RuntimeError("reference Spatha kernel failed at step %d" % rc)
        return out, (float(ms.value) if repeats > 0 else None)
