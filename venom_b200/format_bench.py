"""Times the dense -> V:N:M compressor, the decompressor and the operand re-pack on one GPU.

    python -m venom_b200.format_bench [--m-rows 49152] [--k 12288] [-v 128] [-m 8] [--repeats 10]

Prints one line per kernel: milliseconds (CUDA events) and algorithmic GB/s (bytes of the dense matrix read
plus bytes of values, metadata and column-loc written).  The input is a seeded synthetic matrix that already
follows the V:2:m pattern; the round trip compress -> decompress is checked to be bit-exact.
"""
import argparse

import torch


def _time(fn, repeats, warmup=3):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(repeats):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / repeats


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--m-rows", type=int, default=49152)
    ap.add_argument("--k", type=int, default=12288)
    ap.add_argument("-v", type=int, default=128)
    ap.add_argument("-m", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=10)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device (there is no CPU path)")
    from . import capi
    from .synth import random_vnm_dense_cuda, vnm_sizes
    M, K, V, m = args.m_rows, args.k, args.v, args.m
    dense, colloc = random_vnm_dense_cuda(M, K, V, m, seed=1)
    ksp, nv, nm, nc = vnm_sizes(M, K, V, m)
    values, meta, bad = capi.compress(dense, colloc, V, m)
    ok = torch.equal(capi.decompress(values, meta, colloc, M, K, V, m), dense)
    nbytes = 2 * M * K + 4 * nc + 2 * nv + 4 * nm
    tc = _time(lambda: capi.compress(dense, colloc, V, m, count_violations=False), args.repeats)
    td = _time(lambda: capi.decompress(values, meta, colloc, M, K, V, m), args.repeats)
    print("compress   %dx%d V=%d 2:%d: %.3f ms, %.0f GB/s (%.1f MB), violations %d, round trip %s" % (
        M, K, V, m, tc, nbytes / tc / 1e6, nbytes / 1e6, bad, "bit-exact" if ok else "MISMATCH"))
    print("decompress %dx%d V=%d 2:%d: %.3f ms, %.0f GB/s" % (M, K, V, m, td, nbytes / td / 1e6))
    return 0 if ok and bad == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
