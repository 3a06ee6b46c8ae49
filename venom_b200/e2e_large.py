"""Largest configuration of the path: dense -> V:N:M compression of a 49152 x 12288 matrix on the GPU and the
product with a [12288, 32768] dense operand sharded by columns (N) over the GPUs of one node.

    python -m venom_b200.e2e_large [--m-rows 49152] [--k 12288] [--n-cols 32768] [-v 128] [-m 8] [--repeats 5] [--gather]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m venom_b200.e2e_large ...

Rank 0 builds the seeded matrix, compresses it (timed; the round trip through the decompressor is checked to be
bit-exact) and broadcasts the three reference-format arrays; every rank multiplies its own column shard (total N is
fixed: strong scaling).  The time of the product is the maximum over ranks; --gather adds the all-gather of the
[N, M] result.  Printed: compressor GB/s, product milliseconds, whole-job useful TFLOP/s (2*M*N*K*n/m) and the
ratio to a dense fp16 matmul of the same shard.
"""
import argparse
import os

import torch


def _time(fn, repeats, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(repeats):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / repeats


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--m-rows", type=int, default=49152)
    ap.add_argument("--k", type=int, default=12288)
    ap.add_argument("--n-cols", type=int, default=32768)
    ap.add_argument("-v", type=int, default=128)
    ap.add_argument("-m", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--gather", action="store_true")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device (there is no CPU path)")
    from . import capi
    from .sharded import ShardedSpmm, shard_bounds
    from .synth import random_vnm_dense_cuda, vnm_sizes
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl")
    M, K, N, V, m = args.m_rows, args.k, args.n_cols, args.v, args.m
    ksp, nv, nm, nc = vnm_sizes(M, K, V, m)
    values = meta = colloc = None
    dense = None
    if rank == 0:
        dense, colloc = random_vnm_dense_cuda(M, K, V, m, seed=4)
        values, meta, bad = capi.compress(dense, colloc, V, m)
        ok = torch.equal(capi.decompress(values, meta, colloc, M, K, V, m), dense)
        tc = _time(lambda: capi.compress(dense, colloc, V, m, count_violations=False), args.repeats)
        nbytes = 2 * M * K + 4 * nc + 2 * nv + 4 * nm
        print("compress %dx%d V=%d 2:%d: %.3f ms, %.0f GB/s, violations %d, round trip %s" % (
            M, K, V, m, tc, nbytes / tc / 1e6, bad, "bit-exact" if ok else "MISMATCH"), flush=True)
    sh = ShardedSpmm.from_reference_arrays(values, meta, colloc, M, K, V, m)
    lo, hi = shard_bounds(N, world, rank)
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + rank)
    B = (torch.rand((K, hi - lo), device="cuda", generator=g) * 2 - 1).half()
    out = torch.empty((M, hi - lo), dtype=torch.float16, device="cuda")
    t_sp = _time(lambda: sh.prepared.spmm(B, out=out), args.repeats)
    t_gather = _time(lambda: sh.gathered(B, N), max(1, args.repeats // 2), warmup=1) if args.gather else 0.0
    t_dense = 0.0
    if rank == 0:
        t_dense = _time(lambda: torch.matmul(dense, B), args.repeats)
    times = torch.tensor([t_sp, t_gather], device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    if rank == 0:
        t_sp, t_gather = times.tolist()
        useful = 2.0 * M * N * K * 2 / m
        print("spmm %dx%dx%d V=%d 2:%d on %d GPU(s), %d columns per rank: %.3f ms, %.1f useful TFLOP/s whole job; dense fp16 matmul of one "
              "shard %.3f ms (%.2fx)" % (M, K, N, V, m, world, hi - lo, t_sp, useful / t_sp / 1e9, t_dense, t_dense / t_sp), flush=True)
        if args.gather:
            print("with the all-gather of the [N, M] result: %.3f ms" % t_gather, flush=True)
    if world > 1:
        dist.destroy_process_group()
    return t_sp


if __name__ == "__main__":
    main()
