"""Host-side logic of the N-sharded launcher, run as two gloo ranks on CPU: shard arithmetic, the
all-gather into the [N, M] layout and the broadcast plumbing (the product itself is replaced by a
plain matmul, since there is no CPU SpMM in this library)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from venom_b200.sharded import ShardedSpmm, shard_bounds


def test_shard_bounds_cover_and_align():
    for N, world in [(16384, 8), (16384, 3), (264, 4), (8, 2), (4096 + 8, 5)]:
        edges = [shard_bounds(N, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == N
        for (a, b), (c, d) in zip(edges, edges[1:]):
            assert b == c
        assert all(a % 8 == 0 and b % 8 == 0 for a, b in edges)
        sizes = [b - a for a, b in edges]
        assert max(sizes) - min(sizes) <= 8
    with pytest.raises(ValueError):
        shard_bounds(100, 2, 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, N, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K = 24, 40
        g = torch.Generator().manual_seed(5)
        A = torch.randn(M, K, generator=g)
        B = torch.randn(K, N, generator=g)
        bias = torch.randn(M, generator=g)
        op = ShardedSpmm(M, lambda Bs, b: (A @ Bs).T.contiguous() + (0 if b is None else b), None)
        lo, hi = shard_bounds(N, world, rank)
        want = (A @ B).T + bias
        ok = True
        for chunks in (1, 2, 4):      # plain gather, and the chunked exchange pattern the library uses on GPUs
            full = op.gathered(B[:, lo:hi].contiguous(), N, bias, chunks=chunks)
            ok = ok and torch.allclose(full, want, atol=1e-5)
        local = op.local(B[:, lo:hi].contiguous(), bias)
        ok = ok and torch.allclose(local, want[lo:hi], atol=1e-5)
        q.put((rank, bool(ok), tuple(full.shape)))
    finally:
        dist.destroy_process_group()


def test_library_shard_arithmetic_rejects_bad_arguments():
    """vnm_mgpu_shard is pure arithmetic behind the C ABI: usable (and checked) without a GPU or NCCL."""
    from venom_b200 import capi
    assert capi.mgpu_shard(32768, 8, 3) == (12288, 16384)
    assert capi.mgpu_shard(264, 4, 0) == (0, 72) and capi.mgpu_shard(264, 4, 3) == (200, 264)
    for bad in [(100, 2, 0), (64, 0, 0), (64, 2, 2), (64, 2, -1)]:
        with pytest.raises(capi.VenomError):
            capi.mgpu_shard(*bad)


@pytest.mark.parametrize("N", [64, 72, 256])      # equal, unequal, and equal shards with several chunks each
def test_two_rank_gather_gloo(N):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, N, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res), res
    assert all(shape == (N, 24) for _, _, shape in res)
