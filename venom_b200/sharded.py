"""N-sharded multi-GPU launcher for the V:N:M SpMM (one process per GPU, torch.distributed).

Column c of C = A * B depends only on column c of B, so the dense operand and the output are split by
columns (N) across the ranks; the sparse operand is replicated (broadcast once from rank 0).  There is
no communication inside the product.  An all-gather over the process group is issued only when the
caller asks for a replicated output; in the [N, M] layout an N-shard is a contiguous block of rows, so
the gather writes straight into the full output.

The sharding arithmetic and the collectives are independent of the device: with backend "gloo" and
CPU tensors the same class runs with `compute=None` replaced by a caller-supplied function, which is how
the host-side logic is tested without GPUs.
"""
import torch
import torch.distributed as dist


def shard_bounds(N, world, rank, multiple=8):
    """Half-open column range [lo, hi) of `rank`: contiguous, sizes differ by at most `multiple`, every
    boundary a multiple of `multiple` (the kernel needs N % 8 == 0 per shard)."""
    if N % multiple:
        raise ValueError("N must be a multiple of %d" % multiple)
    units = N // multiple
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * multiple, hi * multiple


class ShardedSpmm:
    """Replicated sparse operand + N-sharded product.

    compute(B_shard, bias) -> [n_shard, M] tensor (layout NM).  For GPUs pass a `capi.Prepared` via
    `from_prepared`; tests pass a plain function."""

    def __init__(self, M, compute, group=None):
        self.M = M
        self.compute = compute
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    @classmethod
    def from_reference_arrays(cls, values, metadata, columns, M, K, V, m, n=2, device=None, group=None, src=0):
        """Broadcast the three reference-format arrays from rank `src` and prepare them on every rank.
        Non-source ranks may pass None for the arrays."""
        from . import capi
        from .synth import vnm_sizes
        ksp, nv, nm, nc = vnm_sizes(M, K, V, m, n)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        if rank == src:
            values, metadata, columns = (values.to(device), metadata.to(device), columns.to(device))
        else:
            values = torch.empty(nv, dtype=torch.float16, device=device)
            metadata = torch.empty(nm, dtype=torch.int32, device=device)
            columns = torch.empty(nc, dtype=torch.int32, device=device)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            for t in (values, metadata, columns):
                dist.broadcast(t, src=src, group=group)
        prep = capi.Prepared(values, metadata, columns, M, K, V, m, n)
        obj = cls(M, lambda B, bias: prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM), group)
        obj.prepared = prep
        return obj

    def local(self, B_shard, bias=None):
        """Product of this rank's shard: [n_shard, M]."""
        return self.compute(B_shard, bias)

    def gathered(self, B_shard, N, bias=None):
        """Replicated output [N, M]: every rank computes its rows and all-gathers the rest.  The shard
        of rank r is rows shard_bounds(N, world, r) of the result."""
        out = torch.empty((N, self.M), dtype=B_shard.dtype, device=B_shard.device)
        lo, hi = shard_bounds(N, self.world, self.rank)
        if B_shard.shape[1] != hi - lo:
            raise ValueError("B shard has %d columns, expected %d" % (B_shard.shape[1], hi - lo))
        out[lo:hi] = self.compute(B_shard, bias)
        if self.world > 1:
            bounds = [shard_bounds(N, self.world, r) for r in range(self.world)]
            equal = len({b[1] - b[0] for b in bounds}) == 1
            if equal and dist.get_backend(self.group) == "nccl":
                # in place: this rank's rows already sit at their final position inside `out`
                dist.all_gather_into_tensor(out, out[lo:hi], group=self.group)
            else:
                # collectives need equal message sizes: pad every shard to the largest one
                rows = max(b - a for a, b in bounds)
                send = torch.zeros((rows, self.M), dtype=out.dtype, device=out.device)
                send[: hi - lo] = out[lo:hi]
                recv = [torch.empty_like(send) for _ in bounds]
                dist.all_gather(recv, send, group=self.group)
                for (a, b), t in zip(bounds, recv):
                    out[a:b] = t[: b - a]
        return out
