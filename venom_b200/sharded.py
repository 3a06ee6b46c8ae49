"""N-sharded multi-GPU launcher for the V:N:M SpMM (one process per GPU): a thin caller of the library's
vnm_mgpu_* entry points (NCCL inside the library) with torch.distributed as the plumbing that starts the ranks.

Column c of C = A * B depends only on column c of B, so the dense operand and the output are split by
columns (N) across the ranks; the sparse operand is replicated (broadcast once from rank 0).  There is
no communication inside the product.  An all-gather over the process group is issued only when the
caller asks for a replicated output; in the [N, M] layout an N-shard is a contiguous block of rows, so
the gather writes straight into the full output.

On GPUs (`from_reference_arrays`) the broadcast of the sparse operand, the shard product and the gathered product
-- chunked, the exchange of one chunk overlapping the product of the next -- all run inside the library.  The
same class also runs with backend "gloo" and CPU tensors when it is given a plain `compute` function: the
sharding arithmetic and the exchange pattern are then exercised with torch collectives, which is how the host-side
logic is tested without GPUs (the arithmetic itself is the library's: vnm_mgpu_shard).
"""
import torch
import torch.distributed as dist


def shard_bounds(N, world, rank, multiple=8):
    """Half-open column range [lo, hi) of `rank`: contiguous, sizes differ by at most `multiple`, every
    boundary a multiple of `multiple` (the kernel needs N % 8 == 0 per shard)."""
    if N % multiple:
        raise ValueError("N must be a multiple of %d" % multiple)
    from . import capi
    return capi.mgpu_shard(N, world, rank, multiple)


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
        ctx = None
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            ctx = capi.Mgpu.create_torch(group)
            ctx.broadcast_operand(values, metadata, columns, M, K, V, m, n, root=src)
        prep = capi.Prepared(values, metadata, columns, M, K, V, m, n)
        obj = cls(M, lambda B, bias: prep.spmm(B, bias=bias, layout=capi.VNM_LAYOUT_NM), group)
        obj.prepared = prep
        obj.ctx = ctx
        return obj

    def local(self, B_shard, bias=None):
        """Product of this rank's shard: [n_shard, M]."""
        return self.compute(B_shard, bias)

    ctx = None        # capi.Mgpu when the ranks run on GPUs
    prepared = None

    def gathered_p2p(self, B_shard, N, out, bias=None):
        """Replicated output [N, M] without an exchange step (GPUs only, dense-B operand form): `out` is registered on
        first use (collective: every rank calls this with its own buffer of the same size at the same time), and the
        product's epilogue stores this rank's rows to every rank's buffer -- vnm_mgpu_spmm_gathered_p2p.  Keep passing
        the same `out`; release_outputs() (collective) unmaps it."""
        if self.ctx is None:
            raise RuntimeError("gathered_p2p needs the GPU launcher (capi.Mgpu)")
        lo, hi = shard_bounds(N, self.world, self.rank)
        if B_shard.shape[1] != hi - lo:
            raise ValueError("B shard has %d columns, expected %d" % (B_shard.shape[1], hi - lo))
        shared = self.__dict__.setdefault("_shared_outputs", {})
        if out.data_ptr() not in shared:
            self.ctx.register_output(out)
            shared[out.data_ptr()] = out   # the tensor stays alive while peers may store into it
        return self.ctx.spmm_gathered_p2p(self.prepared, B_shard, N, out, bias=bias)

    def release_outputs(self):
        """Collective: unmaps every buffer gathered_p2p registered."""
        shared = self.__dict__.get("_shared_outputs", {})
        for ptr in sorted(shared):
            self.ctx.unregister_output(shared[ptr])
        shared.clear()

    def gathered(self, B_shard, N, bias=None, chunks=None, out=None):
        """Replicated output [N, M]: every rank computes its rows and receives the rest.  The shard of rank r is rows
        shard_bounds(N, world, r) of the result.  On GPUs with equal shards this is vnm_mgpu_spmm_gathered: the shard
        goes through in `chunks` column chunks, each exchanged while the next is multiplied (chunks=1: product, then
        one in-place all-gather)."""
        if chunks is None:
            # measured on NVSwitch: the chunked exchange pays up to 4 ranks; beyond that its world - 1 messages per chunk
            # cost more than the overlap hides (8 ranks: 10.6 ms chunked against 9.6 ms plain)
            chunks = 4 if self.world <= 4 else 1
        lo, hi = shard_bounds(N, self.world, self.rank)
        if self.ctx is not None and N % (8 * self.world) == 0:
            if B_shard.shape[1] != hi - lo:
                raise ValueError("B shard has %d columns, expected %d" % (B_shard.shape[1], hi - lo))
            return self.ctx.spmm_gathered(self.prepared, B_shard, N, bias=bias, out=out, chunks=chunks)
        if out is None:
            out = torch.empty((N, self.M), dtype=B_shard.dtype, device=B_shard.device)
        if B_shard.shape[1] != hi - lo:
            raise ValueError("B shard has %d columns, expected %d" % (B_shard.shape[1], hi - lo))
        bounds = [shard_bounds(N, self.world, r) for r in range(self.world)]
        equal = len({b[1] - b[0] for b in bounds}) == 1
        if self.world > 1 and equal and chunks > 1:
            # The library's pattern with torch point-to-point messages (what the CPU tests run): every chunk is
            # computed, then sent to every peer and the peers' chunks are received at their final rows; the
            # requests of chunk c are only waited for after chunk c+1 has been computed.
            ns = hi - lo
            w = -(-(-(-ns // chunks)) // 8) * 8
            pending = []
            for c0 in range(0, ns, w):
                cw = min(w, ns - c0)
                out[lo + c0:lo + c0 + cw] = self.compute(B_shard[:, c0:c0 + cw].contiguous(), bias)
                for req in pending:
                    req.wait()
                ops = []
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    peer = dist.get_global_rank(self.group, r) if self.group is not None else r
                    ops.append(dist.P2POp(dist.isend, out[lo + c0:lo + c0 + cw], peer, self.group))
                    ops.append(dist.P2POp(dist.irecv, out[r * ns + c0:r * ns + c0 + cw], peer, self.group))
                pending = dist.batch_isend_irecv(ops)
            for req in pending:
                req.wait()
            return out
        out[lo:hi] = self.compute(B_shard, bias)
        if self.world > 1:
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
