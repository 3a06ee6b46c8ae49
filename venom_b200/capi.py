"""ctypes binding of the C ABI (include/venom_b200.h).

PyTorch is used only for device memory and streams: every wrapper takes CUDA tensors, passes their
data pointers through the C ABI and runs on torch's current stream.  There is no CPU fallback: loading
fails loudly if the library has not been built, and every call raises VenomError on a non-zero status.
"""
import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libvenom_b200.so")

VNM_LAYOUT_MN = 0
VNM_LAYOUT_NM = 1


class VenomError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise VenomError("venom_b200 CUDA library is not built: run `python -m venom_b200.build` "
                             "(expected %s)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        i64p = C.POINTER(C.c_int64)
        L.vnm_last_error_string.restype = C.c_char_p
        L.vnm_version.restype = C.c_int
        L.vnm_sizes.argtypes = [C.c_int] * 5 + [i64p] * 4
        L.vnm_compress_f16.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p] + [C.c_int] * 5 + [C.c_void_p] * 4
        L.vnm_decompress_f16.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5 + [C.c_void_p, C.c_int64, C.c_void_p]
        L.vnm_prune_magnitude_f32.argtypes = [C.c_void_p, C.c_int64] + [C.c_int] * 5 + [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        L.vnm_prune_magnitude_f32.restype = C.c_int
        L.vnm_prepare.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5 + [C.POINTER(C.c_void_p), C.c_void_p]
        L.vnm_prepare_as.argtypes = [C.c_void_p] * 3 + [C.c_int] * 6 + [C.POINTER(C.c_void_p), C.c_void_p]
        L.vnm_prepare_as.restype = C.c_int
        L.vnm_prepared_bytes.argtypes = [C.c_int] * 5 + [i64p]
        L.vnm_destroy.argtypes = [C.c_void_p]
        L.vnm_spmm_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
                                   C.c_int, C.c_void_p]
        L.vnm_spmm_f16_host_async.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.vnm_spmm_f16_host_async.restype = C.c_int
        L.vnm_selftest_wait_expiry.argtypes = [C.c_void_p, C.c_void_p]
        L.vnm_selftest_wait_expiry.restype = C.c_int
        L.vnm_host_wait.argtypes = [C.c_void_p]
        L.vnm_host_wait.restype = C.c_int
        L.vnm_spmm_f16_nk.argtypes = L.vnm_spmm_f16.argtypes
        L.vnm_spmm_f16_nk.restype = C.c_int
        L.vnm_operand_form.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        L.vnm_operand_form.restype = C.c_int
        L.vnm_spmm_f16_host.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.vnm_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_void_p]
        L.vnm_spmm_config.argtypes = [C.c_void_p, C.c_int] + [C.POINTER(C.c_int)] * 5
        L.vnm_set_gather_mode.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_gather_mode.restype = C.c_int
        L.vnm_set_strategy.argtypes = [C.c_int]
        L.vnm_set_strategy.restype = C.c_int
        L.vnm_set_producer_warps.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_producer_warps.restype = C.c_int
        L.vnm_set_gather_split.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_gather_split.restype = C.c_int
        L.vnm_set_pair_mode.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_pair_mode.restype = C.c_int
        L.vnm_set_l2_prefetch.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_host_slices.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_host_slices.restype = C.c_int
        L.vnm_set_l2_prefetch.restype = C.c_int
        L.vnm_set_epilogue.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_epilogue.restype = C.c_int
        L.vnm_set_max_ctas.argtypes = [C.c_void_p, C.c_int]
        L.vnm_set_max_ctas.restype = C.c_int
        L.vnm_handle_info.argtypes = [C.c_void_p] + [C.POINTER(C.c_int)] * 5
        L.vnm_handle_info.restype = C.c_int
        ip = C.POINTER(C.c_int)
        L.vnm_mgpu_shard.argtypes = [C.c_int] * 4 + [ip, ip]
        L.vnm_mgpu_unique_id.argtypes = [C.c_void_p]
        L.vnm_mgpu_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        L.vnm_mgpu_create_from_comm.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        L.vnm_mgpu_destroy.argtypes = [C.c_void_p]
        L.vnm_mgpu_info.argtypes = [C.c_void_p, ip, ip]
        L.vnm_mgpu_set_comm_sms.argtypes = [C.c_void_p, C.c_int]
        L.vnm_mgpu_broadcast_operand.argtypes = [C.c_void_p] * 4 + [C.c_int] * 6 + [C.c_void_p]
        L.vnm_mgpu_spmm_shard.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
                                          C.c_int, C.c_void_p]
        L.vnm_mgpu_spmm_gathered.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
                                             C.c_int, C.c_void_p]
        L.vnm_mgpu_register_output.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.vnm_mgpu_unregister_output.argtypes = [C.c_void_p, C.c_void_p]
        L.vnm_mgpu_spmm_gathered_p2p.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        L.vnm_spmm_f16_multi.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int64, C.c_int,
                                         C.c_void_p]
        L.vnm_spmm_f16_multi.restype = C.c_int
        for name in ("vnm_mgpu_shard", "vnm_mgpu_unique_id", "vnm_mgpu_create", "vnm_mgpu_create_from_comm", "vnm_mgpu_destroy",
                     "vnm_mgpu_info", "vnm_mgpu_set_comm_sms", "vnm_mgpu_broadcast_operand", "vnm_mgpu_spmm_shard", "vnm_mgpu_spmm_gathered",
                     "vnm_mgpu_register_output", "vnm_mgpu_unregister_output", "vnm_mgpu_spmm_gathered_p2p"):
            getattr(L, name).restype = C.c_int
        for name in ("vnm_sizes", "vnm_compress_f16", "vnm_decompress_f16", "vnm_prepare", "vnm_prepared_bytes",
                     "vnm_destroy", "vnm_spmm_f16", "vnm_spmm_f16_host", "vnm_device_status", "vnm_spmm_config"):
            getattr(L, name).restype = C.c_int
        _lib = L
    return _lib


STRATEGY_AUTO, STRATEGY_GATHER, STRATEGY_DENSE_B = 0, 1, 2


def set_strategy(strategy):
    """Layout chosen by later Prepared(...) constructions: auto / gather (V:N:M form) / dense-B (2:4 over all K)."""
    _check(lib().vnm_set_strategy(strategy))


def _check(rc):
    if rc != 0:
        raise VenomError("venom_b200 error %d: %s" % (rc, lib().vnm_last_error_string().decode()))


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise VenomError("expected CUDA tensors (there is no CPU path)")


def sizes(M, K, V, m, n=2):
    """(Ksp, values_elems, meta_words, colloc_words) from the library."""
    out = [C.c_int64() for _ in range(4)]
    _check(lib().vnm_sizes(M, K, V, n, m, *[C.byref(o) for o in out]))
    return tuple(int(o.value) for o in out)


def compress(dense, colloc, V, m, n=2, mask=None, count_violations=True):
    """dense: [M,K] fp16 CUDA (pruned); colloc: int32/uint32 CUDA.  Returns (values fp16, meta int32,
    violations int or None).  Reading the violation count synchronises the stream."""
    _need_cuda(dense, colloc, mask)
    if dense.dtype != torch.float16 or dense.dim() != 2 or dense.stride(1) != 1:
        raise VenomError("dense must be a 2-D fp16 tensor with unit inner stride")
    M, K = dense.shape
    ksp, nv, nm, nc = sizes(M, K, V, m, n)
    if colloc.numel() != nc or colloc.element_size() != 4 or not colloc.is_contiguous():
        raise VenomError("colloc must hold %d 32-bit words" % nc)
    if mask is not None and (mask.dtype != torch.int32 or tuple(mask.shape) != (M, K) or mask.stride() != dense.stride()):
        raise VenomError("mask must be int32 with the shape and strides of dense")
    values = torch.empty(nv, dtype=torch.float16, device=dense.device)
    meta = torch.empty(nm, dtype=torch.int32, device=dense.device)
    viol = torch.zeros(1, dtype=torch.int64, device=dense.device) if count_violations else None
    _check(lib().vnm_compress_f16(dense.data_ptr(), dense.stride(0), None if mask is None else mask.data_ptr(),
                                  colloc.data_ptr(), M, K, V, n, m, values.data_ptr(), meta.data_ptr(),
                                  None if viol is None else viol.data_ptr(), _stream()))
    return values, meta, (int(viol.item()) if viol is not None else None)


def prune_magnitude(w, V, m, n=2):
    """w: [M,K] CUDA tensor (any float dtype; converted to fp32 like the reference does).  Returns
    (mask int32 [M,K], colloc int32) -- the outputs of the reference's nm_vector_mask_sparsify."""
    _need_cuda(w)
    M, K = w.shape
    ksp, nv, nm, nc = sizes(M, K, V, m, n)
    wf = w.detach().to(torch.float32).contiguous()
    mask = torch.empty((M, K), dtype=torch.int32, device=w.device)
    colloc = torch.empty(nc, dtype=torch.int32, device=w.device)
    _check(lib().vnm_prune_magnitude_f32(wf.data_ptr(), K, M, K, V, n, m, mask.data_ptr(), K, colloc.data_ptr(), _stream()))
    return mask, colloc


def decompress(values, meta, colloc, M, K, V, m, n=2):
    _need_cuda(values, meta, colloc)
    dense = torch.empty((M, K), dtype=torch.float16, device=values.device)
    _check(lib().vnm_decompress_f16(values.data_ptr(), meta.data_ptr(), colloc.data_ptr(), M, K, V, n, m,
                                    dense.data_ptr(), K, _stream()))
    return dense


class Prepared:
    """Owns a vnm_handle_t: the kernel-private copy of one sparse operand."""

    def __init__(self, values, meta, colloc, M, K, V, m, n=2, strategy=None):
        """strategy: None = the process-wide setting (set_strategy), else STRATEGY_AUTO / _GATHER / _DENSE_B."""
        _need_cuda(values, meta, colloc)
        ksp, nv, nm, nc = sizes(M, K, V, m, n)
        if values.numel() != nv or meta.numel() != nm or colloc.numel() != nc:
            raise VenomError("array sizes do not match the format (%d, %d, %d expected)" % (nv, nm, nc))
        if values.dtype != torch.float16 or meta.element_size() != 4 or colloc.element_size() != 4:
            raise VenomError("values must be fp16, metadata and colloc 32-bit")
        self.M, self.K, self.V, self.m, self.n = M, K, V, m, n
        self.device = values.device
        self._h = C.c_void_p()
        if strategy is None:
            _check(lib().vnm_prepare(values.data_ptr(), meta.data_ptr(), colloc.data_ptr(), M, K, V, n, m,
                                     C.byref(self._h), _stream()))
        else:
            _check(lib().vnm_prepare_as(values.data_ptr(), meta.data_ptr(), colloc.data_ptr(), M, K, V, n, m, int(strategy),
                                        C.byref(self._h), _stream()))

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            lib().vnm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def spmm(self, B, bias=None, layout=VNM_LAYOUT_MN, out=None):
        """B: [K,N] fp16 CUDA (unit inner stride).  Returns [M,N] (layout MN) or [N,M] (layout NM)."""
        _need_cuda(B, bias, out)
        if B.dtype != torch.float16 or B.dim() != 2 or B.shape[0] != self.K or B.stride(1) != 1:
            raise VenomError("B must be a [K,N] fp16 tensor with unit inner stride (K=%d)" % self.K)
        N = B.shape[1]
        if out is None:
            shape = (self.M, N) if layout == VNM_LAYOUT_MN else (N, self.M)
            out = torch.empty(shape, dtype=torch.float16, device=B.device)
        if bias is not None and (bias.dtype != torch.float16 or bias.numel() != self.M or not bias.is_contiguous()):
            raise VenomError("bias must be a contiguous fp16 vector of M elements")
        _check(lib().vnm_spmm_f16(self._h, B.data_ptr(), B.stride(0), N, None if bias is None else bias.data_ptr(),
                                  out.data_ptr(), out.stride(0), layout, _stream()))
        return out

    def dense_b_form(self):
        v = C.c_int(0)
        _check(lib().vnm_operand_form(self._h, C.byref(v)))
        return bool(v.value)

    def spmm_nk(self, Bt, bias=None, layout=VNM_LAYOUT_NM, out=None):
        """Bt: [N,K] fp16 CUDA (unit inner stride), the transpose of B.  Same result as spmm(Bt.T)."""
        _need_cuda(Bt, bias, out)
        if Bt.dtype != torch.float16 or Bt.dim() != 2 or Bt.shape[1] != self.K or Bt.stride(1) != 1:
            raise VenomError("Bt must be a [N,K] fp16 tensor with unit inner stride (K=%d)" % self.K)
        N = Bt.shape[0]
        if out is None:
            shape = (self.M, N) if layout == VNM_LAYOUT_MN else (N, self.M)
            out = torch.empty(shape, dtype=torch.float16, device=Bt.device)
        _check(lib().vnm_spmm_f16_nk(self._h, Bt.data_ptr(), Bt.stride(0), N, None if bias is None else bias.data_ptr(),
                                     out.data_ptr(), out.stride(0), layout, _stream()))
        return out

    def spmm_multi(self, B, outs, bias=None, layout=VNM_LAYOUT_MN):
        """One product stored to every tensor of `outs` (1 .. 8 tensors of one shape and stride; dense-B form, or gather form
        with layout NM)."""
        _need_cuda(B, bias, *outs)
        if B.dtype != torch.float16 or B.dim() != 2 or B.shape[0] != self.K or B.stride(1) != 1:
            raise VenomError("B must be a [K,N] fp16 tensor with unit inner stride (K=%d)" % self.K)
        N = B.shape[1]
        shape = (self.M, N) if layout == VNM_LAYOUT_MN else (N, self.M)
        for o in outs:
            if o.dtype != torch.float16 or tuple(o.shape) != shape or o.stride() != outs[0].stride() or o.stride(1) != 1:
                raise VenomError("every destination must be a %s fp16 tensor with the same strides" % (shape,))
        ptrs = (C.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
        _check(lib().vnm_spmm_f16_multi(self._h, B.data_ptr(), B.stride(0), N, None if bias is None else bias.data_ptr(), ptrs, len(outs),
                                        outs[0].stride(0), layout, _stream()))
        return outs

    def spmm_host(self, B_host, out_host, bias_host=None, layout=VNM_LAYOUT_MN):
        """End-to-end call with HOST tensors (ideally pinned): H2D, kernel, D2H, synchronise."""
        N = B_host.shape[1]
        _check(lib().vnm_spmm_f16_host(self._h, B_host.data_ptr(), N, None if bias_host is None else bias_host.data_ptr(),
                                       out_host.data_ptr(), layout, _stream()))
        return out_host

    def spmm_host_async(self, B_host, out_host, bias_host=None, layout=VNM_LAYOUT_MN):
        """spmm_host without the final wait (pinned host tensors); collect with host_wait()."""
        N = B_host.shape[1]
        _check(lib().vnm_spmm_f16_host_async(self._h, B_host.data_ptr(), N, None if bias_host is None else bias_host.data_ptr(),
                                             out_host.data_ptr(), layout, _stream()))
        return out_host

    def host_wait(self):
        _check(lib().vnm_host_wait(self._h))

    def selftest_wait_expiry(self):
        """Lets a bounded device-side wait run out on purpose (about two seconds); device_status() then raises."""
        _check(lib().vnm_selftest_wait_expiry(self._h, _stream()))

    def device_status(self):
        st = C.c_int(0)
        rc = lib().vnm_device_status(self._h, C.byref(st), _stream())
        if rc != 0:
            raise VenomError("venom_b200 error %d: %s" % (rc, lib().vnm_last_error_string().decode()))
        return int(st.value)

    def set_gather_mode(self, mode):
        """0 = TMA gather4 (default for m > 4), 3 = per-thread 16-byte cp.async copies (ablation), 1 = 64-row TMA tiles (exact for m == 4, otherwise the
        "no column-loc" ablation), 2 = no B loads (timing floor only)."""
        _check(lib().vnm_set_gather_mode(self._h, mode))

    def set_producer_warps(self, warps):
        _check(lib().vnm_set_producer_warps(self._h, warps))

    def set_gather_split(self, tma_rows):
        """Gather mode 3: rows of every 64-row stage fetched by TMA gather4 beside the per-thread copies (0, 16, 32, 48)."""
        _check(lib().vnm_set_gather_split(self._h, tma_rows))

    def set_pair_mode(self, mode):
        """Dense-B form: 1 = two-SM (cta_group::2) kernel where it applies (default), 0 = single-SM kernel only,
        2 = pairs without L2 hints, 3 / 4 = pairs with one / two row tiles per CTA forced where the shape allows."""
        _check(lib().vnm_set_pair_mode(self._h, mode))

    def set_host_slices(self, slices):
        """Equal column slices of the host-buffer pipeline (spmm_host): 1 .. 32; 0 = the default (8)."""
        _check(lib().vnm_set_host_slices(self._h, slices))

    def set_l2_prefetch(self, ktiles_ahead):
        """Two-SM kernel: L2-only prefetches this many k-tiles ahead of the loads into shared memory (0 = none)."""
        _check(lib().vnm_set_l2_prefetch(self._h, ktiles_ahead))

    def set_epilogue(self, mode):
        """Gather form: 0 = default, 1 = 32-bit stores per thread for layout MN, 2 = layout NM through TMA stores also for a single
        destination (ablations)."""
        _check(lib().vnm_set_epilogue(self._h, mode))

    def set_max_ctas(self, n):
        """Cap on the persistent CTAs of this operand's products (0 = one per SM)."""
        _check(lib().vnm_set_max_ctas(self._h, n))

    def config(self, N):
        v = [C.c_int() for _ in range(5)]
        _check(lib().vnm_spmm_config(self._h, N, *[C.byref(x) for x in v]))
        return dict(zip(("tile_m", "tile_n", "stages", "grid", "smem_bytes"), (int(x.value) for x in v)))


def mgpu_shard(N, world, rank, multiple=8):
    """Half-open column range [lo, hi) of `rank` (vnm_mgpu_shard; pure arithmetic, no GPU needed)."""
    lo, hi = C.c_int(), C.c_int()
    _check(lib().vnm_mgpu_shard(N, world, rank, multiple, C.byref(lo), C.byref(hi)))
    return int(lo.value), int(hi.value)


class Mgpu:
    """Owns a vnm_mgpu_t: this rank's place in the N-sharded launcher (NCCL communicator + exchange stream).

    Mgpu.create(exchange_id) is collective: rank 0 draws the id (Mgpu.unique_id()) and `exchange_id(bytes_or_None)`
    hands it to every rank (torch.distributed, MPI, a file ... -- the library does not care)."""

    def __init__(self, handle, world, rank):
        self._c, self.world, self.rank = handle, world, rank

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(128)
        _check(lib().vnm_mgpu_unique_id(buf))
        return buf.raw

    @classmethod
    def create(cls, world, rank, exchange_id):
        ident = exchange_id(cls.unique_id() if rank == 0 else None)
        if len(ident) != 128:
            raise VenomError("the communicator id must be 128 bytes")
        h = C.c_void_p()
        _check(lib().vnm_mgpu_create(C.create_string_buffer(bytes(ident), 128), world, rank, C.byref(h)))
        return cls(h, world, rank)

    @classmethod
    def create_torch(cls, group=None):
        """Collective over a torch.distributed group (any backend): the id travels through the group."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)

        def exchange(ident):
            box = [ident]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            return box[0]
        return cls.create(world, rank, exchange)

    def close(self):
        if getattr(self, "_c", None) is not None and self._c.value:
            lib().vnm_mgpu_destroy(self._c)
            self._c = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_comm_sms(self, sms):
        _check(lib().vnm_mgpu_set_comm_sms(self._c, sms))

    def broadcast_operand(self, values, meta, colloc, M, K, V, m, n=2, root=0):
        _need_cuda(values, meta, colloc)
        _check(lib().vnm_mgpu_broadcast_operand(self._c, values.data_ptr(), meta.data_ptr(), colloc.data_ptr(), M, K, V, n, m, root, _stream()))

    def spmm_shard(self, prep, B_shard, bias=None, layout=VNM_LAYOUT_MN, out=None):
        _need_cuda(B_shard, bias, out)
        n = B_shard.shape[1]
        if out is None:
            out = torch.empty((prep.M, n) if layout == VNM_LAYOUT_MN else (n, prep.M), dtype=torch.float16, device=B_shard.device)
        _check(lib().vnm_mgpu_spmm_shard(self._c, prep._h, B_shard.data_ptr(), B_shard.stride(0), n, None if bias is None else bias.data_ptr(),
                                         out.data_ptr(), out.stride(0), layout, _stream()))
        return out

    def spmm_gathered(self, prep, B_shard, N_total, bias=None, out=None, chunks=4):
        """Every rank ends with the full [N_total, M] result; the exchange overlaps the product chunk by chunk."""
        _need_cuda(B_shard, bias, out)
        if B_shard.dtype != torch.float16 or B_shard.dim() != 2 or B_shard.stride(1) != 1 or B_shard.shape[1] * self.world != N_total:
            raise VenomError("B shard must be [K, N_total / world] fp16 with unit inner stride")
        if out is None:
            out = torch.empty((N_total, prep.M), dtype=torch.float16, device=B_shard.device)
        _check(lib().vnm_mgpu_spmm_gathered(self._c, prep._h, B_shard.data_ptr(), B_shard.stride(0), N_total,
                                            None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0), chunks, _stream()))
        return out

    def register_output(self, out_full):
        """Collective: maps every rank's [N_total, M] result buffer into every other rank (CUDA IPC), for spmm_gathered_p2p."""
        _need_cuda(out_full)
        if not out_full.is_contiguous():
            raise VenomError("the gathered result buffer must be contiguous")
        _check(lib().vnm_mgpu_register_output(self._c, out_full.data_ptr(), out_full.numel() * out_full.element_size()))
        return out_full

    def unregister_output(self, out_full):
        """Collective: waits for this device and all ranks, then unmaps the peers' buffers."""
        _check(lib().vnm_mgpu_unregister_output(self._c, out_full.data_ptr()))

    def spmm_gathered_p2p(self, prep, B_shard, N_total, out, bias=None):
        """Every rank ends with the full [N_total, M] result in its registered `out`: one product launch whose epilogue
        stores each tile of this rank's rows to all ranks' buffers (own first, peers over NVLink); no exchange step."""
        _need_cuda(B_shard, bias, out)
        if B_shard.dtype != torch.float16 or B_shard.dim() != 2 or B_shard.stride(1) != 1 or B_shard.shape[1] * self.world != N_total:
            raise VenomError("B shard must be [K, N_total / world] fp16 with unit inner stride")
        _check(lib().vnm_mgpu_spmm_gathered_p2p(self._c, prep._h, B_shard.data_ptr(), B_shard.stride(0), N_total,
                                                None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0), _stream()))
        return out
