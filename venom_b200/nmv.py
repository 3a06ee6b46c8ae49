"""Host-side mirror of the reference's Python format / model-integration layer for the V:N:M path.

Mirrors (same names, argument meaning and return conventions):
  * SrNMTensor                 end2end/grouped_nmv_tensor.py:677-744 (values / columns / metadata, nnz, to_dense)
  * NMVectorSparsifier         end2end/bert_pytorch.py:56-83 (the shipped fixed-mask sparsifier)
  * sparse_dense_mul_dispatch  end2end/bert_pytorch.py:85-106
  * SrnmSpmm, linear_to_spmm   end2end/bert_pytorch.py:109-167
The compressor and the product run on the GPU through the C ABI (there is no CPU path); the `spatha`
torch extension is used when it has been built, else the ctypes binding -- both call the same library.
"""
import numpy as np
import torch

from . import capi
from .synth import vnm_sizes


def round_up(x, y):
    return -(-x // y) * y


class SrNMTensor:
    """V:N:M compressed matrix: `values` fp16 [nrows*Ksp], `columns` int32 column-loc, `metadata` int32.

    Built from a dense (already masked) matrix, an int mask of the kept entries and the column-loc
    array, exactly like the reference class; the arrays are bit-identical to the reference's."""

    def __init__(self, n_, m_, tileM_, dense_, mask_, columns_, device_):
        self.n, self.m, self.tileM = n_, m_, tileM_
        self.device = torch.device(device_)
        if self.device.type != "cuda":
            raise capi.VenomError("SrNMTensor needs a CUDA device (there is no CPU path)")
        self.nrows, self.ncols = dense_.shape
        ksp, nv, nm, nc = vnm_sizes(self.nrows, self.ncols, tileM_, m_, n_)
        self.nnz = nv
        d = dense_.detach().to(device=self.device, dtype=torch.float16).contiguous()
        self.columns = columns_.to(device=self.device, dtype=torch.int32).contiguous().reshape(-1)
        mask = None if mask_ is None else mask_.to(device=self.device, dtype=torch.int32).contiguous()
        self.values, self.metadata, self.violations = capi.compress(d, self.columns, tileM_, m_, n_, mask=mask)
        self._prepared = None

    def prepared(self):
        if self._prepared is None:
            self._prepared = capi.Prepared(self.values, self.metadata, self.columns, self.nrows, self.ncols, self.tileM, self.m, self.n)
        return self._prepared

    def to_dense(self):
        return capi.decompress(self.values, self.metadata, self.columns, self.nrows, self.ncols, self.tileM, self.m, self.n)


def nm_vector_mask_sparsify(tensor, n, m, tileM):
    """Magnitude pruning to V:n:m on the GPU; same return value as the reference function of this name
    (end2end/grouped_nmv_tensor.py:746-779): (masks int32 [nrows, ncols], columns int32)."""
    return capi.prune_magnitude(tensor, tileM, m, n)


class MagnitudeSparsifier:
    """The magnitude path the reference keeps commented out in its scripts (end2end/bert_pytorch.py:63-64)."""

    def __init__(self, n, m, tileM):
        self.n, self.m, self.tileM = n, m, tileM

    def __call__(self, tensor, device=None):
        device = tensor.device if device is None else device
        mask, columns = nm_vector_mask_sparsify(tensor.to(device), self.n, self.m, self.tileM)
        dense = tensor.detach().to(device=device, dtype=torch.float16) * mask.to(torch.float16)
        return SrNMTensor(self.n, self.m, self.tileM, dense, mask, columns, device)


class NMVectorSparsifier:
    """The sparsifier the reference's end-to-end scripts ship with: a fixed pattern that keeps columns
    0 and 2 of every group of m and uses column-loc {0,1,2,3} (end2end/bert_pytorch.py:66-75)."""

    def __init__(self, n, m, tileM):
        self.n, self.m, self.tileM = n, m, tileM

    def __call__(self, tensor, device=None):
        nrows, ncols = tensor.shape
        device = tensor.device if device is None else device
        ksp, nv, nm, nc = vnm_sizes(nrows, ncols, self.tileM, self.m, self.n)
        columns = torch.zeros(nc, dtype=torch.int32).reshape(-1, 4) + torch.tensor([0, 1, 2, 3], dtype=torch.int32)
        pattern = torch.zeros(self.m, dtype=torch.int32, device=tensor.device)  # built where the weight lives: GBs for large layers
        pattern[0] = 1
        pattern[2] = 1
        reps = -(-ncols // self.m)
        mask = pattern.repeat(reps)[:ncols].unsqueeze(0).expand(nrows, ncols).contiguous()
        dense = tensor.detach().to(torch.float16) * mask.to(torch.float16)
        return SrNMTensor(self.n, self.m, self.tileM, dense, mask, columns, device)


def sparse_dense_mul_dispatch(sparse_values, sparse_indices, sparse_metadata, dense, nrows_sp, ncols_sp, ncols_d, m, n, v, nnz, bias):
    """Same call as the reference helper: returns [ncols_d, nrows_sp] = (A @ dense).T + bias."""
    from . import spatha_module
    # the reference materialises `dense.contiguous()` here; the op accepts the transposed view itself and
    # copies only when it has to
    dense_ = dense
    return spatha_module().spmm(sparse_metadata, sparse_indices, sparse_values, dense_, bias, nrows_sp, ncols_sp, ncols_d, v, n, m, nnz, 0, 32, 4)


class SrnmSpmm(torch.nn.Module):
    """Drop-in replacement of torch.nn.Linear whose weight is stored in V:N:M form."""

    def __init__(self, original, n=2, m=8, v=64, sparsifier=None):
        super().__init__()
        self.n, self.m, self.v = n, m, v
        self.bias = original.bias
        w = (sparsifier or NMVectorSparsifier(n, m, v))(original.weight)
        self.values = torch.nn.Parameter(w.values, requires_grad=False)
        self.columns = w.columns
        self.metadata = w.metadata
        self.nrows_sp, self.ncols_sp, self.nnz = w.nrows, w.ncols, w.nnz

    def forward(self, input):
        flat = torch.flatten(input, start_dim=0, end_dim=-2)
        ncols_d = flat.shape[0]
        bias = self.bias if self.bias is not None else None
        out = sparse_dense_mul_dispatch(self.values, self.columns, self.metadata, flat.T, self.nrows_sp, self.ncols_sp, ncols_d,
                                        self.m, self.n, self.v, self.nnz, bias)
        return out.reshape((*input.shape[0:-1], -1))


def linear_to_spmm(mod, n=2, m=8, v=64, skip=()):
    """Replaces every torch.nn.Linear below `mod` by SrnmSpmm (end2end/bert_pytorch.py:155-167)."""
    if isinstance(mod, torch.nn.Linear):
        return SrnmSpmm(mod, n, m, v)
    for name, child in mod.named_children():
        if isinstance(child, SrnmSpmm) or name in skip:
            continue
        if isinstance(child, torch.nn.Linear):
            setattr(mod, name, SrnmSpmm(child, n, m, v))
        elif child is not mod:
            linear_to_spmm(child, n, m, v, skip)
    return mod
