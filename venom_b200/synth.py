"""Seeded synthetic inputs for the V:N:M path (host side, numpy).

These stand in for the reference's own random instances (Format_sr_nm<T>::init / random_mask,
src/format/format_sr_nm.cpp:31-75,151-237 of the reference, which draw from the unseeded libc rand()
stream): dense A uniform[-1,1] in fp16; in every V x m block 4 of the m columns are chosen uniformly
(sorted ascending = column-loc); every row keeps 2 of those 4 at random positions; the rest is zero.
Kept values that round to +-0 in fp16 are replaced, because the reference compressor identifies kept
entries by value (`val != 0`, format_sr_nm.cpp:474).
"""
import numpy as np


def vnm_sizes(M, K, V, m, n=2):
    """(Ksp, values_elems, meta_words, colloc_words) -- format_sr_nm.cpp:53-60 of the reference."""
    if n != 2:
        raise ValueError("only n == 2 is supported (2:4 inside the selected columns)")
    if m < 4 or M <= 0 or K <= 0 or V <= 0 or M % V or V % 32:
        raise ValueError("need m >= 4, V %% 32 == 0 and M %% V == 0 (got M=%d V=%d m=%d)" % (M, V, m))
    ksp = -(-(-(-K // m) * 2) // 16) * 16
    return ksp, M * ksp, (M // 2) * (ksp // 8), (M // V) * (ksp // 2) * 4


def random_vnm_dense(M, K, V, m, seed, integer_values=False):
    """Returns (dense [M,K] float16 already pruned to V:2:m, columns uint32 column-loc, mask int32 [M,K]).

    integer_values=True draws kept values from {-4..4} \\ {0} like the reference's `rand()%9-4`
    instances (products and sums are then exact in fp16/fp32)."""
    ksp, _, _, nc = vnm_sizes(M, K, V, m)
    rng = np.random.default_rng(seed)
    G_full = K // m
    rem = K - G_full * m
    G_in = G_full + (1 if rem else 0)        # groups that own at least one real column
    G_all = ksp // 2
    nb = M // V
    cols = np.zeros((nb, G_all, 4), dtype=np.uint32)
    if G_full:
        cols[:, :G_full, :] = np.sort(np.argsort(rng.random((nb, G_full, m)), axis=-1)[..., :4], axis=-1)
    n_keep_last = 2
    if rem:
        if rem >= 4:
            cols[:, G_full, :] = np.sort(np.argsort(rng.random((nb, rem)), axis=-1)[..., :4], axis=-1)
        else:
            cols[:, G_full, :] = np.arange(4, dtype=np.uint32)
            n_keep_last = 2 - max(0, 2 - rem)     # out-of-range candidates j<2 yield (0,0) slots
    dense = np.zeros((M, K), dtype=np.float16)
    mask = np.zeros((M, K), dtype=np.int32)
    if integer_values:
        vals = rng.integers(1, 5, size=(M, G_in, 2)).astype(np.float16) * rng.choice(
            np.array([-1, 1], dtype=np.float16), size=(M, G_in, 2))
    else:
        vals = rng.uniform(-1.0, 1.0, size=(M, G_in, 2)).astype(np.float16)
        vals[vals == 0] = np.float16(0.5)
    rows = np.arange(M)
    for g in range(G_in):
        ragged = rem and g == G_full
        ncand = min(4, rem) if (ragged and rem < 4) else 4
        nkeep = n_keep_last if ragged else 2
        if nkeep <= 0:
            continue
        sel = np.sort(np.argsort(rng.random((M, ncand)), axis=-1)[:, :nkeep], axis=-1)
        c4 = cols[rows // V, g, :]                       # [M,4]
        for s in range(nkeep):
            col = g * m + c4[rows, sel[:, s]].astype(np.int64)
            dense[rows, col] = vals[:, g, s]
            mask[rows, col] = 1
    return dense, cols.reshape(-1), mask


def random_dense_b(K, N, seed, integer_values=False):
    """Dense operand B [K,N]: uniform[-1,1] fp16 (or integers in [-4,4] like the reference's
    `rand()%9-4`, src/util/matrix_utils.h:93)."""
    rng = np.random.default_rng(seed)
    if integer_values:
        return rng.integers(-4, 5, size=(K, N)).astype(np.float16)
    return (rng.random((K, N), dtype=np.float32) * 2.0 - 1.0).astype(np.float16)   # drawn in fp32: 20x faster than float64 for GB-sized operands


def random_vnm_dense_cuda(M, K, V, m, seed, device="cuda"):
    """Same distribution as random_vnm_dense for K % m == 0, drawn on the GPU with torch's generator so
    that matrices of many hundreds of MB (49152 x 12288 and up) take milliseconds instead of minutes.
    Returns (dense [M,K] float16 CUDA tensor pruned to V:2:m, column-loc int32 CUDA tensor)."""
    import torch
    if K % m:
        raise ValueError("random_vnm_dense_cuda needs K %% m == 0")
    ksp, _, _, nc = vnm_sizes(M, K, V, m)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    nb, G = M // V, K // m
    cols = torch.argsort(torch.rand((nb, G, m), device=device, generator=g), dim=-1)[..., :4].sort(dim=-1).values.to(torch.int32)
    dense = torch.zeros((M, G, m), dtype=torch.float16, device=device)
    rows_per_step = max(V, (1 << 26) // max(G, 1) // V * V)      # bounds the temporaries to a few hundred MB
    for r0 in range(0, M, rows_per_step):
        r1 = min(M, r0 + rows_per_step)
        sel = torch.argsort(torch.rand((r1 - r0, G, 4), device=device, generator=g), dim=-1)[..., :2]
        vals = (torch.rand((r1 - r0, G, 2), device=device, generator=g) * 2 - 1).half()
        vals[vals == 0] = 0.5
        c4 = cols[r0 // V:(r1 + V - 1) // V].repeat_interleave(V, dim=0)[:r1 - r0]
        dense[r0:r1].scatter_(2, torch.gather(c4.long(), 2, sel), vals)
    colloc = torch.zeros((nb, ksp // 2, 4), dtype=torch.int32, device=device)
    colloc[:, :G, :] = cols
    return dense.reshape(M, K), colloc.reshape(-1)
