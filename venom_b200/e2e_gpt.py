"""GPT-3-shaped decoder block inference, dense vs V:N:M, sharded by sequences over the GPUs of one node.

Mirrors the reference's end2end/gpt3_pytorch.py (argument names -m -n -v, every linear of the decoder layers
replaced by SrnmSpmm, output lines `0,n,m,v,mean,median,std,len` in milliseconds), with these differences:
  * weights are pruned by magnitude inside every V x m block on the GPU (the path the reference keeps commented
    out, end2end/bert_pytorch.py:63-64); --fixed-mask selects the fixed pattern the reference's script ships;
  * the layers are written out here (pre-LayerNorm attention + GELU MLP with torch.nn.Linear) instead of
    instantiating transformers' GPT2Model, whose Conv1D weights the reference has to transpose first; weights are
    random-init N(0, 0.02) -- no checkpoint is available offline;
  * the token dimension (batch x seq) is what the product shards: under torchrun every rank takes
    batch / world_size whole sequences through the same replicated sparse weights (no collective inside the
    layers: attention never crosses a sequence) and the final hidden states are all-gathered once, so that every
    rank ends with the full [batch, seq, hidden] output, as a following un-sharded layer would need;
  * timing uses CUDA events, the maximum over ranks is reported.

    python -m venom_b200.e2e_gpt -m 16 -n 2 -v 128 [--layers 4] [--hidden 12288] [--heads 96] [--ffn 49152]
           [--batch 8] [--seq 2048] [--repeats 5] [--fixed-mask]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m venom_b200.e2e_gpt ...
"""
import argparse
import os
import statistics

import torch
import torch.nn.functional as F


class DecoderLayer(torch.nn.Module):
    def __init__(self, hidden, heads, ffn):
        super().__init__()
        self.heads = heads
        self.ln_1 = torch.nn.LayerNorm(hidden)
        self.c_attn = torch.nn.Linear(hidden, 3 * hidden)
        self.c_proj = torch.nn.Linear(hidden, hidden)
        self.ln_2 = torch.nn.LayerNorm(hidden)
        self.c_fc = torch.nn.Linear(hidden, ffn)
        self.c_fc_proj = torch.nn.Linear(ffn, hidden)
        for lin in (self.c_attn, self.c_proj, self.c_fc, self.c_fc_proj):
            torch.nn.init.normal_(lin.weight, std=0.02)
            torch.nn.init.zeros_(lin.bias)

    def forward(self, x):
        b, s, h = x.shape
        q, k, v = self.c_attn(self.ln_1(x)).split(h, dim=-1)
        q, k, v = (t.reshape(b, s, self.heads, h // self.heads).transpose(1, 2) for t in (q, k, v))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, h)
        x = x + self.c_proj(a)
        return x + self.c_fc_proj(F.gelu(self.c_fc(self.ln_2(x))))


def build_block(layers, hidden, heads, ffn):
    return torch.nn.Sequential(*[DecoderLayer(hidden, heads, ffn) for _ in range(layers)]).eval()


def sparsify(block, n, m, v, magnitude):
    from .nmv import MagnitudeSparsifier, NMVectorSparsifier, SrnmSpmm
    sp = (MagnitudeSparsifier if magnitude else NMVectorSparsifier)(n, m, v)
    count = 0
    for layer in block:
        for name, child in list(layer.named_children()):
            if isinstance(child, torch.nn.Linear):
                setattr(layer, name, SrnmSpmm(child, n, m, v, sparsifier=sp))
                child.weight = None  # the dense copy is not needed any more
                count += 1
    return count


def time_forward(fn, repeats, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    return ms


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", type=int, default=16)
    ap.add_argument("-n", type=int, default=2)
    ap.add_argument("-v", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=12288)
    ap.add_argument("--heads", type=int, default=96)
    ap.add_argument("--ffn", type=int, default=49152)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--fixed-mask", action="store_true", help="the reference script's fixed pattern instead of magnitude pruning")
    ap.add_argument("--magnitude", action="store_true", help="accepted for compatibility: magnitude pruning is the default")
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--gather-every-layer", action="store_true",
                    help="additionally all-gather the output of every linear (communication-bound variant; the gathered copies are discarded)")
    ap.add_argument("--peer-store", action="store_true",
                    help="with --gather-every-layer: no exchange step, every sparse linear stores its output tiles into all ranks' buffers "
                         "(vnm_mgpu_spmm_gathered_p2p) instead of the chunked NCCL exchange")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device (there is no CPU path)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl")
    if args.batch % world:
        raise SystemExit("batch must be a multiple of the number of ranks")
    torch.set_grad_enabled(False)
    torch.manual_seed(0)                       # the same weights on every rank
    # built on the GPU in fp16 straight away: on the host the fp32 copy would take 29 GB and minutes per rank
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float16)
    try:
        with torch.device("cuda"):
            block = build_block(args.layers, args.hidden, args.heads, args.ffn)
    finally:
        torch.set_default_dtype(prev)
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    x_all = torch.randn((args.batch, args.seq, args.hidden), device="cuda", generator=g).half()
    per = args.batch // world
    x = x_all[rank * per:(rank + 1) * per].contiguous()
    gathered = torch.empty_like(x_all) if world > 1 else None

    hooks = []
    mgpu_ctx = None
    shared_bufs = []   # result buffers registered for peer stores

    def install_gather_hooks():
        """The replicated copy of every linear's output, as a caller that does not shard the following op would need it.
        Sparse linears go through the library's chunked gathered product (the exchange of one column chunk travels while
        the next chunk is multiplied); dense linears use a plain all-gather after the product."""
        nonlocal mgpu_ctx
        from . import capi
        bufs = {}

        def hook(mod, inp, out):
            flat = out.reshape(-1, out.shape[-1])
            key = flat.shape
            if key not in bufs:
                bufs[key] = torch.empty((flat.shape[0] * world, flat.shape[1]), dtype=flat.dtype, device=flat.device)
            dist.all_gather_into_tensor(bufs[key], flat.contiguous())

        class GatheredSparseLinear(torch.nn.Module):
            def __init__(self, sp):
                super().__init__()
                self.sp = sp
                self.prep = capi.Prepared(sp.values, sp.metadata, sp.columns, sp.nrows_sp, sp.ncols_sp, sp.v, sp.m, sp.n)

            def forward(self, x):
                flat = x.reshape(-1, x.shape[-1])
                ns = flat.shape[0]
                key = (ns * world, self.sp.nrows_sp)
                if key not in bufs:
                    bufs[key] = torch.empty(key, dtype=flat.dtype, device=flat.device)
                    if args.peer_store:
                        mgpu_ctx.register_output(bufs[key])   # collective: every rank reaches a new shape at the same layer
                        shared_bufs.append(bufs[key])
                if args.peer_store:
                    full = mgpu_ctx.spmm_gathered_p2p(self.prep, flat.t().contiguous(), ns * world, bufs[key], bias=self.sp.bias)
                else:
                    full = mgpu_ctx.spmm_gathered(self.prep, flat.t().contiguous(), ns * world, bias=self.sp.bias, out=bufs[key], chunks=4)
                return full[rank * ns:(rank + 1) * ns].reshape(*x.shape[:-1], -1)

        for h in hooks:
            h.remove()
        hooks.clear()
        for layer in block:
            for name, child in list(layer.named_children()):
                if hasattr(child, "nrows_sp"):
                    if mgpu_ctx is None:
                        mgpu_ctx = capi.Mgpu.create_torch()
                    setattr(layer, name, GatheredSparseLinear(child))
                elif isinstance(child, torch.nn.Linear):
                    hooks.append(child.register_forward_hook(hook))

    if args.gather_every_layer and world > 1:
        install_gather_hooks()

    def step():
        y = block(x)
        if world > 1:
            dist.all_gather_into_tensor(gathered, y.contiguous())   # shards are contiguous blocks of sequences
            return gathered
        return y

    def max_over_ranks(ms):
        t = torch.tensor(ms, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    d_ms = None
    if not args.skip_dense:
        d_ms = max_over_ranks(time_forward(step, args.repeats))
    replaced = sparsify(block, args.n, args.m, args.v, not args.fixed_mask)
    torch.cuda.empty_cache()
    if args.gather_every_layer and world > 1:
        install_gather_hooks()
    s_ms = max_over_ranks(time_forward(step, args.repeats))
    if rank == 0:
        def line(tag, ms):
            std = statistics.stdev(ms) if len(ms) > 1 else 0.0
            print("0," + tag + str(args.v) + "," + str(statistics.mean(ms)) + "," + str(statistics.median(ms)) + "," + str(std) + "," + str(len(ms)))
        tokens = args.batch * args.seq
        if d_ms:
            line("0,0,", d_ms)
        line("%d,%d," % (args.n, args.m), s_ms)
        msg = "# %d GPUs%s, %d linears replaced (%s mask); %d:%d:%d %.0f tokens/s" % (
            world, (", every linear's output replicated by peer stores" if args.peer_store else ", all-gather after every linear") if args.gather_every_layer and world > 1 else "", replaced,
            "fixed" if args.fixed_mask else "magnitude", args.v, args.n, args.m, tokens / statistics.median(s_ms) * 1e3)
        if d_ms:
            msg += "; dense %.0f tokens/s, speed-up %.2fx" % (tokens / statistics.median(d_ms) * 1e3, statistics.median(d_ms) / statistics.median(s_ms))
        print(msg)
    if world > 1:
        if args.peer_store and mgpu_ctx is not None:
            for buf in shared_bufs:
                mgpu_ctx.unregister_output(buf)
        dist.destroy_process_group()
    return (statistics.median(d_ms) if d_ms else None), statistics.median(s_ms)


if __name__ == "__main__":
    main()
