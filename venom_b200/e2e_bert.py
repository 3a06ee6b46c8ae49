"""BERT-large encoder inference, dense vs V:N:M, through the `spatha` torch op.

Mirrors the reference's end2end/bert_pytorch.py (argument names -m -n -v, the replacement of every
encoder torch.nn.Linear by SrnmSpmm, the output lines `0,n,m,v,mean,median,std,len` in milliseconds), with
three differences that the missing network access and the missing `sten` dependency force or allow:
  * weights are random-init N(0, 0.02) from a BertConfig (no hub download); token ids are uniform random;
  * linears are pruned by magnitude on the GPU (the path the reference keeps commented out) unless
    --fixed-mask asks for the shipped fixed pattern;
  * timing uses CUDA events around each forward pass instead of timeit without synchronisation.

    python -m venom_b200.e2e_bert -m 8 -n 2 -v 64 [--layers 24] [--batch 32] [--seq 512] [--repeats 10]
"""
import argparse
import statistics

import torch


def build_model(layers, hidden=1024, heads=16, ffn=4096, vocab=30522):
    from transformers import BertConfig, BertModel
    cfg = BertConfig(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                     intermediate_size=ffn, hidden_act="gelu", max_position_embeddings=512, initializer_range=0.02)
    return BertModel(cfg, add_pooling_layer=False).eval()


def sparsify_encoder(model, n, m, v, fixed_mask=False):
    from .nmv import MagnitudeSparsifier, NMVectorSparsifier, SrnmSpmm
    sp = (NMVectorSparsifier if fixed_mask else MagnitudeSparsifier)(n, m, v)
    count = 0
    for name, mod in list(model.named_modules()):
        if "encoder.layer" not in name:
            continue
        for cname, child in list(mod.named_children()):
            if isinstance(child, torch.nn.Linear):
                setattr(mod, cname, SrnmSpmm(child, n, m, v, sparsifier=sp))
                count += 1
    return count


def time_forward(model, ids, repeats, warmup=3):
    for _ in range(warmup):
        model(ids)
    torch.cuda.synchronize()
    ms = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model(ids)
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    return ms


def report_time(name, ms, n, m, v):
    cfg = "%d,%d," % (n, m) if name == "n:m" else "0,0,"
    std = statistics.stdev(ms) if len(ms) > 1 else 0.0
    print("0," + cfg + str(v) + "," + str(statistics.mean(ms)) + "," + str(statistics.median(ms)) + "," + str(std) + "," + str(len(ms)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", type=int, default=8)
    ap.add_argument("-n", type=int, default=2)
    ap.add_argument("-v", type=int, default=64)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--fixed-mask", action="store_true")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device (there is no CPU path)")
    torch.set_grad_enabled(False)
    torch.manual_seed(0)
    dense = build_model(args.layers).half().cuda()
    sparse = build_model(args.layers).half().cuda()
    sparse.load_state_dict(dense.state_dict())
    replaced = sparsify_encoder(sparse, args.n, args.m, args.v, args.fixed_mask)
    ids = torch.randint(0, 30522, (args.batch, args.seq), device="cuda")
    d_ms = time_forward(dense, ids, args.repeats)
    s_ms = time_forward(sparse, ids, args.repeats)
    report_time("dense", d_ms, args.n, args.m, args.v)
    report_time("n:m", s_ms, args.n, args.m, args.v)
    tokens = args.batch * args.seq
    print("# %d linears replaced; dense %.0f tokens/s, %d:%d:%d %.0f tokens/s, speed-up %.2fx" % (
        replaced, tokens / statistics.median(d_ms) * 1e3, args.v, args.n, args.m, tokens / statistics.median(s_ms) * 1e3,
        statistics.median(d_ms) / statistics.median(s_ms)))
    return statistics.median(d_ms), statistics.median(s_ms)


if __name__ == "__main__":
    main()
