"""Latent-attention (MLA) decode over the paged latent cache: the tensor-core kernel against batched statements.

    python -m benchmarks.bench_mla_decode [--heads 16] [--batch 128]

Moonlight-16B-A3B shapes: 16 heads, cached rows of 512 latent + 64 rotary values, 64-row blocks, bf16; ragged
contexts as in the GRPO rollout (prompts of 128-1024 tokens plus the tokens generated so far).  The cached rows
of one step exceed L2 (236 MB at a mean context of 1600).  CUDA events around 5 replays of a CUDA graph holding 4
launches; prints microseconds, the fraction of the measured copy bandwidth (cached bytes / time), and the time
of the statements (gather of the block table + two batched matmuls + softmax) on the same inputs.
"""
import argparse
import json
import math
import os

import torch


def timed(fn, reps=4):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (5 * reps) * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--batch", type=int, default=128)
    args = ap.parse_args()
    from chatlearn_b200.models.nn.mla import latent_paged_attention
    from chatlearn_b200.ops import native
    C = native.C
    dev = "cuda"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    bw = json.load(open(p))["hbm_gbs"] if os.path.exists(p) else 6650.0
    torch.manual_seed(0)
    B, nh, D, lora, bs = args.batch, args.heads, 576, 512, 64
    scale = 192 ** -0.5
    for gen in (256, 1024, 2040):
        ctx = (torch.randint(128, 1025, (B,)) + gen).int()
        nblk = [math.ceil(int(c) / bs) for c in ctx]
        total = sum(nblk)
        cache = (torch.randn(total + 1, bs, 1, D, device=dev) * 0.5).bfloat16()
        perm = torch.randperm(total).int()
        bt = torch.zeros(B, max(nblk), dtype=torch.int32)
        o = 0
        for i, n in enumerate(nblk):
            bt[i, :n] = perm[o:o + n]
            o += n
        bt, sl = bt.to(dev), ctx.to(dev)
        q = (torch.randn(B, nh, D, device=dev) * 0.3).bfloat16()
        nbytes = int(ctx.sum()) * D * 2
        row = {}
        for ns in (1, 2, 0):
            us = timed(lambda: C.mla_paged_decode(q, cache, bt, sl, scale, ns))
            row["auto" if ns == 0 else str(ns)] = {"us": round(us, 1), "frac_copy_bw": round(nbytes / us / 1e3 / bw, 3)}
        us = timed(lambda: latent_paged_attention(q, cache, lora, bt, sl, None, 1, scale), reps=1)
        row["statements"] = {"us": round(us, 1)}
        err = (C.mla_paged_decode(q, cache, bt, sl, scale, 0).float()
               - latent_paged_attention(q.float(), cache.float(), lora, bt, sl, None, 1, scale)).abs().max().item()
        print(json.dumps({"generated": gen, "mean_context": round(float(ctx.float().mean())), "cache_MB": round(nbytes / 1e6),
                          "splits": row, "max_abs_err_vs_fp32": round(err, 5)}), flush=True)


if __name__ == "__main__":
    main()
