"""Paged decode attention: effect of splitting every sequence's context over several CTAs.

    python -m benchmarks.bench_paged_decode

128 sequences with ragged contexts (the decode batch of the GRPO rollout: prompts of 128-1024 tokens plus the
tokens generated so far), 32 query / 8 KV heads, head dim 128, 64-token blocks, bf16.  Each variant runs inside a
CUDA graph over enough distinct KV blocks to exceed L2; CUDA events, 5 replays.  Prints microseconds and the
fraction of the measured copy bandwidth for 1, 2, 3, 4 and 6 splits and for the automatic choice.
"""
import json
import math
import os

import torch


def main():
    from chatlearn_b200.ops import native
    C = native.C
    dev = "cuda"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    bw = json.load(open(p))["hbm_gbs"] if os.path.exists(p) else 6650.0
    torch.manual_seed(0)
    B, nq, nkv, d, bs = 128, 32, 8, 128, 64
    for gen in (256, 1024, 2040):
        ctx = (torch.randint(128, 1025, (B,)) + gen).int()
        nblk = [math.ceil(int(c) / bs) for c in ctx]
        total = sum(nblk)
        kc = torch.randn(total + 1, bs, nkv, d, device=dev).bfloat16()
        vc = torch.randn(total + 1, bs, nkv, d, device=dev).bfloat16()
        perm = torch.randperm(total).int()
        bt = torch.zeros(B, max(nblk), dtype=torch.int32)
        o = 0
        for i, n in enumerate(nblk):
            bt[i, :n] = perm[o:o + n]
            o += n
        bt, sl = bt.to(dev), ctx.to(dev)
        q = torch.randn(B, nq, d, device=dev).bfloat16()
        kv_bytes = int(ctx.sum()) * nkv * d * 2 * 2
        row = {}
        auto = native._num_splits(B * nkv, bt.shape[1])
        for ns in (1, 2, 3, 4, 6, "auto"):
            n = auto if ns == "auto" else ns
            fn = lambda: C.paged_decode_tc(q, kc, vc, bt, None, sl, 1 / math.sqrt(d), n)  # noqa: E731
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(4):
                    fn()
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 20 * 1e3
            row[f"{ns}" + (f"(={n})" if ns == "auto" else "")] = {"us": round(us, 1), "frac_copy_bw": round(kv_bytes / us / 1e3 / bw, 3)}
        print(f"generated {gen}: mean context {float(ctx.float().mean()):.0f}, KV {kv_bytes / 1e6:.0f} MB", row, flush=True)


if __name__ == "__main__":
    main()
