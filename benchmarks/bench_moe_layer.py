"""Expert layer of a mixture-of-experts model, forward + backward: grouped kernels against per-expert library GEMMs.

    python -m benchmarks.bench_moe_layer [--tokens 16384] [--experts 128] [--topk 8] [--hidden 2048] [--ffn 768]

Qwen3-30B-A3B shapes by default (128 experts of 2048 x 768, 8 per token), uniform-random routing, bf16.  Times
``ops.moe_experts`` (permute -> gate/up GEMM -> SwiGLU -> down GEMM -> combine) forward and forward + backward with
CUDA events (3 warm-ups, 5 iterations; 786 MB of expert weights and 270 MB of permuted activations per pass exceed
L2), once with the backward on the grouped tcgen05 kernels (rows padded to 64 per expert, no host read-back) and once
with ``CLB200_MOE_BWD=library`` semantics (a loop over the experts on library GEMMs after a read-back of the group
sizes).  Prints milliseconds and the expert-GEMM FLOP rate.
"""
import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=768)
    args = ap.parse_args()
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import native_moe
    from chatlearn_b200.ops import reference as ref
    ops.set_mode("native")
    dev = torch.device("cuda", 0)
    T, E, k, H, F = args.tokens, args.experts, args.topk, args.hidden, args.ffn
    torch.manual_seed(0)
    x = torch.randn(T, H, device=dev).bfloat16().requires_grad_(True)
    w13 = (torch.randn(E, 2 * F, H, device=dev) * 0.02).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E, H, F, device=dev) * 0.02).bfloat16().requires_grad_(True)
    wts, idx, _ = ref.moe_router(torch.randn(T, E, device=dev), k)
    wts = wts.detach().requires_grad_(True)
    g = torch.randn(T, H, device=dev).bfloat16()

    def fwd():
        with torch.no_grad():
            ops.moe_experts(x, w13, w2, wts, idx)

    def fwd_bwd():
        for t in (x, w13, w2, wts):
            t.grad = None
        ops.moe_experts(x, w13, w2, wts, idx).backward(g)

    def timed(fn, n=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    flops_fwd = 2.0 * T * k * (2 * F * H + H * F)
    out = {"tokens": T, "experts": E, "topk": k, "hidden": H, "ffn": F, "forward_ms": round(timed(fwd), 3)}
    for impl in ("grouped", "library"):
        native_moe._BWD_IMPL = impl
        ms = timed(fwd_bwd)
        out[f"fwd_bwd_ms_{impl}"] = round(ms, 3)
        out[f"fwd_bwd_TFLOPs_{impl}"] = round(3 * flops_fwd / ms / 1e9, 1)
    out["forward_TFLOPs"] = round(flops_fwd / out["forward_ms"] / 1e9, 1)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
