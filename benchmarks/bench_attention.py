"""Packed causal attention forward: this package's kernels (tensor-memory tcgen05 kernel, warp-level MMA kernel)
next to the flash-attn library.

    python -m benchmarks.bench_attention

Three workloads (6 x 2730, 32 x 512, 2 x 8192 tokens; 32 query / 8 KV heads, head dim 128), 3 warm-up and
10 timed calls each, CUDA events; prints milliseconds and TFLOP/s of causal work per implementation.
"""
import math

import torch


def main():
    from chatlearn_b200.ops import native
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception:                      # the library is optional: report the kernel alone
        flash_attn_varlen_func = None
    dev = torch.device("cuda")
    for lens in ([2730] * 6, [512] * 32, [8192, 8192]):
        T, nq, nkv, D = sum(lens), 32, 8, 128
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
        q = torch.randn(T, nq, D, device=dev).bfloat16()
        k = torch.randn(T, nkv, D, device=dev).bfloat16()
        v = torch.randn(T, nkv, D, device=dev).bfloat16()
        sc = 1 / math.sqrt(D)
        flops = sum(4 * n * n / 2 * D * nq for n in lens)
        impls = [("tcgen05", lambda: native.C.attn_fwd_sm100(q, k, v, cu, sc, True)),
                 ("mma_sync", lambda: native.C.attn_varlen_fwd(q, k, v, cu, sc, True))]
        if flash_attn_varlen_func is not None:
            impls.append(("flash_attn", lambda: flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens),
                                                                        softmax_scale=sc, causal=True)))
        row = {}
        for name, fn in impls:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            row[name] = {"ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1)}
        # backward (dQ, dK, dV; 2.5x the forward's work): the tensor-memory kernel against the library's
        out, lse = native.C.attn_fwd_sm100(q, k, v, cu, sc, True)
        d_out = torch.randn_like(out)
        bwd = [("tcgen05_bwd", lambda: native.C.attn_bwd_sm100(q, k, v, out, d_out, lse, cu, sc, True))]
        if flash_attn_varlen_func is not None:
            qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            og = flash_attn_varlen_func(qg, kg, vg, cu, cu, max(lens), max(lens), softmax_scale=sc, causal=True)
            bwd.append(("flash_attn_bwd", lambda: torch.autograd.grad(og, (qg, kg, vg), d_out, retain_graph=True)))
        for name, fn in bwd:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            row[name] = {"ms": round(ms, 3), "tflops": round(2.5 * flops / ms / 1e9, 1)}
        print(f"{len(lens)} x {lens[0]}", row, flush=True)


if __name__ == "__main__":
    main()
