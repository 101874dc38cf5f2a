"""Per-kernel micro-benchmarks with roofline fractions.

    python -m benchmarks.bench_ops [--only gemm,decode,...] [--json out.json]

Each kernel is timed with CUDA events on the launching stream after warm-up;
between timed iterations a buffer larger than L2 is written so operands start
cold.  Fractions are relative to the measured peaks in ``MEASURED_PEAKS.json``
(copy bandwidth, cuBLAS bf16 throughput) when that file is present.
"""
import argparse
import json
import math
import os

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def timeit(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    only = set(filter(None, args.only.split(",")))
    from chatlearn_b200.ops import native, reference as ref
    hbm, tf, kind = peaks()
    rows = []

    def rec(name, ms, bytes_=0, flops=0, base_ms=None, note=""):
        r = {"kernel": name, "ms": round(ms, 4)}
        if bytes_:
            r["GBps"] = round(bytes_ / ms / 1e6, 1)
            r["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["TFLOPs"] = round(flops / ms / 1e9, 1)
            r["frac_gemm"] = round(flops / ms / 1e9 / tf, 3)
        if base_ms:
            r["library_ms"] = round(base_ms, 4)
            r["speedup_vs_library"] = round(base_ms / ms, 3)
        if note:
            r["note"] = note
        rows.append(r)
        print(json.dumps(r), flush=True)

    dev = "cuda"
    if not only or "gemm" in only:
        for (M, N, K) in [(16384, 6144, 4096), (16384, 4096, 4096), (16384, 24576, 4096), (16384, 4096, 12288),
                          (2048, 151936, 4096), (128, 6144, 4096), (128, 24576, 4096)]:
            a = torch.randn(M, K, device=dev).bfloat16()
            b = torch.randn(N, K, device=dev).bfloat16()
            ms = timeit(lambda: native.C.gemm_bf16_nt(a, b, False))
            base = timeit(lambda: torch.nn.functional.linear(a, b))
            rec(f"gemm_bf16_nt {M}x{N}x{K}", ms, bytes_=2 * (M * K + N * K + M * N), flops=2.0 * M * N * K, base_ms=base)
            if M <= 128:
                native.C.gemm_set_splitk(False)
                ms1 = timeit(lambda: native.C.gemm_bf16_nt(a, b, False))
                native.C.gemm_set_splitk(True)
                rec(f"gemm_bf16_nt {M}x{N}x{K} (split-K off)", ms1, bytes_=2 * (M * K + N * K + M * N), flops=2.0 * M * N * K)
            assert native.C.gemm_last_status() == 0
            del a, b
        # the backward layouts of the same layers over 16384 tokens: dx = dy W (NN), dW += dy^T x (TN, fp32 accumulate)
        for (T, N, K) in [(16384, 6144, 4096), (16384, 24576, 4096), (16384, 4096, 12288)]:
            dy = torch.randn(T, N, device=dev).bfloat16()
            w = torch.randn(N, K, device=dev).bfloat16()
            x = torch.randn(T, K, device=dev).bfloat16()
            acc = torch.zeros(N, K, device=dev)
            ms = timeit(lambda: native.C.gemm_bf16_nn(dy, w, False))
            base = timeit(lambda: torch.mm(dy, w))
            rec(f"gemm_bf16_nn dgrad {T}x{K}x{N}", ms, bytes_=2 * (T * N + N * K + T * K), flops=2.0 * T * N * K, base_ms=base)
            ms = timeit(lambda: native.C.gemm_bf16_tn(dy, x, acc, True, True))
            base = timeit(lambda: acc.add_(torch.mm(dy.t(), x)))
            rec(f"gemm_bf16_tn wgrad+accumulate {N}x{K}x{T}", ms, bytes_=2 * (T * N + T * K) + 8 * N * K, flops=2.0 * T * N * K,
                base_ms=base, note="library: cuBLAS mm + separate fp32 add")
            assert native.C.gemm_last_status() == 0
            del dy, w, x, acc
    if not only or "norm" in only:
        T, H = 16384, 4096
        x = torch.randn(T, H, device=dev).bfloat16()
        w = torch.ones(H, device=dev).bfloat16()
        ms = timeit(lambda: native.C.rmsnorm_fwd(x, w, 1e-6))
        base = timeit(lambda: ref.rmsnorm(x, w, 1e-6))
        rec("rmsnorm_fwd 16384x4096", ms, bytes_=2 * T * H * 2, base_ms=base)
        y, rstd = native.C.rmsnorm_fwd(x, w, 1e-6)
        ms = timeit(lambda: native.C.rmsnorm_bwd(x, w, y, rstd))
        rec("rmsnorm_bwd 16384x4096", ms, bytes_=3 * T * H * 2)
        F = 12288
        gu = torch.randn(T, 2 * F, device=dev).bfloat16()
        ms = timeit(lambda: native.C.swiglu_fwd(gu))
        base = timeit(lambda: ref.swiglu(gu))
        rec("swiglu_fwd 16384x12288", ms, bytes_=3 * T * F * 2, base_ms=base)
        qkv = torch.randn(T, 6144, device=dev).bfloat16()
        pos = torch.arange(T, device=dev)
        qw = torch.ones(128, device=dev).bfloat16()
        inv = native._inv_freq(128, 1e6, x.device)
        ms = timeit(lambda: (native.C.qk_norm_rope_fwd(qkv[:, :4096], 32, 128, qw, pos, inv, 1e-6),
                             native.C.qk_norm_rope_fwd(qkv[:, 4096:5120], 8, 128, qw, pos, inv, 1e-6)))
        q, k = qkv[:, :4096].view(T, 32, 128), qkv[:, 4096:5120].view(T, 8, 128)
        base = timeit(lambda: ref.qk_norm_rope(q, k, qw, qw, 1e-6, pos, 1e6))
        rec("qk_norm_rope_fwd 16384x(32+8)x128", ms, bytes_=2 * T * 5120 * 2, base_ms=base)
    if not only or "decode" in only:
        B, nq, nkv, d, bs = 128, 32, 8, 128, 64
        for L in (512, 2048):
            nblk = math.ceil(L / bs)
            kc = torch.randn(B * nblk + 1, bs, nkv, d, device=dev).bfloat16()
            vc = torch.randn(B * nblk + 1, bs, nkv, d, device=dev).bfloat16()
            bt = torch.randperm(B * nblk, device=dev).view(B, nblk).int()
            sl = torch.full((B,), L, dtype=torch.int32, device=dev)
            q = torch.randn(B, nq, d, device=dev).bfloat16()
            for impl in ("tc", "simt"):
                native.set_decode_impl(impl)
                ms = timeit(lambda: native.paged_attention(q, kc, vc, bt, sl, None, None))
                rec(f"paged_decode[{impl}] B{B} L{L} gqa32/8 d128", ms, bytes_=2 * B * L * nkv * d * 2)
            native.set_decode_impl("tc")
            del kc, vc
    if not only or "sample" in only:
        B, V = 128, 151936
        z = torch.randn(B, V, device=dev) * 2
        u = torch.rand(B, device=dev)
        ms = timeit(lambda: native.C.sample(z, u, 1.0, -1, 1.0, 0.0))
        base = timeit(lambda: ref.sample(z, u, 1.0, -1, 1.0, 0.0))
        rec("sample B128 V151936 (T=1)", ms, bytes_=B * V * 4, base_ms=base, note="3 passes over the logits")
        ms = timeit(lambda: native.C.sample(z, u, 0.6, 20, 0.95, 0.0))
        base = timeit(lambda: ref.sample(z, u, 0.6, 20, 0.95, 0.0))
        rec("sample B128 V151936 (top-k 20, top-p .95)", ms, base_ms=base)
        lab = torch.randint(0, V, (B,), device=dev)
        T2 = 2048
        z2 = torch.randn(T2, V, device=dev)
        lab2 = torch.randint(0, V, (T2,), device=dev)
        ms = timeit(lambda: native.C.logits_stats(z2, lab2, 1.0))
        base = timeit(lambda: (ref.logprobs_from_logits(z2, lab2), ref.entropy_from_logits(z2)))
        rec("logits_stats 2048x151936 fp32", ms, bytes_=T2 * V * 4, base_ms=base)
    if not only or "optim" in only:
        n = 1 << 28
        master, g = torch.randn(n, device=dev), torch.randn(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        out = torch.empty(n, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: native.C.adamw_step(master, g, m, v, out, 1, 1e-4, 0.9, 0.95, 1e-8, 0.01, None, 1.0), iters=5)
        base = timeit(lambda: ref.adamw_step(master, g, m, v, out, 1, 1e-4, 0.9, 0.95, 1e-8, 0.01, 1.0), iters=3)
        rec("adamw_step 268M fp32 -> bf16", ms, bytes_=n * (4 * 7 + 2), base_ms=base)
        ms = timeit(lambda: native.C.sumsq(g), iters=5)
        rec("sumsq 268M fp32", ms, bytes_=n * 4)
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "kind": kind}, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
