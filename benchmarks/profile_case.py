"""Small, self-ending workloads for profiler captures of single kernels.

    python -m benchmarks.profile_case --kernel gemm|gemm_nn|gemm_tn|gemm_decode|decode|rmsnorm|swiglu|logits|adamw|sample|attn_fwd|attn_fwd_sm100|attn_bwd_sm100|grouped_gemm|moe_router

Each case allocates a few hundred MB (operands larger than the 126 MB L2 so DRAM
figures mean something), runs 3 warm-up launches and 3 measured launches of ONE
kernel and exits.  Meant to be run as  `<cmd> && ncu --set full --clock-control none
-k regex:<kernel> -s 3 -c 1 -o <out> <cmd>`.
"""
import argparse
import math

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    a = ap.parse_args()
    from chatlearn_b200.ops import native
    C = native.C
    dev = "cuda"
    torch.manual_seed(0)
    if a.kernel == "gemm":
        A = torch.randn(8192, 4096, device=dev).bfloat16()
        B = torch.randn(4096, 4096, device=dev).bfloat16()
        fn = lambda: C.gemm_bf16_nt(A, B, False)  # noqa: E731
    elif a.kernel == "gemm_nn":          # input gradient of a 4096 -> 12288 layer over 8192 tokens: dx = dy W
        A = torch.randn(8192, 12288, device=dev).bfloat16()
        B = torch.randn(12288, 4096, device=dev).bfloat16()
        fn = lambda: C.gemm_bf16_nn(A, B, False)  # noqa: E731
    elif a.kernel == "gemm_tn":          # weight gradient of the same layer, accumulated into fp32: dW += dy^T x
        A = torch.randn(8192, 12288, device=dev).bfloat16()
        B = torch.randn(8192, 4096, device=dev).bfloat16()
        acc = torch.zeros(12288, 4096, device=dev)
        fn = lambda: C.gemm_bf16_tn(A, B, acc, True, True)  # noqa: E731
    elif a.kernel == "gemm_decode":
        A = torch.randn(128, 4096, device=dev).bfloat16()
        B = torch.randn(24576, 4096, device=dev).bfloat16()
        fn = lambda: C.gemm_bf16_nt(A, B, False)  # noqa: E731
    elif a.kernel == "decode":
        Bsz, nq, nkv, d, bs, L = 64, 32, 8, 128, 64, 2048
        nblk = math.ceil(L / bs)
        kc = torch.randn(Bsz * nblk + 1, bs, nkv, d, device=dev).bfloat16()
        vc = torch.randn(Bsz * nblk + 1, bs, nkv, d, device=dev).bfloat16()
        bt = torch.randperm(Bsz * nblk, device=dev).view(Bsz, nblk).int()
        sl = torch.full((Bsz,), L, dtype=torch.int32, device=dev)
        q = torch.randn(Bsz, nq, d, device=dev).bfloat16()
        fn = lambda: native.paged_attention(q, kc, vc, bt, sl, None, None)  # noqa: E731
    elif a.kernel == "rmsnorm":
        x = torch.randn(32768, 4096, device=dev).bfloat16()
        w = torch.ones(4096, device=dev).bfloat16()
        fn = lambda: C.rmsnorm_fwd(x, w, 1e-6)  # noqa: E731
    elif a.kernel == "swiglu":
        gu = torch.randn(8192, 2 * 12288, device=dev).bfloat16()
        fn = lambda: C.swiglu_fwd(gu)  # noqa: E731
    elif a.kernel == "logits":
        z = torch.randn(1024, 151936, device=dev)
        lab = torch.randint(0, 151936, (1024,), device=dev)
        fn = lambda: C.logits_stats(z, lab, 1.0)  # noqa: E731
    elif a.kernel == "adamw":
        n = 1 << 26
        m0, g = torch.randn(n, device=dev), torch.randn(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        out = torch.empty(n, device=dev, dtype=torch.bfloat16)
        fn = lambda: C.adamw_step(m0, g, m, v, out, 1, 1e-4, 0.9, 0.95, 1e-8, 0.01, None, 1.0)  # noqa: E731
    elif a.kernel == "sample":
        z = torch.randn(128, 151936, device=dev)
        u = torch.rand(128, device=dev)
        fn = lambda: C.sample(z, u, 1.0, -1, 1.0, 0.0)  # noqa: E731
    elif a.kernel == "attn_fwd":
        lens = [2730] * 6
        T, nq, nkv, d = sum(lens), 32, 8, 128
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
        q = torch.randn(T, nq, d, device=dev).bfloat16()
        k = torch.randn(T, nkv, d, device=dev).bfloat16()
        v = torch.randn(T, nkv, d, device=dev).bfloat16()
        fn = lambda: C.attn_varlen_fwd(q, k, v, cu, 1 / math.sqrt(d), True)  # noqa: E731
    elif a.kernel in ("attn_fwd_sm100", "attn_bwd_sm100"):
        lens = [2730] * 6
        T, nq, nkv, d = sum(lens), 32, 8, 128
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
        q = torch.randn(T, nq, d, device=dev).bfloat16()
        k = torch.randn(T, nkv, d, device=dev).bfloat16()
        v = torch.randn(T, nkv, d, device=dev).bfloat16()
        sc = 1 / math.sqrt(d)
        if a.kernel == "attn_fwd_sm100":
            fn = lambda: C.attn_fwd_sm100(q, k, v, cu, sc, True)  # noqa: E731
        else:
            out, lse = C.attn_fwd_sm100(q, k, v, cu, sc, True)
            d_out = torch.randn_like(out)
            fn = lambda: C.attn_bwd_sm100(q, k, v, out, d_out, lse, cu, sc, True)  # noqa: E731
    elif a.kernel == "grouped_gemm":
        # Qwen3-30B-A3B expert up-projection: 128 experts, 16384 tokens x top-8 rows, [1536, 2048] each
        E, R, N, K = 128, 16384 * 8, 1536, 2048
        xs = torch.randn(R, K, device=dev).bfloat16()
        w = (torch.randn(E, N, K, device=dev) * 0.02).bfloat16()
        cnt = torch.randint(600, 1450, (E,))
        cnt = (cnt.float() / cnt.sum() * R).long()
        cnt[-1] += R - cnt.sum()
        off = torch.zeros(E + 1, dtype=torch.long)
        off[1:] = cnt.cumsum(0)
        off = off.to(dev)
        fn = lambda: C.grouped_gemm_bf16_nt(xs, w, off)  # noqa: E731
    elif a.kernel == "moe_router":
        z = torch.randn(131072, 128, device=dev)
        fn = lambda: C.moe_router_topk(z, 8, False, True, None, 1, 1, 1.0)  # noqa: E731
    else:
        raise SystemExit(f"unknown kernel {a.kernel}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print("done", a.kernel, f"{e0.elapsed_time(e1) / 3 * 1e3:.1f} us per call")


if __name__ == "__main__":
    main()
