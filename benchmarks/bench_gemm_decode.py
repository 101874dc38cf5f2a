"""tcgen05 GEMM on decode shapes: fixed tile widths against the automatic plan.

    python -m benchmarks.bench_gemm_decode

Qwen3-8B layer shapes at tensor-parallel size 1 and 2, 128 and 256 rows.  Every GEMM is timed inside a
CUDA graph that walks enough weight copies to exceed L2 (5 replays, CUDA events); prints microseconds per
GEMM for tile width 0 (automatic), 256, 128, 64, the relative error against the fp32 product, and the
weight-streaming roofline at the measured copy bandwidth.
"""
import json

import torch


def main():
    from chatlearn_b200.ops import native
    C = native.C
    dev = torch.device("cuda")
    shapes = {"tp1": [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)],
              "tp2": [(3072, 4096), (4096, 2048), (12288, 4096), (4096, 6144)]}
    out = {}
    for tag, lst in shapes.items():
        for M in (128, 256):
            for (N, K) in lst:
                copies = max(2, int(400e6 // (N * K * 2)))
                ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
                x = torch.randn(M, K, device=dev).bfloat16()
                row = {}
                for bn in (0, 256, 128, 64):
                    C.gemm_set_tile_n(bn)
                    for i in range(3):
                        C.gemm_bf16_nt(x, ws[i % copies], False)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for i in range(copies):
                            C.gemm_bf16_nt(x, ws[i], False)
                    g.replay()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(5):
                        g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    row[bn] = round(e0.elapsed_time(e1) * 1e3 / (5 * copies), 2)
                C.gemm_set_tile_n(0)
                ref = x.float() @ ws[0].float().t()
                row["rel_err"] = float((C.gemm_bf16_nt(x, ws[0], False).float() - ref).norm() / ref.norm())
                row["roofline_us"] = round(N * K * 2 / 6543e9 * 1e6, 2)
                out[f"{tag} M={M} N={N} K={K}"] = row
                print(f"{tag} M={M} N={N} K={K}", row, flush=True)
                del ws
    print("status", C.gemm_last_status())
    print(json.dumps(out))


if __name__ == "__main__":
    main()
