"""Gated delta-net decode kernel on Qwen3-Next-80B-A3B shapes against the same update on PyTorch statements.

    python -m benchmarks.bench_gdn

32 value heads over 16 key heads, 128 x 128 state per head (fp32), 64 / 128 / 256 sequences.  The state of one
layer (64 KB per head and sequence) is read and written once per token, so the roofline is twice its size over
the measured copy bandwidth; several layers' states are walked so that every launch misses L2.  CUDA events,
5 warm-up and 20 timed rounds; prints microseconds per launch.
"""
import json

import torch


def main():
    from chatlearn_b200.models.nn.hybrid import _l2norm, gated_delta_step
    from chatlearn_b200.ops import native
    C = native.C
    dev = torch.device("cuda")
    nk, nv, dk, dv = 16, 32, 128, 128
    out = {}
    for B in (64, 128, 256):
        layers = max(2, int(600e6 // (B * nv * dk * dv * 4)))
        states = [torch.randn(B, nv, dk, dv, device=dev) * 0.1 for _ in range(layers)]
        q = torch.randn(B, nk, dk, device=dev).bfloat16()
        k = torch.randn(B, nk, dk, device=dev).bfloat16()
        v = torch.randn(B, nv, dv, device=dev).bfloat16()
        g = -torch.rand(B, nv, device=dev)
        beta = torch.rand(B, nv, device=dev)
        slots = torch.randperm(B, device=dev)
        fresh = torch.zeros(B, dtype=torch.bool, device=dev)

        def kernel():
            for s in states:
                C.gdn_decode_step(q, k, v, g, beta, s, slots, fresh, dk ** -0.5)

        def statements():
            qn = (_l2norm(q.float()) * dk ** -0.5).repeat_interleave(nv // nk, dim=1)
            kn = _l2norm(k.float()).repeat_interleave(nv // nk, dim=1)
            for s in states:
                o, S = gated_delta_step(qn, kn, v.float(), g, beta, s.index_select(0, slots))
                s.index_copy_(0, slots, S)

        row = {}
        for name, fn in (("kernel_us", kernel), ("statements_us", statements)):
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                fn()
            e1.record()
            torch.cuda.synchronize()
            row[name] = round(e0.elapsed_time(e1) * 1e3 / (20 * layers), 2)
        row["state_mb"] = round(B * nv * dk * dv * 4 / 1e6, 1)
        row["roofline_us"] = round(2 * B * nv * dk * dv * 4 / 6543e9 * 1e6, 2)
        row["of_measured_copy"] = round(row["roofline_us"] / row["kernel_us"], 3)
        out[f"B={B}"] = row
        print(f"B={B}", row, flush=True)
        del states
    print(json.dumps(out))


if __name__ == "__main__":
    main()
