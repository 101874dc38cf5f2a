"""Where a training micro-batch spends its time: forward + backward of a few layers of the flagship model.

    python -m benchmarks.bench_train_layers [--layers 4] [--tokens 16384] [--seqs 6] [--profile] [--recompute]

Qwen3-8B shapes with ``--layers`` decoder layers (the per-layer cost times 36 plus the head is the cost of a
micro-batch of the flagship trainer), one packed row of ``--tokens`` tokens in ``--seqs`` sequences, bf16, the
trainer's own state (fp32 gradient buffers that the weight-gradient GEMMs accumulate into).  Times forward,
forward + backward and the optimizer step with CUDA events (3 warm-up, 5 timed iterations; the activations and
weights of an iteration exceed L2), prints the model FLOPs rate against the measured cuBLAS peak, and with
``--profile`` the per-kernel device time of one forward + backward from the PyTorch profiler.
"""
import argparse
import json
import os

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3_8b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--seqs", type=int, default=6)
    ap.add_argument("--recompute", action="store_true", help="recompute every layer in backward")
    ap.add_argument("--profile", action="store_true")
    args = ap.parse_args()
    from chatlearn_b200 import ops
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.models.nn.model import FwdCtx, decoder_layer
    from chatlearn_b200.parallel.zero import ShardedTrainState
    ops.set_mode("native")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    arch = PRESETS[args.model]()
    arch.num_hidden_layers = args.layers
    model = CausalLM(arch, dtype=torch.bfloat16, device=dev).init_weights(0)
    state = ShardedTrainState(model, lr=2e-6)
    T, S = args.tokens, args.seqs
    lens = [T // S] * S
    lens[-1] += T - sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    tokens = torch.randint(0, arch.vocab_size - 1, (T,), device=dev)
    labels = torch.roll(tokens, -1)
    positions = torch.cat([torch.arange(n, device=dev) for n in lens])
    hook = None
    if args.recompute:
        from torch.utils.checkpoint import checkpoint

        def hook(l, p, x, c):
            return checkpoint(lambda xx: decoder_layer(arch, p, xx, c, l), x, use_reentrant=False)

    def forward():
        ctx = FwdCtx(positions=positions, cu_seqlens=cu, max_seqlen=max(lens), fuse_add_norm=False)
        h = model.hidden_states(tokens, ctx, hook)
        lp, ent = ops.lmhead_logprob_entropy(h, model.lm_head_weight(), labels)
        return -(lp.mean()) + 0.0 * ent.mean()

    def fwd_bwd():
        forward().backward()

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

    with torch.no_grad():
        t_f = timed(forward)
    state.zero_grad()
    t_fb = timed(fwd_bwd)
    t_opt = timed(lambda: state.step(), n=3)
    H, F, V = arch.hidden_size, arch.intermediate_size, arch.vocab_size
    qd, kvd = arch.num_attention_heads * arch.head_dim, arch.num_key_value_heads * arch.head_dim
    lin = 2 * T * (H * (qd + 2 * kvd) + qd * H + 3 * H * F)                  # per layer, forward
    attn = sum(2 * 2 * n * n * qd / 2 for n in lens)                          # causal: half of the square
    head = 2 * T * H * V
    fwd_flops = args.layers * (lin + attn) + head
    fb_flops = 3 * fwd_flops + (args.layers * (lin + attn) if args.recompute else 0)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    peak = json.load(open(p)).get("bf16_tflops_sustained", 1400.0) if os.path.exists(p) else 1400.0
    print(json.dumps({"layers": args.layers, "tokens": T, "seqs": S, "recompute": args.recompute,
                      "forward_ms": round(t_f, 2), "fwd_bwd_ms": round(t_fb, 2), "optimizer_ms": round(t_opt, 2),
                      "forward_TFLOPs": round(fwd_flops / t_f / 1e9, 1), "fwd_bwd_TFLOPs": round(fb_flops / t_fb / 1e9, 1),
                      "frac_of_measured_sustained_gemm": round(fb_flops / t_fb / 1e9 / peak, 3),
                      "library_calls": {k: int(v) for k, v in ops.library_counts.items()}}), flush=True)
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fwd_bwd()
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=28, max_name_column_width=64))


if __name__ == "__main__":
    main()
