"""Rollout-engine micro-benchmark: decode step time and its kernel breakdown.

    python -m benchmarks.bench_decode --model qwen3_8b --batch 128 --context 1024 --steps 32

Builds a random-init model, prefills ``batch`` sequences of ``context`` tokens and
times decode steps (CUDA-graph replay and eager).  ``--profile`` prints the
per-kernel device time of one eager step from the PyTorch profiler.
"""
import argparse
import json
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3_8b")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = model default)")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (launch with torchrun --nproc-per-node TP)")
    args = ap.parse_args()
    import os
    tp_group, tp_rank = None, 0
    if args.tp > 1:
        import torch.distributed as dist
        from chatlearn_b200.launcher.initialize import init_distributed
        from chatlearn_b200.parallel.groups import Group
        init_distributed()
        assert dist.get_world_size() == args.tp
        tp_rank = dist.get_rank()
        tp_group = Group(dist.group.WORLD, list(range(args.tp)), "tp")
    from chatlearn_b200 import ops
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.rollout import RolloutEngine, SamplingParams
    from chatlearn_b200.rollout.scheduler import Scheduler, Sequence
    arch = PRESETS[args.model]()
    if args.layers:
        arch.num_hidden_layers = args.layers
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    model = CausalLM(arch, dtype=torch.bfloat16, device=dev, tp=args.tp, tp_rank=tp_rank).init_weights(0)
    max_len = args.context + args.steps * 3 + 64
    eng = RolloutEngine(model, tp_group=tp_group, block_size=64, max_num_seqs=args.batch, max_num_batched_tokens=16384,
                        gpu_memory_utilization=0.8, max_model_len=max_len)
    eng.alloc_kv_cache()
    sched = Scheduler(eng.num_blocks, eng.block_size, args.batch, 16384)
    sp = SamplingParams(temperature=1.0, max_tokens=args.steps * 3 + 8, ignore_eos=True)
    g = torch.Generator().manual_seed(0)
    for i in range(args.batch):
        sched.add(Sequence(i, torch.randint(0, arch.vocab_size - 1, (args.context,), generator=g).tolist(),
                           sp.max_tokens, sp))
    # warm-up outside the timed prefill (library probes, kernel attribute set-up)
    eng.generate([[1, 2, 3, 4]], SamplingParams(temperature=1.0, max_tokens=2, ignore_eos=True))
    # prefill
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while sched.waiting or any(s.length - s.num_computed > 1 for s in sched.running):
        eng.step(sched, sched.schedule(), None)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0

    def run(n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t = time.perf_counter()
        e0.record()
        for _ in range(n):
            eng.step(sched, sched.schedule(), None)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n, (time.perf_counter() - t) * 1e3 / n

    run(3)
    graph_ms, graph_wall = run(args.steps)
    eng.use_graphs = False
    run(2)
    eager_ms, eager_wall = run(args.steps)
    weights_gb = model.num_params() * 2 / 1e9
    kv_gb = args.batch * args.context * eng.kv_bytes_per_block() / eng.block_size / 1e9
    out = {"model": args.model, "layers": arch.num_hidden_layers, "batch": args.batch, "context": args.context,
           "prefill_s": round(prefill_s, 3), "prefill_tok_per_s": round(args.batch * args.context / prefill_s, 1),
           "decode_graph_ms": round(graph_ms, 3), "decode_graph_wall_ms": round(graph_wall, 3),
           "decode_eager_ms": round(eager_ms, 3), "decode_eager_wall_ms": round(eager_wall, 3),
           "weights_gb": round(weights_gb, 2), "kv_gb": round(kv_gb, 2),
           "roofline_ms_at_6543GBps": round((weights_gb + kv_gb) / 6543 * 1e3, 3),
           "library_calls": dict(ops.library_counts)}
    out["tp"] = args.tp
    if tp_rank == 0:
        print(json.dumps(out), flush=True)
    if args.profile:
        # every rank runs the profiled step (it contains collectives); rank 0 prints
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            eng.step(sched, sched.schedule(), None)
            torch.cuda.synchronize()
        if tp_rank == 0:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=18, max_name_column_width=70))
    if args.tp > 1:
        from chatlearn_b200.launcher.initialize import shutdown
        eng._graphs.clear()
        shutdown()


if __name__ == "__main__":
    main()
