"""Flagship benchmark: GRPO samples/sec and step time (rollout + sync + train).

    python bench.py --gpus N --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one GRPO episode through the public ``Engine`` API: rollout with the
native engine → old / reference log-probs → rule reward → group advantages →
optimizer steps → trainer→rollout weight sync.  Model and workload follow the
Qwen3-8B GRPO configuration (36 layers, hidden 4096, 32/8 heads, FFN 12288, vocab
151936; 16 prompts x 8 samples per GPU, prompts uniform in [128, 1024] tokens,
responses up to 2048 tokens, packing to 16k tokens, 2 mini-batches per step,
optimizer offload during rollout), with synthetic prompts, the hash reward and
random-init weights.  Per-GPU work is fixed as N grows (weak scaling).

Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

T_START = time.time()
ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=["native", "library", "reference"])
    p.add_argument("--model", default="qwen3_8b")
    p.add_argument("--prompts-per-gpu", type=int, default=16)
    p.add_argument("--samples-per-prompt", type=int, default=8)
    p.add_argument("--prompt-len", type=int, nargs=2, default=[128, 1024])
    p.add_argument("--max-response", type=int, default=2048)
    p.add_argument("--pack-tokens", type=int, default=16384)
    p.add_argument("--gemm", default=None, choices=[None, "tcgen05", "cublas"])
    p.add_argument("--layers", type=int, default=0,
                   help="run the model with this many decoder layers instead of its own depth (exercises a large "
                        "architecture on few GPUs; the JSON line then names the reduced depth and is not a figure "
                        "for the full model)")
    p.add_argument("--ulysses", type=int, default=1,
                   help="Ulysses sequence-parallel size of the trainer and the reference model (heads <-> sequence "
                        "all-to-all around attention, through the peer-memory exchange kernels)")
    p.add_argument("--no-offload", action="store_true")
    p.add_argument("--rollout-tp", type=int, default=1,
                   help="tensor-parallel size of a rollout replica (1: every GPU generates for its own samples; 2: pairs "
                        "of GPUs share a replica through the fused GEMM + all-reduce kernel, 13.1 ms per decode step of "
                        "256 sequences against 10.4 ms for 128 on one GPU)")
    p.add_argument("--reshard", action="store_true",
                   help="parameter-sharded trainer (FSDP2 reshard_after_forward): 1/N of parameters, gradients and "
                        "optimizer state resident per GPU instead of whole bf16 parameters and fp32 gradients")
    p.add_argument("--time-budget", type=float, default=float(os.environ.get("CLB200_BENCH_BUDGET", "740")),
                   help="wall-clock seconds for the whole process (set-up included).  When the requested "
                        "warm-up + steps would not fit, warm-up is cut to no fewer than 3 episodes and the "
                        "timed loop stops early; the JSON line reports the steps actually timed.  0 = no limit")
    return p.parse_args()


def reference_arm(args):
    """The unmodified reference cannot run here: importing its public API fails."""
    why = None
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import chatlearn  # noqa: F401
        from chatlearn.runtime.engine import Engine  # noqa: F401
    except Exception as e:  # noqa: BLE001
        why = f"reference public API does not import offline ({type(e).__name__}: {e}); " \
              "it needs ray, hydra/omegaconf and vllm==0.8.5, none installed"
    if why is None:
        why = "reference imports but needs a Ray cluster, Megatron/FSDP HF weights and vllm==0.8.5 to run"
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))
    return 0


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampling during the timed region (rank 0)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, enabled):
        self.proc, self.path = None, None
        if enabled:
            self.path = tempfile.mktemp(suffix=".csv")
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                    stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            except OSError:
                self.proc = None

    def stop(self, gpu_index=0):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9 or f[0] != str(gpu_index):
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            # under load = samples in the upper half of the observed power/clock activity
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


def vs_baseline(n_gpu, value, args):
    """value / the same-box library-class baseline of this configuration at this GPU count: this framework
    with torch matmul, flash-attn and NCCL statements in place of its kernels (``--impl library``), recorded in
    ``baseline/library_baseline.json``.  The reference publishes no GRPO throughput and cannot run here, so
    this is the number there is to divide by; None where no record exists for the configuration."""
    try:
        rec = json.load(open(os.path.join(ROOT, "baseline", "library_baseline.json")))
        r = rec["runs"].get(str(n_gpu))
        same = rec["config"] == {"model": args.model, "prompts_per_gpu": args.prompts_per_gpu,
                                 "samples_per_prompt": args.samples_per_prompt, "prompt_len": list(args.prompt_len),
                                 "max_response": args.max_response, "pack_tokens": args.pack_tokens}
        return round(value / r["value"], 4) if (r and same and args.impl == "native") else None
    except (OSError, KeyError, ValueError, ZeroDivisionError):
        return None


def rollout_trainer_diff(out_dir, last_k):
    """Mean |log-prob the rollout engine sampled with - log-prob the trainer assigns to the same token| over the
    timed episodes (from the run's metrics file): a check that generation and scoring see the same model."""
    try:
        vals = [v for line in open(os.path.join(out_dir, "metrics.jsonl")) for k, v in json.loads(line).items()
                if k.endswith("rollout_logprob_abs_diff")]
        vals = vals[-last_k:]
        return round(sum(vals) / len(vals), 6) if vals else None
    except (OSError, ValueError):
        return None


def build_config(args, out_dir, data_path, n_gpu):
    tp = max(1, min(int(args.rollout_tp), n_gpu))
    n = args.samples_per_prompt
    spe = args.prompts_per_gpu * n * n_gpu
    offload = not args.no_offload
    arch = {"preset": args.model}
    if args.layers > 0:
        arch["num_hidden_layers"] = args.layers
    seq = args.prompt_len[1] + args.max_response
    common = {"model_arch": arch, "packing": True, "max_token_in_packing": args.pack_tokens,
              "max_prompt_tokens_length": args.prompt_len[1] + 1, "max_response_tokens_length": args.max_response}
    return {
        "runtime_args": {
            "train_backend": "fsdp", "rollout_backend": "native", "exp_name": "bench",
            "colocation": ["policy", "policy_trainer", "ref_policy"], "output_dir": out_dir,
            "data_path": data_path, "num_episode": args.steps + args.warmup, "sample_per_episode": spe,
            "train_micro_batch_size": 1, "train_global_batch_size": spe // 2, "num_inference_per_prompt": n,
            "save_episode_interval": 0, "max_replay_episode": 1, "data_shuffle": False,
            "enable_resume_training": False, "log_args_dict": {"log_dir": out_dir}},
        "models": {
            "policy_trainer": dict(common, num_gpu=n_gpu, fsdp_size=n_gpu, trainable=True,
                                   generation_batch_size=spe, kl_coef=0.001, gradient_checkpointing=True,
                                   # the library statements save more per layer than the estimate behind
                                   # "auto" assumes (they ran out of memory with it): every layer recomputes
                                   checkpoint_layers="all" if args.impl == "library" else "auto",
                                   optimizer={"lr": 2e-6}, save_hf=False, reshard_after_forward=bool(args.reshard),
                                   ulysses_sequence_parallel_size=int(args.ulysses),
                                   # fp32 master + Adam shards stay on the GPU (180 GB HBM); the fp32
                                   # gradient buffer is released outside training
                                   # On one GPU (all optimizer state on it) the bf16 compute copy is dropped
                                   # outside training and rebuilt by a cast of the resident master weights:
                                   # 16 GB more KV cache for the rollout.
                                   free_gpu_memory={"offload_weights": offload and n_gpu == 1,
                                                    "offload_optimizer_states": False,
                                                    "free_grad_buffers": offload}),
            # the frozen reference weights (16 GB) go to pinned host memory between uses only where the
            # GPU is short of room (1-2 GPUs hold large optimizer shards); from 4 GPUs on they stay resident
            "ref_policy": dict(common, num_gpu=n_gpu, fsdp_size=n_gpu, generation_batch_size=spe,
                               ulysses_sequence_parallel_size=int(args.ulysses),
                               free_gpu_memory={"offload_weights": offload and n_gpu < 4}),
            "policy": dict(common, num_gpu=n_gpu, tensor_model_parallel_size=tp, generation_batch_size=spe,
                           num_inference_per_prompt=n, temperature=1.0, top_p=1.0, top_k=-1,
                           gpu_memory_utilization=0.94, max_num_seqs=256, kv_block_size=64,
                           max_num_batched_tokens=16384, ignore_eos=True,
                           free_gpu_memory={"offload_weights": offload}),
            "reward": {"num_cpu": n_gpu, "synthetic_reward": "hash30"},
        }}, seq


def main():
    import faulthandler
    faulthandler.enable()
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist
    from chatlearn_b200 import ops
    from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig
    from chatlearn_b200.configs import resolve, to_dataclass
    from chatlearn_b200.data.synthetic import make_prompts, write_jsonl
    from chatlearn_b200.models.nn import PRESETS
    from chatlearn_b200.utils import xfer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun when started as a plain script
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29577", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    assert torch.cuda.is_available(), "bench.py needs CUDA devices"
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29578")
        os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1"); os.environ.setdefault("LOCAL_RANK", "0")
    # --impl library: the trainer and the reference policy (scoring passes, forward + backward, optimizer) run on
    # library statements (torch matmul = cuBLAS, flash-attn, PyTorch elementwise ops, NCCL collectives) instead
    # of this package's kernels.  The rollout keeps the native engine: generation on PyTorch statements has no
    # CUDA graphs and synchronises with the host every token, and did not finish one episode in 20 minutes; the
    # library-class rollout figure is vLLM's, measured by baseline/vllm_rollout.py.
    ops.set_mode("native")
    if args.gemm:
        from chatlearn_b200.ops import native
        native.set_gemm_impl(args.gemm)

    out_dir = os.environ.get("BENCH_OUT", os.path.join(tempfile.gettempdir(), f"clb200_bench_{os.getpid() if world == 1 else os.environ.get('MASTER_PORT', '0')}"))
    os.makedirs(out_dir, exist_ok=True)
    data_path = os.path.join(out_dir, "prompts.jsonl")
    arch = PRESETS[args.model]()
    total_steps = args.steps + args.warmup
    if rank == 0:
        rows = make_prompts(args.prompts_per_gpu * world * total_steps, args.prompt_len[0], args.prompt_len[1],
                            arch.vocab_size, seed=1234, data_source="synthetic:hash30")
        write_jsonl(rows, data_path + ".tmp")
        os.replace(data_path + ".tmp", data_path)
    while not os.path.exists(data_path):
        time.sleep(0.05)

    cfg_dict, seq = build_config(args, out_dir, data_path, world)
    cfg = to_dataclass(GrpoConfig, resolve(cfg_dict))
    algo = GrpoAlgorithm(cfg)
    algo.validate()
    engine = algo.build_engine()
    engine.prepare()
    if args.impl == "library":
        import functools
        for role in ("policy_trainer", "ref_policy"):
            m = engine.named_models[role]          # (filled by prepare())
            for fn_name in ("forward_step", "train_step"):
                fn = getattr(m, fn_name, None)
                if fn is None:
                    continue

                def wrapped(*a, _fn=fn, **k):
                    with ops.mode("library"):
                        return _fn(*a, **k)
                setattr(m, fn_name, functools.wraps(fn)(wrapped))

    def barrier():
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        torch.cuda.synchronize()

    multi = dist.is_initialized() and dist.get_world_size() > 1

    def fits(n_more: int, step_s: float) -> bool:
        """Do ``n_more`` further episodes of ``step_s`` seconds fit in the time budget?  Every rank must
        take the same decision (an episode is collective): the slowest rank's clock decides."""
        if args.time_budget <= 0:
            return True
        left = args.time_budget - (time.time() - T_START) - 15.0 - 1.1 * n_more * step_s
        if multi:
            t = torch.tensor([left], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            left = float(t.item())
        return left >= 0.0

    # warm-up: as many as requested while the rest of the run still fits; never fewer than 3 unless fewer were asked for
    done_warm, last = 0, 0.0
    for ep in range(args.warmup):
        if ep >= min(3, args.warmup) and not fits(args.warmup - ep + min(args.steps, 2), last):
            break
        t_ep = time.time()
        engine.run_episode(ep)
        last = time.time() - t_ep
        done_warm += 1
    barrier()
    sampler = ClockSampler(rank == 0)
    xfer.reset()
    launches0 = sum(ops.launch_counts.values())
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    summaries = []
    for i in range(args.steps):
        if i >= 1 and not fits(1, last):
            break
        t_ep = time.time()
        summaries.append(engine.run_episode(done_warm + i))
        last = time.time() - t_ep
    done_steps = len(summaries)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    dev_ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(int(os.environ.get("LOCAL_RANK", "0")))
    t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device="cuda")
    cnt = torch.tensor([float(sum(ops.launch_counts.values()) - launches0), float(xfer.h2d_bytes), float(xfer.d2h_bytes)],
                       dtype=torch.float64, device="cuda")
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(cnt, op=dist.ReduceOp.SUM)
    dev_ms, wall_ms = t.tolist()
    launches, h2d, d2h = cnt.tolist()
    if rank == 0:
        K = done_steps
        samples = cfg.runtime_args.sample_per_episode
        ms_per_step = dev_ms / K
        value = samples / (ms_per_step / 1e3)
        tokens = sum(s.get("tps_throughput", 0.0) * s.get("episode", 0.0) for s in summaries) / max(K, 1)
        phases = {k: sum(s.get(k, 0.0) for s in summaries) / K for k in ("environment", "train", "sync_parameters")}
        tr = engine.named_models["policy_trainer"]
        sync_ms = [g.last_ms for g in engine.model_manager.parameter_sync_groups.values()]
        line = {
            "metric": "GRPO samples/sec (rollout+sync+train step)", "value": round(value, 4), "unit": "samples/s",
            "n_gpus": world, "steps": K, "warmup": done_warm, "steps_requested": args.steps,
            "warmup_requested": args.warmup, "time_budget_s": args.time_budget, "ms_per_step": round(ms_per_step, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": vs_baseline(world, value, args), "dtype": "bf16", "data": "synthetic",
            "impl": args.impl if args.impl == "native" else "library trainer (cuBLAS + flash-attn + PyTorch statements), native rollout",
            "config": {"model": args.model if args.layers <= 0 else f"{args.model} cut to {args.layers} layers",
                       "global_batch": samples, "seq_len": seq,
                       "trainer_parameters": "sharded 1/N per GPU (gathered per segment)" if args.reshard else "whole per GPU (optimizer state sharded)",
                       "parallelism": (f"ulysses{args.ulysses} x " if args.ulysses > 1 else "") + f"trainer zero-dp{world} + rollout tp{max(1, min(args.rollout_tp, world))}x{world // max(1, min(args.rollout_tp, world))}",
                       "prompts": samples // args.samples_per_prompt, "samples_per_prompt": args.samples_per_prompt,
                       "prompt_len": args.prompt_len, "max_response": args.max_response,
                       "pack_tokens": args.pack_tokens, "mini_batches_per_step": 2,
                       "activation_recompute": "every layer" if args.impl == "library" else "as many layers kept as fit (auto)",
                       "ignore_eos": True, "response_len": "every response runs to max_response (random weights)",
                       "l2_policy": "inputs larger than L2 (16 GB of weights + KV streamed every step)",
                       "gemm": __import__("chatlearn_b200.ops.native", fromlist=["x"]).get_gemm_impl() if args.impl == "native" else "cublas"},
            "step_time_s": round(ms_per_step / 1e3, 3),
            "phase_s": {k: round(v, 3) for k, v in phases.items()},
            "weight_sync_ms": round(max(sync_ms), 3) if sync_ms else None,
            "tokens_per_s": round(tokens / (ms_per_step / 1e3), 1) if tokens else None,
            "rollout_tok_per_s": round(samples * args.max_response / max(phases["environment"], 1e-9), 1),
            "clocks": clocks,
            "e2e": {"value": round(samples / (wall_ms / 1e3 / K), 4), "unit": "samples/s",
                    "h2d_bytes_per_step": int(h2d / K), "d2h_bytes_per_step": int(d2h / K),
                    "how": "host wall clock around the same K episodes driven through Engine.run_episode"},
            "rollout_vs_trainer_logprob_abs_diff": rollout_trainer_diff(out_dir, K),
            "gpu_launches": int(launches),
            "library_calls": {k: int(v) for k, v in ops.library_counts.items()},
        }
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        from chatlearn_b200.launcher.initialize import shutdown
        shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
