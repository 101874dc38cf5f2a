"""Parameter-sharded (FSDP2-style) training state against the replicated one, on gloo with two ranks."""
import json

from tests.dist_utils import run_ranks

UNIT = r'''
import json, os, torch, torch.distributed as dist
from chatlearn_b200.launcher.initialize import init_distributed
from chatlearn_b200.models.nn import PRESETS, CausalLM, packed_ctx
from chatlearn_b200.parallel.groups import Group
from chatlearn_b200.parallel.zero import ShardedTrainState
from chatlearn_b200.parallel.fsdp2 import ReshardedTrainState

init_distributed()
rank, world = dist.get_rank(), dist.get_world_size()
g = Group(dist.group.WORLD, list(range(world)), "dp")
dev = torch.device("cpu")
arch = PRESETS[os.environ.get("PRESET", "tiny_qwen3")]()
ma = CausalLM(arch, dtype=torch.float32, device=dev, pad_to=world * 8).init_weights(7)
mb = CausalLM(arch, dtype=torch.float32, device=dev, pad_to=world * 8).init_weights(7)
sa = ShardedTrainState(ma, g, lr=1e-2, clip_grad=1.0)
sb = ReshardedTrainState(mb, g, lr=1e-2, clip_grad=1.0)
assert all(s.block.flat is None for s in sb.states), "no whole block may stay bound between segments"
res = {"rank": rank, "loss": [], "norm": []}
for step in range(2):
    sa.zero_grad(); sb.zero_grad()
    # rank 1 has one micro-batch fewer than rank 0 in the first step: it still joins the reduce-scatters
    nmb = 2 if (rank == 0 or step == 1) else 1
    for mbi in range(2):
        if mbi >= nmb:
            sb.join_empty_microbatch()
            continue
        torch.manual_seed(100 * step + 10 * mbi + rank)
        lens = [17 + rank, 30, 5 + mbi]
        T = sum(lens)
        toks = torch.randint(0, arch.vocab_size - 1, (T,))
        labels = toks.roll(-1)
        ctx_a, _ = packed_ctx(lens, dev)
        ctx_b, _ = packed_ctx(lens, dev)
        lp_a, ent_a = ma.logprobs(toks, labels, ctx_a)
        lp_b, ent_b = sb.logprobs(toks, labels, ctx_b)
        la = -(lp_a.sum() + 0.01 * ent_a.sum()) / T
        lb = -(lp_b.sum() + 0.01 * ent_b.sum()) / T
        la.backward(); lb.backward()
        res["loss"].append((la.item(), lb.item()))
    na, nb = sa.step(), sb.step()
    res["norm"].append((float(na), float(nb)))
# scoring pass without a tape
with torch.no_grad():
    lens = [9, 20]
    toks = torch.randint(0, arch.vocab_size - 1, (sum(lens),))
    c1, _ = packed_ctx(lens, dev); c2, _ = packed_ctx(lens, dev)
    res["score_diff"] = (ma.logprobs(toks, toks.roll(-1), c1)[0] - sb.logprobs(toks, toks.roll(-1), c2)[0]).abs().max().item()
# the two models after two optimizer steps
with sb.all_gathered() as whole:
    res["param_diff"] = max((x.flat - y.flat).abs().max().item() for x, y in zip(ma.blocks, whole.blocks))
assert all(s.block.flat is None for s in sb.states)
res["resident_fraction"] = sum(s.param_shard.numel() for s in sb.states) / sum(b.numel for b in ma.blocks)
print("RESULT " + json.dumps(res))
'''


def _results(outs):
    return [json.loads(l[7:]) for o in outs for l in o.splitlines() if l.startswith("RESULT ")]


def test_resharded_state_matches_replicated_state():
    outs, _ = run_ranks(UNIT, 2)
    res = _results(outs)
    assert len(res) == 2
    for r in res:
        for la, lb in r["loss"]:
            assert abs(la - lb) < 1e-5 * max(1.0, abs(la)), r
        for na, nb in r["norm"]:
            assert abs(na - nb) < 1e-4 * max(1.0, abs(na)), r
        # AdamW normalises every element's update to about lr = 1e-2, so a last-bit difference in a tiny gradient
        # (the sharded state sums micro-batches after the reduce-scatter, the replicated one before) shows up as a
        # small fraction of one update
        assert r["score_diff"] < 1e-5 and r["param_diff"] < 5e-4, r
        assert abs(r["resident_fraction"] - 0.5) < 1e-6


def test_resharded_state_with_expert_blocks():
    outs, _ = run_ranks(UNIT, 2, env={"PRESET": "tiny_moe"})
    res = _results(outs)
    assert len(res) == 2
    for r in res:
        # the router's auxiliary loss is not part of this loss, so the two states must still agree
        assert r["param_diff"] < 5e-4 and r["score_diff"] < 1e-4, r


E2E = r'''
import os, json, torch, time
from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl

out = os.environ["OUT_DIR"]
data = os.path.join(out, "train.jsonl")
if int(os.environ["RANK"]) == 0:
    write_jsonl(make_prompts(8, 16, 48, 1024, seed=0, data_source="synthetic:mod7"), data + ".tmp")
    os.replace(data + ".tmp", data)
while not os.path.exists(data): time.sleep(0.05)
arch = {"preset": "tiny_qwen3"}
cfg = {
  "runtime_args": {"train_backend": "fsdp", "rollout_backend": "native", "exp_name": "tiny",
     "colocation": ["policy", "policy_trainer", "ref_policy"], "output_dir": out, "data_path": data,
     "num_episode": 2, "sample_per_episode": 32, "train_micro_batch_size": 4, "train_global_batch_size": 32,
     "num_inference_per_prompt": 4, "save_episode_interval": 1, "max_replay_episode": 2,
     "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": {"num_gpu": 2, "fsdp_size": 2, "trainable": True, "generation_batch_size": 8, "model_arch": arch,
       "kl_coef": 0.001, "optimizer": {"lr": 1e-5}, "packing": True, "max_token_in_packing": 256, "save_hf": True,
       "reshard_after_forward": True,
       "free_gpu_memory": {"offload_weights": True, "offload_optimizer_states": True, "free_grad_buffers": True}},
    "ref_policy": {"num_gpu": 2, "fsdp_size": 2, "generation_batch_size": 8, "model_arch": arch, "packing": True,
       "max_token_in_packing": 256, "free_gpu_memory": {"offload_weights": True}},
    "policy": {"num_gpu": 2, "tensor_model_parallel_size": 2, "generation_batch_size": 16, "model_arch": arch,
       "num_inference_per_prompt": 4, "max_prompt_tokens_length": 64, "max_response_tokens_length": 32,
       "kv_block_size": 8, "num_kv_blocks": 256, "ignore_eos": True},
    "reward": {"num_cpu": 2},
  }}
cfg = to_dataclass(GrpoConfig, resolve(cfg))
algo = GrpoAlgorithm(cfg); algo.validate()
stats = algo.run()
eng = algo.engine
pol, tr = eng.named_models["policy"], eng.named_models["policy_trainer"]
tr.onload()
assert tr.resharded
with tr.state.all_gathered() as whole:
    sd_t = whole.hf_state_dict()
sd_p = pol.model.hf_state_dict()
maxdiff = 0.0
for k, v in sd_p.items():
    nz = v != 0
    maxdiff = max(maxdiff, (v - sd_t[k])[nz].abs().max().item() if nz.any() else 0.0)
hf = os.path.join(out, "save_model", "policy_trainer", str(eng.trainer.iteration), "huggingface")
print("RESULT " + json.dumps({"rank": int(os.environ["RANK"]), "episodes": len(stats), "maxdiff": maxdiff,
      "hf_saved": os.path.isdir(hf) or int(os.environ["RANK"]) != 0}))
'''


def test_grpo_end_to_end_with_sharded_parameters(tmp_path):
    """Rollout (TP=2) pulls its weights from the trainer's parameter slices; offload, checkpoints and the
    HuggingFace export work on the sharded state."""
    outs, _ = run_ranks(E2E, 2, env={"OUT_DIR": str(tmp_path)})
    res = _results(outs)
    assert len(res) == 2
    for r in res:
        assert r["episodes"] == 2 and r["maxdiff"] < 1e-6 and r["hf_saved"], r


HSDP = r'''
import json, os, torch, torch.distributed as dist
from chatlearn_b200.launcher.initialize import init_distributed
from chatlearn_b200.models.nn import PRESETS, CausalLM, packed_ctx
from chatlearn_b200.parallel import build_mesh
from chatlearn_b200.parallel.zero import ShardedTrainState

init_distributed()
rank, world = dist.get_rank(), dist.get_world_size()
mesh = build_mesh(list(range(world)), kinds=("dp", "dp_shard", "dp_rep"), shard=2)
whole, shard, rep = mesh.groups["dp"], mesh.groups["dp_shard"], mesh.groups["dp_rep"]
assert shard.ranks == [rank - rank % 2, rank - rank % 2 + 1] and rep.ranks == [rank % 2, rank % 2 + 2]
dev = torch.device("cpu")
arch = PRESETS["tiny_qwen3"]()
ma = CausalLM(arch, dtype=torch.float32, device=dev, pad_to=world * 8).init_weights(7)
mb = CausalLM(arch, dtype=torch.float32, device=dev, pad_to=world * 8).init_weights(7)
sa = ShardedTrainState(ma, whole, lr=1e-2, clip_grad=1.0)                       # shards over all four ranks
sb = ShardedTrainState(mb, shard, lr=1e-2, clip_grad=1.0, replica_group=rep)    # two shard groups of two
res = {"rank": rank, "norm": [], "shard_fraction": sb.states[0].shard_numel / sb.states[0].block.numel}
for step in range(2):
    sa.zero_grad(); sb.zero_grad()
    torch.manual_seed(100 * step + rank)
    lens = [11 + rank, 23, 6]
    T = sum(lens)
    toks = torch.randint(0, arch.vocab_size - 1, (T,))
    for m in (ma, mb):
        ctx, _ = packed_ctx(lens, dev)
        lp, ent = m.logprobs(toks, toks.roll(-1), ctx)
        (-(lp.sum() + 0.01 * ent.sum()) / T).backward()
    na, nb = sa.step(), sb.step()
    res["norm"].append((float(na), float(nb)))
res["param_diff"] = max((x.flat - y.flat).abs().max().item() for x, y in zip(ma.blocks, mb.blocks))
# every rank of the job holds the same parameters afterwards
ref = [b.flat.clone() for b in mb.blocks]
for t in ref:
    dist.broadcast(t, 0)
res["rank_diff"] = max((x.flat - t).abs().max().item() for x, t in zip(mb.blocks, ref))
print("RESULT " + json.dumps(res))
'''


def test_hybrid_sharding_matches_sharding_over_all_ranks():
    """Four ranks as two shard groups of two (reduce-scatter and all-gather inside a group, all-reduce of the
    gradient shards between the groups) against one shard group of four: same gradient norm, same parameters."""
    outs, _ = run_ranks(HSDP, 4)
    res = _results(outs)
    assert len(res) == 4
    for r in res:
        assert abs(r["shard_fraction"] - 0.5) < 1e-6
        for na, nb in r["norm"]:
            assert abs(na - nb) < 1e-4 * max(1.0, abs(na)), r
        assert r["param_diff"] < 5e-4 and r["rank_diff"] == 0.0, r
