"""Unit tests of the host-side pieces: planner, sampler, config loader, flow tracing, packing,
scheduler, checkpoints and the offline converter."""
import os

import pytest
import torch

from chatlearn_b200.models.nn import PRESETS, CausalLM


# ------------------------------------------------------------------ weight-sync planner
def _run_plan(plan, src_bufs_by_rank, dst_bufs_by_rank):
    for dst, descs in plan.items():
        for d in descs:
            s = src_bufs_by_rank[d.src_rank][d.src_buffer]
            t = dst_bufs_by_rank[dst][d.dst_buffer]
            sv = torch.as_strided(s, (d.rows, d.cols), (d.src_stride, 1), d.src_offset)
            tv = torch.as_strided(t, (d.rows, d.cols), (d.dst_stride, 1), d.dst_offset)
            tv.copy_(sv)


@pytest.mark.parametrize("preset,src_dp,dst_tp,dst_ep", [
    ("tiny_qwen3", 2, 2, 1),       # ZeRO shards -> TP2 (QKV / gate-up re-packing, GQA heads split)
    ("tiny_qwen3", 4, 1, 1),       # shards -> whole
    ("tiny_moe", 2, 1, 2),         # experts re-homed onto EP ranks
    ("tiny_mla_moe", 2, 2, 2),
])
def test_planner_reshards_exactly(preset, src_dp, dst_tp, dst_ep):
    from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
    from chatlearn_b200.synchronizer.plan import build_plan, plan_stats, validate_plan
    arch = PRESETS[preset]()
    full = CausalLM(arch, dtype=torch.float32, pad_to=src_dp).init_weights(11)
    hf = full.hf_state_dict()
    src_lays, src_bufs = [], {}
    for r in range(src_dp):
        shards = {b.name: (r * b.numel // src_dp, (r + 1) * b.numel // src_dp) for b in full.blocks}
        src_lays.append(layout_of_model(full, r, lambda n, s=shards: s[n], "s/"))
        src_bufs[r] = {f"s/{b.name}": b.flat[shards[b.name][0]:shards[b.name][1]].clone() for b in full.blocks}
    dst_lays, dst_models, dst_bufs = [], {}, {}
    rank = 0
    for e in range(dst_ep):
        for t in range(dst_tp):
            m = CausalLM(arch, dtype=torch.float32, tp=dst_tp, tp_rank=t, ep=dst_ep, ep_rank=e)
            dst_lays.append(layout_of_model(m, rank, prefix="d/"))
            dst_models[rank] = m
            dst_bufs[rank] = {f"d/{b.name}": b.flat for b in m.blocks}
            rank += 1
    plan = build_plan(src_lays, dst_lays)
    validate_plan(plan, dst_lays)
    _run_plan(plan, src_bufs, dst_bufs)
    for r, m in dst_models.items():
        want = CausalLM(arch, dtype=torch.float32, tp=m.tp, tp_rank=m.tp_rank, ep=m.ep, ep_rank=m.ep_rank)
        want.load_hf_state_dict(hf)
        for a, b in zip(m.blocks, want.blocks):
            assert torch.equal(a.flat, b.flat), (r, a.name)
    st = plan_stats(plan, 4)
    assert st["descriptors"] > 0


def test_planner_balances_senders_and_prefers_local():
    from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
    from chatlearn_b200.synchronizer.plan import build_plan
    arch = PRESETS["tiny_qwen3"]()
    full = CausalLM(arch, dtype=torch.float32)
    # four data-parallel replicas hold everything; destinations are ranks 0..3 as TP4? no: whole copies
    src = [layout_of_model(full, r, prefix="s/") for r in range(4)]
    dst = [layout_of_model(CausalLM(arch, dtype=torch.float32, device="meta", allocate=False), r, prefix="d/") for r in range(4)]
    plan = build_plan(src, dst)
    assert all(d.src_rank == r for r, ds in plan.items() for d in ds)          # everything local
    dst_far = [layout_of_model(CausalLM(arch, dtype=torch.float32, device="meta", allocate=False), r, prefix="d/") for r in (4, 5, 6, 7)]
    plan = build_plan(src, dst_far)
    sent = {}
    for ds in plan.values():
        for d in ds:
            sent[d.src_rank] = sent.get(d.src_rank, 0) + d.numel
    assert set(sent) == {0, 1, 2, 3} and max(sent.values()) < 1.5 * min(sent.values())


# ------------------------------------------------------------------ sampler
def test_sampler_interleave_rerank_resume_and_mixing():
    from chatlearn_b200.data.sampler import MultiDatasetSampler
    s = MultiDatasetSampler([10], 8, num_inference_per_prompt=2, shuffle=False)
    ep = next(iter(s))
    assert [r for _, r, _ in ep] == [0, 0, 1, 1, 2, 2, 3, 3]
    s = MultiDatasetSampler([10], 8, num_inference_per_prompt=2, shuffle=False, data_rerank=True)
    assert [r for _, r, _ in next(iter(s))] == [0, 1, 2, 3, 0, 1, 2, 3]
    # two replicas split an episode; resuming from consumed_samples continues the stream
    a = MultiDatasetSampler([10], 8, num_inference_per_prompt=2, shuffle=True, seed=3, data_parallel_rank=0, data_parallel_size=2)
    b = MultiDatasetSampler([10], 8, num_inference_per_prompt=2, shuffle=True, seed=3, data_parallel_rank=1, data_parallel_size=2)
    ia, ib = iter(a), iter(b)
    e0, e1 = next(ia) + next(ib), next(ia) + next(ib)
    assert len(e0) == 8 and len({r for _, r, _ in e0}) == 4
    c = MultiDatasetSampler([10], 8, consumed_samples=8, num_inference_per_prompt=2, shuffle=True, seed=3)
    assert [r for _, r, _ in next(iter(c))] == [r for _, r, _ in e1]
    # ratio 2:1 mixing of two datasets
    m = MultiDatasetSampler([100, 100], 12, data_ratio=[2, 1], num_inference_per_prompt=1, shuffle=False)
    ds = [d for d, _, _ in next(iter(m))]
    assert ds == [0, 0, 1] * 4
    ev = MultiDatasetSampler([3, 2], 4, is_eval=True, data_parallel_rank=1, data_parallel_size=2)
    assert len(next(iter(ev))) in (2, 3)


# ------------------------------------------------------------------ config loader
def test_config_interpolation_dotlist_and_errors(tmp_path, monkeypatch):
    from chatlearn_b200.configs.conf import ConfigError, apply_dotlist, load_yaml, resolve, to_dataclass
    from chatlearn_b200.configs import PolicyConfig
    p = tmp_path / "c.yaml"
    p.write_text("a:\n  x: 2e-6\n  y: ${a.x}\n  z: ${oc.env:MY_VAR,7}\nb: ${a.y}\nlst: [1, 2]\n")
    monkeypatch.setenv("MY_VAR", "11")
    cfg = resolve(apply_dotlist(load_yaml(str(p)), ["a.w=hello", "lst=[3,4,5]", "c.d.e=true"]))
    assert cfg["a"]["x"] == 2e-6 and cfg["b"] == 2e-6 and cfg["a"]["z"] in (11, "11")
    assert cfg["a"]["w"] == "hello" and cfg["lst"] == [3, 4, 5] and cfg["c"]["d"]["e"] is True
    pol = to_dataclass(PolicyConfig, {"num_gpu": 4, "tensor_model_parallel_size": 2, "vllm_extra": 1, "temperature": "0.5"})
    assert pol.num_replica == 2 and pol.vllm_extra == 1 and pol.temperature == 0.5
    with pytest.raises(ConfigError):
        to_dataclass(PolicyConfig, {"nope": 1}, strict=True)


# ------------------------------------------------------------------ flow tracing
class _M:
    def __init__(self, name):
        self.name = name
        self.call_funcs = []

    def forward_step(self, *a, **k):
        raise AssertionError("real method must not run while tracing")

    train_step = eval_forward = forward_step


def test_model_flow_levels_fanout_and_repeat():
    from chatlearn_b200.runtime.model_flow import ModelFlow
    p, r, v, w = _M("policy"), _M("ref"), _M("value"), _M("reward")

    def flow(batch):
        a = p.forward_step(batch)
        b = r.forward_step(a)
        c = v.forward_step(a)
        d = w.forward_step(a, b, c)
        e = p.forward_step(d)            # the same model twice
        return c, e

    mf = ModelFlow([p, r, v, w])
    mf.trace(flow)
    levels = [[(n.model.name, n.func_name) for n in lvl] for lvl in mf.flow_topology]
    assert levels[0] == [("policy", "forward_step")]
    assert sorted(levels[1]) == [("ref", "forward_step"), ("value", "forward_step")]
    assert levels[2] == [("reward", "forward_step")] and levels[3] == [("policy", "forward_step")]
    assert [n.model.name for n in mf.return_nodes] == ["value", "policy"]
    assert len(mf.model_nodes) == 5


# ------------------------------------------------------------------ packing
def test_bin_packing_limits_and_balance():
    from chatlearn_b200.algorithm.grpo_utils.packing_utils import bin_packing, bin_packing_fix_bin, regroup_data_packing
    lens = [900, 800, 300, 250, 200, 100, 60, 50]
    ids, ls = bin_packing(lens, 1024)
    assert sorted(i for b in ids for i in b) == list(range(8))
    assert all(sum(x) <= 1024 for x in ls)
    ids, ls = bin_packing_fix_bin(lens, 3)
    loads = [sum(x) for x in ls]
    assert len(ids) == 3 and max(loads) - min(loads) <= 300
    data = [{"prompt_token_length": n // 2, "response_token_length": n - n // 2} for n in lens]
    mbs = regroup_data_packing(data, lambda n: n + 1, 1024)      # a peer needs one more bin: so do we
    assert len(mbs) == len(bin_packing(lens, 1024)[0]) + 1
    assert sorted(s["id_in_list"] for mb in mbs for s in mb) == list(range(8))


def test_pack_samples_alignment_and_masks():
    from chatlearn_b200.algorithm.grpo_utils.trainer_utils import pack_samples, unpack_per_sample
    s = [{"all_tokens": torch.arange(10), "prompt_token_length": 4, "response_token_length": 6, "advantages": 0.5,
          "old_logprobs": torch.arange(6).float()},
         {"all_tokens": torch.arange(7), "prompt_token_length": 5, "response_token_length": 2, "advantages": -1.0,
          "old_logprobs": torch.arange(2).float(), "loss_mask": torch.tensor([0, 0, 0, 0, 0, 1, 0])}]
    b = pack_samples(s, pad_multiple=4, seq_multiple=4)
    assert b.tokens.numel() % 4 == 0 and b.seq_lens[:2] == [12, 8]
    assert b.loss_mask[:12].tolist() == [0, 0, 0, 1, 1, 1, 1, 1, 1, 0, 0, 0]      # labels of response tokens
    assert b.loss_mask[12:20].sum() == 1 and b.loss_mask[12 + 4] == 1              # explicit mask, shifted to labels
    assert b.old_logprobs[3:9].tolist() == [0, 1, 2, 3, 4, 5]
    per = unpack_per_sample(torch.arange(b.tokens.numel()).float(), b, s)
    # one value per label position of the unpadded sequence (length n - 1)
    assert per[0].numel() == 9 and per[1].numel() == 6 and per[0][3] == 3 and per[1][0] == 12


# ------------------------------------------------------------------ rollout scheduler
def test_scheduler_preempts_and_recomputes_without_losing_tokens():
    from chatlearn_b200.rollout.scheduler import Scheduler, Sequence
    sch = Scheduler(num_blocks=6, block_size=4, max_num_seqs=4, max_num_batched_tokens=64)
    seqs = [Sequence(i, list(range(6)), 10) for i in range(3)]
    for q in seqs:
        sch.add(q)
    steps = 0
    while sch.has_work() and steps < 500:
        plan = sch.schedule()
        if plan is None:
            break
        for q, n, smp in zip(plan.seqs, plan.q_lens, plan.samples):
            q.num_computed += n
            if smp:
                q.output.append(7)
                if len(q.output) >= q.max_new_tokens:
                    sch.finish(q, "length")
        steps += 1
    assert all(q.finished and len(q.output) == 10 for q in seqs)
    assert sch.stats["preemptions"] > 0 and sch.alloc.num_free == 6


# ------------------------------------------------------------------ checkpoints
def test_safetensors_roundtrip_sharded_and_tp_load(tmp_path):
    from chatlearn_b200.checkpoint.safetensors_io import SafetensorsDir, load_into_model, save_hf_checkpoint
    arch = PRESETS["tiny_qwen3"]()
    m = CausalLM(arch, dtype=torch.float32).init_weights(4)
    save_hf_checkpoint(m, str(tmp_path), dtype=torch.float32, max_shard_bytes=200_000)
    assert os.path.exists(tmp_path / "model.safetensors.index.json") and os.path.exists(tmp_path / "config.json")
    d = SafetensorsDir(str(tmp_path))
    sd = m.hf_state_dict()
    assert set(d.keys()) == set(sd)
    k = "model.layers.1.self_attn.q_proj.weight"
    assert torch.equal(d.get(k)[3:9], sd[k][3:9]) and d.get("missing") is None
    for r in range(2):
        part = CausalLM(arch, dtype=torch.float32, tp=2, tp_rank=r)
        load_into_model(part, str(tmp_path))
        want = CausalLM(arch, dtype=torch.float32, tp=2, tp_rank=r)
        want.load_hf_state_dict(sd)
        assert all(torch.equal(a.flat, b.flat) for a, b in zip(part.blocks, want.blocks))


def test_scheduler_never_mixes_fresh_prompts_with_continuation_chunks():
    from chatlearn_b200.rollout.scheduler import Scheduler, Sequence
    sch = Scheduler(num_blocks=64, block_size=4, max_num_seqs=8, max_num_batched_tokens=16)
    seqs = [Sequence(0, list(range(40)), 3), Sequence(1, list(range(10)), 3), Sequence(2, list(range(12)), 3)]
    for q in seqs:
        sch.add(q)
    for _ in range(200):
        if not sch.has_work():
            break
        plan = sch.schedule()
        starts = [q.num_computed for q in plan.seqs]
        prefilling = [n > 1 for n in plan.q_lens]
        if any(prefilling):
            # all at position 0 (packed attention) or all continuations (paged attention)
            assert all(s == 0 for s in starts) or all(s > 0 for s in starts)
            assert plan.is_prefill == all(s == 0 for s in starts)
        for q, n, smp in zip(plan.seqs, plan.q_lens, plan.samples):
            q.num_computed += n
            if smp:
                q.output.append(1)
                if len(q.output) >= q.max_new_tokens:
                    sch.finish(q, "length")
    assert all(q.finished for q in seqs)


def test_planner_gathers_expert_tensor_parallel_slices():
    """Trainer ranks with tensor- and expert-tensor-parallel slices (tp = etp = 2, experts on two ep ranks each)
    feed a rollout model whose experts are whole and spread over two ep ranks."""
    from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
    from chatlearn_b200.synchronizer.plan import build_plan, validate_plan
    arch = PRESETS["tiny_moe"]()
    full = CausalLM(arch, dtype=torch.float32).init_weights(11)
    hf = full.hf_state_dict()
    src_lays, src_bufs, rank = [], {}, 0
    for e in range(2):
        for t in range(2):
            m = CausalLM(arch, dtype=torch.float32, tp=2, tp_rank=t, ep=2, ep_rank=e, etp=2, etp_rank=t)
            m.load_hf_state_dict(hf)
            assert m.block_by_name["layer0.experts"].params["w13"].shape == (4, arch.moe_intermediate_size, arch.hidden_size)
            src_lays.append(layout_of_model(m, rank, prefix="s/"))
            src_bufs[rank] = {f"s/{b.name}": b.flat for b in m.blocks}
            rank += 1
    dst_lays, dst_models, dst_bufs = [], {}, {}
    for e in range(2):
        m = CausalLM(arch, dtype=torch.float32, ep=2, ep_rank=e)
        dst_lays.append(layout_of_model(m, e, prefix="d/"))
        dst_models[e], dst_bufs[e] = m, {f"d/{b.name}": b.flat for b in m.blocks}
    plan = build_plan(src_lays, dst_lays)
    validate_plan(plan, dst_lays)
    _run_plan(plan, src_bufs, dst_bufs)
    for e, m in dst_models.items():
        want = CausalLM(arch, dtype=torch.float32, ep=2, ep_rank=e)
        want.load_hf_state_dict(hf)
        for a, b in zip(m.blocks, want.blocks):
            assert torch.equal(a.flat, b.flat), (e, a.name)


def test_batched_paged_decode_matches_the_per_sequence_statements():
    """The host-synchronisation-free decode attention (used for head sizes without a kernel instance, inside
    captured steps) against the per-sequence reference, grouped-query heads and ragged lengths."""
    from chatlearn_b200.ops import reference as ref
    from chatlearn_b200.ops.paged_fallback import paged_decode_batched
    torch.manual_seed(0)
    nb, bs, nkv, d, nq = 24, 8, 2, 48, 8
    kc, vc = torch.randn(nb, bs, nkv, d), torch.randn(nb, bs, nkv, d)
    bt = torch.tensor([[3, 5, 0, 0], [1, 2, 4, 7], [9, 0, 0, 0], [11, 12, 13, 0]], dtype=torch.int32)
    sl = torch.tensor([11, 32, 1, 17], dtype=torch.int32)
    q = torch.randn(4, nq, d)
    want = ref.paged_attention(q, kc, vc, bt, sl, None, 0.2)
    got = paged_decode_batched(q, kc, vc, bt, sl, 0.2)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)


def test_latent_attention_matches_expanded_heads():
    """Latent-space attention over compressed rows equals ordinary attention over the per-head keys and values
    obtained by up-projecting those rows (decode rows and a multi-token tail)."""
    from chatlearn_b200.models.nn.mla import latent_paged_attention
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(1)
    nb, bs, lora, rp, nh, nope, dv = 12, 4, 16, 8, 3, 10, 6
    cache = torch.randn(nb, bs, 1, lora + rp)
    w_uk, w_uv = torch.randn(nh, nope, lora), torch.randn(nh, dv, lora)
    bt = torch.tensor([[2, 4, 6], [1, 3, 0]], dtype=torch.int32)
    sl = torch.tensor([10, 5], dtype=torch.int32)
    # expanded cache: k = [W_uk c | rope part], v = W_uv c for every head
    c, kr = cache[..., 0, :lora], cache[..., 0, lora:]
    k_full = torch.cat([torch.einsum("hnc,bsc->bshn", w_uk, c), kr[:, :, None].expand(nb, bs, nh, rp)], -1)
    v_full = torch.einsum("hvc,bsc->bshv", w_uv, c)
    for q_lens in (None, torch.tensor([3, 2], dtype=torch.int32)):
        T = 2 if q_lens is None else int(q_lens.sum())
        q_nope, q_rope = torch.randn(T, nh, nope), torch.randn(T, nh, rp)
        want = ref.paged_attention(torch.cat([q_nope, q_rope], -1), k_full, v_full, bt, sl, q_lens, 0.3)
        q_lat = torch.cat([torch.einsum("thn,hnc->thc", q_nope, w_uk), q_rope], -1)
        o_lat = latent_paged_attention(q_lat, cache, lora, bt, sl, q_lens, 1 if q_lens is None else 3, 0.3)
        got = torch.einsum("thc,hvc->thv", o_lat, w_uv)
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), float((got - want).abs().max())


def test_gather_payloads_two_planes():
    """Tensors of a payload travel as flat per-dtype buffers, the rest is pickled; every rank gets every payload."""
    from tests.dist_utils import run_ranks
    script = r'''
import json, torch, torch.distributed as dist
from chatlearn_b200.launcher.initialize import init_distributed
from chatlearn_b200.runtime.executor import gather_payloads
init_distributed()
r = dist.get_rank()
payload = None if r == 2 else (r, [{"uid": f"p{r}-{i}", "all_tokens": torch.arange(20 + r + i), "n": i,
                                    "lp": torch.full((17 + i,), float(r)), "tiny": torch.tensor([r])} for i in range(3)], False)
out = gather_payloads(payload)
ok = out[2] is None and len(out) == 3
for q in (0, 1):
    rr, lst, flag = out[q]
    ok &= rr == q and flag is False and len(lst) == 3
    for i, s in enumerate(lst):
        ok &= s["uid"] == f"p{q}-{i}" and s["n"] == i and torch.equal(s["all_tokens"], torch.arange(20 + q + i))
        ok &= s["lp"].dtype == torch.float32 and torch.equal(s["lp"], torch.full((17 + i,), float(q))) and int(s["tiny"]) == q
print("RESULT " + json.dumps({"ok": bool(ok)}))
'''
    outs, _ = run_ranks(script, 3)
    import json as _json
    res = [_json.loads(l[7:]) for o in outs for l in o.splitlines() if l.startswith("RESULT ")]
    assert len(res) == 3 and all(r["ok"] for r in res)


def _drive(sch, seqs, token=7, max_steps=2000):
    for q in seqs:
        sch.add(q)
    steps = 0
    while sch.has_work() and steps < max_steps:
        plan = sch.schedule()
        if plan is None:
            break
        for q, n, smp in zip(plan.seqs, plan.q_lens, plan.samples):
            q.num_computed += n
            if smp:
                q.output.append(token)
                if len(q.output) >= q.max_new_tokens:
                    sch.finish(q, "length")
        steps += 1
    return steps


def test_scheduler_shares_the_prompt_blocks_of_a_group():
    """Eight samples of one prompt: one of them computes the prompt, the others adopt its full blocks by reference,
    compute only the tail, and the pool is whole again at the end."""
    from chatlearn_b200.rollout.scheduler import Scheduler, Sequence
    bs = 4
    prompts = [list(range(100, 100 + 22)), list(range(300, 300 + 9))]       # 5 and 2 full blocks
    sch = Scheduler(num_blocks=200, block_size=bs, max_num_seqs=32, max_num_batched_tokens=64)
    seqs = [Sequence(i, list(prompts[i // 8]), 6) for i in range(16)]
    for q in seqs:
        sch.add(q)
    plan = sch.schedule()                                # the two owners start at position 0; everybody else waits
    assert plan.is_prefill and [q.req_id for q in plan.seqs] == [0, 8]
    for q, n in zip(plan.seqs, plan.q_lens):
        q.num_computed += n
        q.output.append(7)
    plan = sch.schedule()                                # the adopters: continuation chunks over shared blocks
    # (the second group's adopters have a single prompt token left: they join the running set and take it in
    # the next decode step)
    assert not plan.is_prefill and sorted(q.req_id for q in plan.seqs) == list(range(1, 8))
    adopters = [q for q in seqs if q.req_id not in (0, 8)]
    assert all(q in sch.running for q in adopters)
    for q in adopters:
        owner = seqs[0] if q.req_id < 8 else seqs[8]
        n_shared = (len(q.prompt) - 1) // bs
        assert q.blocks[:n_shared] == owner.blocks[:n_shared] and q.num_computed == n_shared * bs
        assert not set(q.blocks[n_shared:]) & set(owner.blocks)
    assert sch.stats["shared_prefix_tokens"] == 7 * 5 * bs + 7 * 2 * bs
    used_with_sharing = sch.alloc.num_blocks - sch.alloc.num_free
    for q, n, smp in zip(plan.seqs, plan.q_lens, plan.samples):
        q.num_computed += n
        if smp:
            q.output.append(7)
    _drive(sch, [])
    assert all(q.finished and len(q.output) == 6 for q in seqs) and sch.alloc.num_free == 200 and not sch._prefix
    # sixteen private copies of the prompts would hold 8 * 6 + 8 * 3 = 72 blocks at this point
    assert used_with_sharing <= 6 + 7 + 3 + 7


def test_prefix_sharing_survives_preemption_of_the_owner():
    """A small pool: owners and adopters are preempted and recomputed; nothing is lost, no block leaks, and a block
    whose owner was preempted before finishing it is never adopted."""
    from chatlearn_b200.rollout.scheduler import Scheduler, Sequence
    sch = Scheduler(num_blocks=14, block_size=4, max_num_seqs=8, max_num_batched_tokens=24)
    seqs = [Sequence(i, list(range(50, 50 + 13)), 12) for i in range(6)]
    steps = _drive(sch, seqs)
    assert steps < 2000 and all(q.finished and len(q.output) == 12 for q in seqs)
    assert sch.stats["preemptions"] > 0 and sch.alloc.num_free == 14 and not sch._prefix and not sch._block_key
    assert all(r == 0 for r in sch.alloc._ref)


def test_engine_generates_the_same_tokens_with_and_without_prefix_sharing(monkeypatch):
    from chatlearn_b200.rollout import RolloutEngine, SamplingParams
    arch = PRESETS["tiny_qwen3"]()
    model = CausalLM(arch, dtype=torch.float32).init_weights(2)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, arch.vocab_size - 1, (n,), generator=g).tolist() for n in (37, 16, 9)]
    batch = [p for p in prompts for _ in range(4)] + [prompts[0][:20] + [3, 4, 5]]     # groups, plus a partial overlap
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("CLB200_PREFIX_SHARING", flag)
        eng = RolloutEngine(model, block_size=8, num_blocks=128, max_num_seqs=16, max_model_len=128)
        res = eng.generate(batch, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
        outs[flag] = [s.output for s in res]
        shared = eng.stats.get("shared_prefix_tokens", 0)
        assert (shared > 0) == (flag == "1")
    assert outs["1"] == outs["0"]
    assert all(outs["1"][i] == outs["1"][i - i % 4] for i in range(12))         # greedy: a group's samples agree


def test_resource_manager_bundles(monkeypatch):
    """Placement groups over ranks: a role that fits a node is packed on one node, a larger one takes whole nodes,
    nothing is handed out twice, and removed groups return their ranks."""
    from chatlearn_b200.schedule.resource_manager import ResourceManager
    monkeypatch.setenv("GPUS_PER_NODE", "4")
    rm = ResourceManager()
    rm.world_size, rm.total_gpu = 12, 12
    rm.nnode = 3
    from chatlearn_b200.schedule.resource_manager import NodeInfo
    rm._nodes = [NodeInfo(i, f"host{i}", list(range(4 * i, 4 * i + 4)), cpus=32, free=list(range(4 * i, 4 * i + 4)))
                 for i in range(3)]
    a = rm.create_placement_group(2, name="reward")
    assert a.ranks == [0, 1] and a.bundle_specs == [{"GPU": 2, "CPU": 16}]
    b = rm.create_placement_group(2, name="ref")                           # PACK: fills node 0 before opening node 1
    assert b.ranks == [2, 3]
    c = rm.create_placement_group(8, name="policy")                        # larger than a node: whole nodes
    assert c.ranks == list(range(4, 12)) and [x["GPU"] for x in c.bundle_specs] == [4, 4]
    with pytest.raises(RuntimeError):
        rm.create_placement_group(1)
    d = rm.create_placement_group(0, num_cpus=[4, 4], name="managers")
    assert d.ranks == [] and d.bundle_specs == [{"GPU": 0, "CPU": 4}, {"GPU": 0, "CPU": 4}]
    assert rm.model_to_placegroup["policy"] is c and rm.get_placement_group_state(c) == "CREATED"
    rm.remove_placement_groups()
    assert all(len(n.free) == 4 for n in rm._nodes) and c.state == "REMOVED"
    s1 = rm.create_placement_group(1, strategy="SPREAD")
    s2 = rm.create_placement_group(1, strategy="SPREAD")
    assert rm.node_of(s1.ranks[0]) != rm.node_of(s2.ranks[0])
    e = rm.reserve("colocated", [5, 6, 9])
    assert [x.node for x in e.bundles] == [1, 2] and 5 not in rm._nodes[1].free


def _tiny_engine(**kw):
    from chatlearn_b200.rollout import RolloutEngine
    arch = PRESETS["tiny_qwen3"]()
    model = CausalLM(arch, dtype=torch.float32).init_weights(2)
    return arch, RolloutEngine(model, block_size=8, num_blocks=128, max_num_seqs=16, max_model_len=128, **kw)


def test_session_requests_join_and_leave_a_running_batch():
    """A request submitted while others decode joins at the next step, finishes on its own schedule, and gets the
    tokens it would get alone (greedy)."""
    from chatlearn_b200.rollout import SamplingParams
    arch, eng = _tiny_engine()
    g = torch.Generator().manual_seed(11)
    pa, pb = (torch.randint(0, arch.vocab_size - 1, (n,), generator=g).tolist() for n in (21, 13))
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    alone = [s.output for s in eng.generate([pa, pb], [sp, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)])]

    sess = eng.open_session()
    a = sess.submit(pa, sp)
    order, steps, b = [], 0, None
    while True:
        done = sess.poll()
        if done is None:
            break
        steps += 1
        order += [s.req_id for s in done]
        if steps == 4:                                # a is in the middle of its decode
            assert not a.finished and len(a.output) == 4
            b = sess.submit(pb, sp, max_new_tokens=5)
    sess.close()
    assert order == [b.req_id, a.req_id]              # the late, short request leaves first
    assert [a.output, b.output] == alone
    assert sess.poll() is None
    z = sess.submit(pa, sp, max_new_tokens=0)         # no budget: handed back at the next poll, no engine step
    assert z.finished and sess.poll() == [z] and sess.poll() is None


def test_async_rollout_resolves_each_request_when_it_finishes():
    import asyncio
    from chatlearn_b200.rollout import SamplingParams
    from chatlearn_b200.rollout.engine import AsyncRollout
    arch, eng = _tiny_engine()
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, arch.vocab_size - 1, (n,), generator=g).tolist() for n in (9, 17, 12)]
    budgets = [10, 3, 6]
    finished = []

    async def trajectory(ar, i):
        # two turns: the second prompt is the first plus its answer
        sp = SamplingParams(temperature=0.0, max_tokens=budgets[i], ignore_eos=True)
        first = await ar.generate(prompts[i], sp)
        finished.append((i, 1))
        second = await ar.generate(prompts[i] + first.output, sp, max_new_tokens=2)
        finished.append((i, 2))
        return first.output + second.output

    async def main():
        ar = AsyncRollout(eng)
        outs = await asyncio.gather(*(trajectory(ar, i) for i in range(3)))
        ar.close()
        return outs

    outs = asyncio.run(main())
    assert [len(o) for o in outs] == [12, 5, 8]
    # the short trajectory ran both of its turns before the long one finished its first
    assert finished.index((1, 2)) < finished.index((0, 1))
    # greedy: a two-turn trajectory equals one uninterrupted generation of the same length
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    whole = eng.generate([prompts[0]], sp)[0].output
    assert outs[0] == whole


def test_budgeted_iterations_cover_the_plan_within_bucket_and_memory_limits():
    """The remote pieces of a plan, cut into row bands and scheduled into iterations: every element is moved exactly
    once, no message exceeds the bucket, no rank stages more than its budget in one iteration, and executing the
    iterations one after the other gives the same result as the whole plan at once."""
    from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
    from chatlearn_b200.synchronizer.plan import build_iterations, build_plan, iteration_stats
    arch = PRESETS["tiny_moe"]()
    src_dp, dst_tp = 2, 2
    full = CausalLM(arch, dtype=torch.float32, pad_to=src_dp).init_weights(11)
    src_lays, src_bufs = [], {}
    for r in range(src_dp):
        shards = {b.name: (r * b.numel // src_dp, (r + 1) * b.numel // src_dp) for b in full.blocks}
        src_lays.append(layout_of_model(full, r, lambda n, s=shards: s[n], "s/"))
        src_bufs[r] = {f"s/{b.name}": b.flat[shards[b.name][0]:shards[b.name][1]].clone() for b in full.blocks}
    dst_lays, dst_bufs, ref_bufs = [], {}, {}
    for t in range(dst_tp):
        m = CausalLM(arch, dtype=torch.float32, tp=dst_tp, tp_rank=t)
        dst_lays.append(layout_of_model(m, t, prefix="d/"))
        dst_bufs[t] = {f"d/{b.name}": b.flat for b in m.blocks}
        ref_bufs[t] = {k: torch.zeros_like(v) for k, v in dst_bufs[t].items()}
    plan = build_plan(src_lays, dst_lays)
    _run_plan(plan, src_bufs, ref_bufs)
    remote = sum(d.numel for ds in plan.values() for d in ds if d.src_rank != d.dst_rank)
    assert remote > 0
    bucket, budget = 4096, {0: 24 * 1024, 1: 24 * 1024}
    iters = build_iterations(plan, 4, bucket, budget)
    assert iters == build_iterations(plan, 4, bucket, budget)                 # every rank derives the same schedule
    assert len(iters) > 1
    moved = 0
    for it in iters:
        staged = {}
        for (s, d), ds in it.items():
            nb = sum(x.numel for x in ds) * 4
            assert nb <= bucket or len(ds) == 1
            staged[s] = staged.get(s, 0) + nb
            staged[d] = staged.get(d, 0) + nb
            moved += sum(x.numel for x in ds)
        assert all(v <= budget[r] for r, v in staged.items())
    assert moved == remote
    st = iteration_stats(iters, 4)
    assert st["iterations"] == len(iters) and st["peak_staged_mb"] <= 24 / 1024 + 1e-9
    # local pieces + the iterations, one after the other, reproduce the one-shot result
    local = {dst: [d for d in ds if d.src_rank == dst] for dst, ds in plan.items()}
    _run_plan(local, src_bufs, dst_bufs)
    for it in iters:
        by_dst = {}
        for (s, d), ds in it.items():
            by_dst.setdefault(d, []).extend(ds)
        _run_plan(by_dst, src_bufs, dst_bufs)
    for r in dst_bufs:
        for k in dst_bufs[r]:
            assert torch.equal(dst_bufs[r][k], ref_bufs[r][k]), (r, k)
    # a piece that cannot fit a rank's budget is reported, not silently staged
    import pytest as _pt
    with _pt.raises(RuntimeError):
        build_iterations(plan, 4, 1 << 30, {0: 16, 1: 16})


def test_interleaved_pipeline_time_table():
    """Every stage runs each (micro-batch, chunk) forward and backward once, inputs exist before they are used, and
    the interleaved table is shorter than plain one-forward-one-backward with the same number of layers per stage."""
    from chatlearn_b200.algorithm.grpo_utils.megatron_policy_trainer import MegatronPolicyTrainer as T
    for P, V, m in [(2, 2, 4), (4, 2, 8), (2, 3, 5), (4, 2, 3), (2, 2, 1), (3, 2, 6)]:
        ticks = T.interleaved_ticks(P, V, m)
        G = P * V
        when = {}
        for r in range(P):
            assert len(ticks[r]) == len(ticks[0])
            units = [u for u in ticks[r] if u is not None]
            assert sorted(units) == sorted([(k, i, j) for k in "FB" for i in range(m) for j in range(V)])
            for t, u in enumerate(ticks[r]):
                if u is not None:
                    when[(u[0], u[1], u[2] * P + r)] = t
        for (kind, mb, g), t in when.items():
            if kind == "F" and g > 0:
                assert when[("F", mb, g - 1)] < t
            if kind == "B":
                assert when[("F", mb, g)] < t and (g == G - 1 or when[("B", mb, g + 1)] < t)
        if m % P == 0 and m >= 2 * P:
            # plain 1F1B: (m + P - 1) slots of V chunk-units each, forward and backward
            assert len(ticks[0]) < 2 * V * (m + P - 1)


def test_scheduler_counts_tokens_in_flight():
    """A token sampled on the device but not read back yet (pipelined decode) counts for block allocation and for
    the 'prompt KV still missing' test: the decode step after it may need a fresh block."""
    from chatlearn_b200.rollout.scheduler import Scheduler, Sequence
    sched = Scheduler(num_blocks=8, block_size=4, max_num_seqs=4, max_num_batched_tokens=64, prefix_sharing=False)
    s = Sequence(0, [1, 2, 3], 16)                      # 3 prompt tokens: one block
    sched.add(s)
    plan = sched.schedule()                             # prefill
    assert plan.is_prefill and plan.q_lens == [3] and len(s.blocks) == 1
    s.num_computed = 3
    s.output.append(7)                                  # first sampled token, known to the host: length 4
    plan = sched.schedule()                             # decode: feeds token 7 at position 3 -> still block 0
    assert plan.q_lens == [1] and len(s.blocks) == 1
    s.num_computed = 4
    s.inflight = 1                                      # its sample is on the device; the host still sees length 4
    plan = sched.schedule()                             # the next step writes position 4: a second block is needed
    assert plan.q_lens == [1] and not plan.is_prefill and len(s.blocks) == 2
    s.num_computed = 5
    s.output.append(9)                                  # the read-back of the first in-flight token arrives
    plan = sched.schedule()                             # length 5 + 1 in flight = 6 tokens: still two blocks
    assert plan.q_lens == [1] and len(s.blocks) == 2
    s.inflight = 0
    s.output.append(11)
    sched.finish(s, "length")
    assert sched.alloc.num_free == 8 and not sched.has_work()


def test_pipelined_decode_host_logic_on_cpu(monkeypatch):
    """The host side of the captured, pipelined decode step (persistent input buffers, cached block tables, input
    tokens taken from the previous step's samples, tokens read back one step late) with the step's body run
    directly: stop tokens seen one step late, length limits known in advance, a request that joins late and a KV
    pool that forces preemptions must give exactly the generations of the plain step-by-step engine."""
    from chatlearn_b200.rollout import RolloutEngine, SamplingParams
    arch = PRESETS["tiny_qwen3"]()
    model = CausalLM(arch, dtype=torch.float32).init_weights(2)
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, arch.vocab_size - 1, (n,), generator=g).tolist() for n in (30, 11, 41, 8, 17, 5)]
    budgets = [24, 3, 17, 1, 20, 24]
    free = RolloutEngine(model, block_size=8, num_blocks=64, max_num_seqs=8, max_model_len=96, use_cuda_graphs=False) \
        .generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True), max_new_tokens=budgets)
    stops = (free[0].output[9], free[5].output[15])
    sp = SamplingParams(temperature=0.0, max_tokens=24, stop_token_ids=stops)
    res, pre = {}, {}
    for name, graphs, pipe in (("pipelined", "emulate", "1"), ("buffers", "emulate", "0"), ("plain", False, "0")):
        monkeypatch.setenv("CLB200_PIPELINED_DECODE", pipe)
        # the six sequences would need 28 blocks at their longest; 13 force preemptions
        eng = RolloutEngine(model, block_size=8, num_blocks=13, max_num_seqs=8, max_model_len=96, use_cuda_graphs=graphs)
        assert eng.pipelined == (pipe == "1")
        sess = eng.open_session(eos_id=-1)
        seqs = [sess.submit(p, sp, b) for p, b in zip(prompts[:5], budgets[:5])]
        steps, order = 0, []
        while True:
            done = sess.poll()
            if done is None:
                break
            steps += 1
            order += [s.req_id - seqs[0].req_id for s in done]
            if steps == 5:
                seqs.append(sess.submit(prompts[5], sp, budgets[5]))
        sess.close()
        assert sorted(order) == list(range(6)) and all(s.finished and not s.inflight for s in seqs), name
        res[name] = [(s.output, s.finish_reason) for s in seqs]
        pre[name] = eng.stats["preemptions"]
    assert res["pipelined"] == res["plain"] and res["buffers"] == res["plain"]
    assert pre["plain"] > 0 and pre["pipelined"] > 0
    assert res["plain"][0][1] == "stop" and res["plain"][1] == (free[1].output[:3], "length") and len(res["plain"][3][0]) == 1


def test_model_chunks_of_uneven_pipeline_stages():
    from chatlearn_b200.models.megatron_module import pipeline_chunk_ranges, pipeline_layer_range, pipeline_stage_sizes
    assert pipeline_stage_sizes(10, 4, first=1, last=1) == [1, 4, 4, 1]
    assert pipeline_layer_range(10, 4, 2, first=1, last=1) == (5, 9)
    assert [pipeline_chunk_ranges(8, 2, 2, s) for s in range(2)] == [[(0, 2), (4, 6)], [(2, 4), (6, 8)]]
    # 16 layers, 4 stages of (2, 6, 6, 2) layers, two chunks each: a round is 1 + 3 + 3 + 1 layers
    got = [pipeline_chunk_ranges(16, 4, 2, s, first=2, last=2) for s in range(4)]
    assert got == [[(0, 1), (8, 9)], [(1, 4), (9, 12)], [(4, 7), (12, 15)], [(7, 8), (15, 16)]]
    covered = sorted(l for st in got for lo, hi in st for l in range(lo, hi))
    assert covered == list(range(16))
    with pytest.raises(AssertionError):
        pipeline_chunk_ranges(10, 4, 2, 0, first=1, last=1)
