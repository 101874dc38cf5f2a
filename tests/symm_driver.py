"""Two-GPU checks of the in-kernel collectives (run under torchrun, one rank per GPU)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from chatlearn_b200.launcher.initialize import init_distributed  # noqa: E402
from chatlearn_b200.ops import reference as ref  # noqa: E402
from chatlearn_b200.parallel import symm_collectives  # noqa: E402
from chatlearn_b200.parallel.groups import Group  # noqa: E402

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
init_distributed()
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
g = Group(dist.group.WORLD, list(range(world)), "world")
sg = symm_collectives.get(g)
assert sg is not None
res = {}

# ---- one-shot all-reduce vs NCCL, several sizes, repeated (counters advance) ----
torch.manual_seed(100 + rank)
ok = True
for n in (8, 4096 * 128, 4096 * 256 + 24, 1 << 21):
    for rep in range(3):
        x = torch.randn(n, device=dev).bfloat16()
        want = x.float().clone()
        dist.all_reduce(want)
        got = sg.all_reduce(x.clone())
        ok &= bool(torch.allclose(got.float(), want, rtol=2e-2, atol=2e-2))
res["allreduce_ok"] = ok

# timing: 256 x 4096 bf16 (decode all-reduce)
x = torch.randn(256 * 4096, device=dev).bfloat16()
for fn_name, fn in (("symm", lambda: sg.all_reduce(x)), ("nccl", lambda: dist.all_reduce(x))):
    for _ in range(5):
        fn()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(50):
        fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 50], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res[f"allreduce_{fn_name}_us"] = round(t.item() * 1e3, 2)

# ---- fused all-reduce + residual + RMSNorm on GEMM partials, eager and graph-replayed ----
H, ok = 4096, True
w_norm = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
dist.broadcast(w_norm, 0)
wmat = (0.02 * torch.randn(H, 1024, device=dev)).bfloat16()        # this rank's slice of a row-parallel weight
for T in (1, 128, 333):
    xin = torch.randn(T, 1024, device=dev).bfloat16()
    resid = torch.randn(T, H, device=dev).bfloat16()
    dist.broadcast(resid, 0)
    for use_norm in (True, False, True, False):                    # even count keeps the buffer alternation
        part = sg.gemm_partial(xin, wmat)
        total = (xin.float() @ wmat.float().t()).bfloat16().float()
        dist.all_reduce(total)
        want_res = (total + resid.float()).bfloat16()
        mine = resid.clone()
        h = sg.ar_residual_rmsnorm(part, mine, w_norm if use_norm else None, 1e-6)
        ok &= bool(torch.allclose(mine.float(), want_res.float(), rtol=2e-2, atol=2e-2))
        if use_norm:
            ok &= bool(torch.allclose(h.float(), ref.rmsnorm(mine, w_norm, 1e-6).float(), rtol=2e-2, atol=2e-2))
        else:
            ok &= h is None
sg.begin_forward()
res["ar_residual_rmsnorm_ok"] = ok
res["tp_push"] = bool(sg.push)

# device time per reduction inside a CUDA graph (how the decode step runs them): 128 x 4096 bf16
T = 128
xin = torch.randn(T, 1024, device=dev).bfloat16()
resid = torch.randn(T, H, device=dev).bfloat16()
y = torch.empty(T, H, device=dev, dtype=torch.bfloat16)


def fused_pair():
    for _ in range(2):
        part = sg.gemm_partial(xin, wmat)
        sg.ar_residual_rmsnorm(part, resid, w_norm, 1e-6)


def nccl_pair():
    for _ in range(2):
        o = ref_linear(xin, wmat)
        dist.all_reduce(o)
        resid.add_(o)
        native_rmsnorm(resid, w_norm, 1e-6)


from chatlearn_b200 import ops  # noqa: E402
ref_linear, native_rmsnorm = ops.linear, ops.rmsnorm
for name, fn in (("fused", fused_pair), ("nccl", nccl_pair)):
    for _ in range(3):
        fn()
    torch.cuda.synchronize(); dist.barrier()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        for _ in range(18):
            fn()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        gr.replay()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / (10 * 36)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res[f"gemm_reduce_norm_{name}_us"] = round(t.item() * 1e3, 2)
    resid.normal_()
res["status_after_graph"] = sg.status()

# ---- reduce-scatter by pulling + AdamW + all-gather by pushing vs the NCCL statement ----
N = 1 << 20
shard = N // world
lo = rank * shard
grad = sg.symmetric_like(N, torch.float32)
param = sg.symmetric_like(N, torch.bfloat16)
torch.manual_seed(7)
full0 = torch.randn(N, device=dev)
param.copy_(full0)
master = full0[lo:lo + shard].clone()
m, v = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
master_r, m_r, v_r = master.clone(), m.clone(), v.clone()
param_r = full0.bfloat16().clone()
gshard = torch.empty(shard, device=dev)
ok = True
for step in (1, 2):
    torch.manual_seed(1000 * step + rank)
    grad.copy_(torch.randn(N, device=dev))
    torch.cuda.synchronize(); dist.barrier()
    want_g = grad.clone()
    dist.all_reduce(want_g)
    part = sg.reduce_scatter_pull(grad, gshard, lo)
    sq = part.sum()
    dist.all_reduce(sq)
    scale = torch.clamp(1.0 / (sq.sqrt() + 1e-6), max=1.0)
    checks = {"rs": bool(torch.allclose(gshard, want_g[lo:lo + shard], rtol=1e-5, atol=1e-5)),
              "sumsq": bool(torch.allclose(sq, want_g.pow(2).sum(), rtol=1e-4))}
    sg.adamw_push(master, gshard, m, v, param, lo, step, 1e-2, 0.9, 0.95, 1e-8, 0.01, scale)
    out_r = torch.empty(shard, device=dev, dtype=torch.bfloat16)
    ref.adamw_step(master_r, want_g[lo:lo + shard], m_r, v_r, out_r, step, 1e-2, 0.9, 0.95, 1e-8, 0.01, scale)
    torch.cuda.synchronize(); dist.barrier()
    # the pushed all-gather must equal an NCCL all-gather of the bf16 cast of every rank's new master shard
    mine_bf = master.bfloat16()
    gathered = [torch.empty_like(mine_bf) for _ in range(world)]
    dist.all_gather(gathered, mine_bf)
    checks["master"] = bool(torch.allclose(master, master_r, rtol=1e-4, atol=1e-5))
    checks["push"] = bool(torch.equal(param, torch.cat(gathered)))
    ok &= all(checks.values())
    res[f"zero_step{step}"] = checks
res["zero_step_ok"] = ok
res["status"] = sg.status()

# ---- the sharded optimizer step through ShardedTrainState: peer-memory kernels vs NCCL ----
from chatlearn_b200.models.nn import PRESETS as _P, CausalLM as _LM  # noqa: E402
from chatlearn_b200.parallel.zero import ShardedTrainState  # noqa: E402

ma = _LM(_P["tiny_qwen3"](), dtype=torch.bfloat16, device=dev, pad_to=world * 8).init_weights(5)
mb = _LM(_P["tiny_qwen3"](), dtype=torch.bfloat16, device=dev, pad_to=world * 8).init_weights(5)
sa = ShardedTrainState(ma, g, lr=1e-3, clip_grad=1.0)
sb = ShardedTrainState(mb, g, lr=1e-3, clip_grad=1.0)
res["zero_state_symm_enabled"] = bool(sa.enable_symm())
norms = []
for step in (1, 2, 3):
    sa.zero_grad(); sb.zero_grad()
    torch.manual_seed(50 * step + rank)
    for x, y in zip(sa.states, sb.states):
        gr_ = torch.randn(x.block.numel, device=dev) * 0.01
        x.grad.copy_(gr_); y.grad.copy_(gr_)
    na, nb = sa.step(), sb.step()
    norms.append((float(na), float(nb)))
torch.cuda.synchronize(); dist.barrier()
res["zero_state_norms"] = norms
# the two paths round the clip factor differently in the last bit, so a few bf16 weights may differ by one ulp
mism = sum(int((x.block.flat != y.block.flat).sum()) for x, y in zip(sa.states, sb.states))
tot = sum(x.block.numel for x in sa.states)
maxd = max(float((x.block.flat.float() - y.block.flat.float()).abs().max()) for x, y in zip(sa.states, sb.states))
res["zero_state_mismatch_frac"], res["zero_state_max_diff"] = mism / tot, maxd
res["zero_state_ok"] = mism / tot < 1e-2 and maxd < 1e-3 and all(abs(a - b) <= 1e-4 * abs(b) for a, b in norms)
res["zero_state_status"] = sg.status()

# ---- expert-parallel MoE layer through peer memory (dispatch with remote atomics, pull combine) ----
from chatlearn_b200.parallel.symm_moe import SymmMoE  # noqa: E402

E, Hm, Fm, kk = 8, 256, 128, 2
El = E // world
torch.manual_seed(77)
w13_all = (torch.randn(E, 2 * Fm, Hm, device=dev) * 0.05).bfloat16()
w2_all = (torch.randn(E, Hm, Fm, device=dev) * 0.05).bfloat16()
moe = SymmMoE(g, E, Hm)
ok = True
for step, Tm in enumerate((64, 300, 17)):
    torch.manual_seed(900 + 10 * step + rank)
    xm = torch.randn(Tm, Hm, device=dev).bfloat16()
    wts, idxm, _ = ref.moe_router(torch.randn(Tm, E, device=dev), kk)
    got = moe.experts(xm, w13_all[rank * El:(rank + 1) * El].contiguous(), w2_all[rank * El:(rank + 1) * El].contiguous(),
                      wts, idxm, pairs_per_rank=300 * kk)
    want = ref.moe_experts(xm.float(), w13_all.float(), w2_all.float(), wts, idxm)
    torch.cuda.synchronize()
    rel = float((got.float() - want).norm() / want.norm())
    ok &= rel < 2e-2
    res[f"symm_moe_rel_err_{Tm}"] = round(rel, 5)
dist.barrier()
res["symm_moe_ok"] = ok
res["symm_moe_status"] = moe.status()

# ---- weight sync: pull fp32 ZeRO shards from the peer into the rollout TP layout (bf16) ----
from chatlearn_b200.models.nn import PRESETS, CausalLM  # noqa: E402
from chatlearn_b200.parallel import symm_mem  # noqa: E402
from chatlearn_b200.synchronizer.kernel_executor import KernelExecutor  # noqa: E402
from chatlearn_b200.synchronizer.parameter_sync import layout_of_model  # noqa: E402
from chatlearn_b200.synchronizer.plan import build_plan, validate_plan  # noqa: E402

arch = PRESETS["tiny_qwen3"]()
full = CausalLM(arch, dtype=torch.float32, device=dev, pad_to=world).init_weights(3)      # identical on every rank
src_bufs, shards = {}, {}
for b in full.blocks:
    sh = b.numel // world
    t = symm_mem.empty(sh, torch.float32, dev)
    t.copy_(b.flat[rank * sh:(rank + 1) * sh])
    src_bufs[f"s/{b.name}"] = t
    shards[b.name] = sh
dst = CausalLM(arch, dtype=torch.bfloat16, device=dev, tp=world, tp_rank=rank)
want = CausalLM(arch, dtype=torch.bfloat16, device=dev, tp=world, tp_rank=rank)
want.load_hf_state_dict(full.hf_state_dict())
src_lays = [layout_of_model(full, r, lambda name, r=r: (r * shards[name], (r + 1) * shards[name]), "s/") for r in range(world)]
dst_lays = []
for r in range(world):
    proto = CausalLM(arch, dtype=torch.bfloat16, device="meta", tp=world, tp_rank=r, allocate=False)
    dst_lays.append(layout_of_model(proto, r, prefix="d/"))
plan = build_plan(src_lays, dst_lays)
validate_plan(plan, dst_lays)
ex = KernelExecutor(plan, rank, world)
torch.cuda.synchronize(); dist.barrier()
ex.run(src_bufs, {f"d/{b.name}": b.flat for b in dst.blocks})
torch.cuda.synchronize()
res["weight_sync_ok"] = all(torch.equal(a.flat, b.flat) for a, b in zip(dst.blocks, want.blocks))
res["weight_sync_remote_descs"] = sum(1 for d in ex.descs if d.src_rank != rank)
if rank == 0:
    print("RESULT " + json.dumps(res), flush=True)
del gr
from chatlearn_b200.launcher.initialize import shutdown  # noqa: E402
shutdown()
