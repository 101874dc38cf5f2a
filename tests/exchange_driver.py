"""Multi-GPU check of the peer-memory all-gather / all-to-all (run under torchrun, one rank per GPU)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from chatlearn_b200.launcher.initialize import init_distributed, shutdown  # noqa: E402
from chatlearn_b200.parallel import symm_collectives  # noqa: E402
from chatlearn_b200.parallel.groups import Group  # noqa: E402
from chatlearn_b200.parallel.ulysses import UlyssesGroup  # noqa: E402

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
init_distributed()
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
g = Group(dist.group.WORLD, list(range(world)), "world")
plain = Group(dist.group.WORLD, list(range(world)), "plain")          # NCCL only
sg = symm_collectives.attach_exchange(g)
assert sg is not None and "exchange" in g.fast
res = {}

torch.manual_seed(7 + rank)
ok = True
for shape in ((8,), (300, 24), (1024, 8, 128), (4096, 1024)):
    for rep in range(3):                                               # both receive buffers, counters advance
        x = torch.randn(*shape, device=dev).bfloat16()
        for dim in (0, len(shape) - 1):
            ok &= bool(torch.equal(g.all_gather_cat(x, dim), plain.all_gather_cat(x, dim)))
res["all_gather_ok"] = ok

ok = True
for shape, dt in (((world * 4, 8), torch.float32), ((world * 512, 4, 128), torch.bfloat16), ((world * 3000, 1024), torch.bfloat16)):
    for rep in range(3):
        x = torch.randn(*shape, device=dev).to(dt)
        ok &= bool(torch.equal(g.all_to_all_single(x), plain.all_to_all_single(x)))
res["all_to_all_ok"] = ok

# tensors the kernel does not take (chunk not a multiple of 16 bytes) go through NCCL
before = sg.native.launch_counts["symm_exchange"]
x = torch.randn(world * 3, 1, device=dev).bfloat16()
ok = bool(torch.equal(g.all_to_all_single(x), plain.all_to_all_single(x)))
ok &= bool(torch.equal(g.all_gather_cat(x[:3]), plain.all_gather_cat(x[:3])))
res["fallback_ok"] = ok and sg.native.launch_counts["symm_exchange"] == before

# Ulysses exchange with gradients: sequence split -> head split -> sequence split
outs = []
for grp in (g, plain):
    torch.manual_seed(50 + rank)
    q = torch.randn(256, 8, 64, device=dev).bfloat16().requires_grad_(True)
    u = UlyssesGroup(grp)
    h = u.seq_to_heads(q)
    y = u.heads_to_seq(h * 2.0)
    (y.float() * torch.arange(y.numel(), device=dev).view_as(y) / y.numel()).sum().backward()
    outs.append((h.detach().clone(), y.detach().clone(), q.grad.clone()))
res["ulysses_ok"] = all(bool(torch.equal(a, b)) for a, b in zip(*outs))


def timed(fn, iters=20):
    for _ in range(5):
        fn()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


# Ulysses query exchange of an 8192-token local sequence, 32 heads x 128 (64 MB), and the
# context-parallel key/value gather of 8192 tokens x 8 kv heads x 128 x 2 (32 MB per rank)
xa = torch.randn(8192 * world, 32 // world, 128, device=dev).bfloat16()
xg = torch.randn(8192, 2 * 8 * 128, device=dev).bfloat16()
for name, grp in (("symm", g), ("nccl", plain)):
    res[f"a2a_ms_{name}"] = round(timed(lambda: grp.all_to_all_single(xa)), 4)
    res[f"ag_ms_{name}"] = round(timed(lambda: grp.all_gather_cat(xg)), 4)
res["a2a_bytes_sent_per_rank"] = xa.numel() * 2 * (world - 1) // world
res["ag_bytes_recv_per_rank"] = xg.numel() * 2 * (world - 1)
# ---- fused GEMM + reduce-scatter (row-parallel layer under sequence parallelism) against GEMM + NCCL ----
from chatlearn_b200 import ops  # noqa: E402
ops.set_mode("native")
fused = symm_collectives.attach_gemm_reduce_scatter(g)
assert fused is not None and "gemm_rs" in g.fast
ok, worst = True, 0.0
for M, N, K in ((world * 256, 512, 384), (world * 1000, 4096, 1024), (16384, 4096, 2048)):
    for rep in range(3):                                               # both receive buffers
        x = (torch.randn(M, K, device=dev) * 0.5).bfloat16().requires_grad_(True)
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16().requires_grad_(True)
        y = g.fast["gemm_rs"](x, w)
        full = x.detach().float() @ w.detach().float().t()
        dist.all_reduce(full)
        want = full[rank * (M // world):(rank + 1) * (M // world)]
        err = ((y.float() - want).norm() / want.norm()).item()
        worst = max(worst, err)
        ok &= y.shape == want.shape and err < 1e-2
        # gradients: those of all_gather(dy) through an ordinary linear layer
        gy = torch.randn_like(y)
        y.backward(gy)
        gfull = plain.all_gather_cat(gy, 0).float()
        ok &= ((x.grad.float() - gfull @ w.detach().float()).norm() / (gfull @ w.detach().float()).norm()).item() < 1e-2
        ok &= ((w.grad.float() - gfull.t() @ x.detach().float()).norm() / (gfull.t() @ x.detach().float()).norm()).item() < 1e-2
res["gemm_reduce_scatter_ok"], res["gemm_reduce_scatter_rel_err"] = bool(ok), round(worst, 5)
M, N, K = 16384, 4096, 12288 // world                                   # down projection of Qwen3-8B, K split over the ranks
x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
out_nccl = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)


def rs_fused():
    return sg.gemm_reduce_scatter(x, w)


def gemm_only():
    return __import__("chatlearn_b200.ops.native", fromlist=["x"]).gemm_nt(x, w)


def rs_nccl2():
    dist.reduce_scatter_tensor(out_nccl, gemm_only())
    return out_nccl


for name, fn in (("fused", rs_fused), ("gemm_then_nccl", rs_nccl2), ("gemm_alone", gemm_only)):
    for _ in range(3):
        fn()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res[f"gemm_rs_{name}_us"] = round(t.item() * 1e3, 1)
res["gemm_rs_shape"] = [M, N, K]
res["gemm_rs_bytes_over_nvlink_per_rank"] = M * N * 2 * (world - 1) // world
res["status"] = sg.status()
if rank == 0:
    print("RESULT " + json.dumps(res), flush=True)
shutdown()
