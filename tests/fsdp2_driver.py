"""Two-GPU check of the parameter-sharded training state (run under torchrun, one rank per GPU): the pull
all-gather and the pull reduce-scatter over symmetric memory against the replicated state on NCCL."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from chatlearn_b200.launcher.initialize import init_distributed, shutdown  # noqa: E402
from chatlearn_b200.models.nn import PRESETS, CausalLM, packed_ctx  # noqa: E402
from chatlearn_b200.parallel.fsdp2 import ReshardedTrainState  # noqa: E402
from chatlearn_b200.parallel.groups import Group  # noqa: E402
from chatlearn_b200.parallel.zero import ShardedTrainState  # noqa: E402

init_distributed()
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
g = Group(dist.group.WORLD, list(range(world)), "dp")
arch = PRESETS["tiny_qwen3"]()
arch.head_dim, arch.num_attention_heads, arch.num_key_value_heads = 128, 4, 2      # the tensor-memory attention kernels
ma = CausalLM(arch, dtype=torch.bfloat16, device=dev, pad_to=world * 8).init_weights(7)
mb = CausalLM(arch, dtype=torch.bfloat16, device=dev, pad_to=world * 8).init_weights(7)
sa = ShardedTrainState(ma, g, lr=1e-3, clip_grad=1.0)
sb = ReshardedTrainState(mb, g, lr=1e-3, clip_grad=1.0)
res = {"symm_pull": sb.symm_gather is not None, "loss": [], "norm": []}
for step in range(2):
    sa.zero_grad(); sb.zero_grad()
    nmb = 2 if (rank == 0 or step == 1) else 1           # rank 1 joins one micro-batch with zeros
    for mbi in range(2):
        if mbi >= nmb:
            sb.join_empty_microbatch()
            continue
        torch.manual_seed(100 * step + 10 * mbi + rank)
        lens = [170 + rank, 300, 50 + mbi]
        T = sum(lens)
        toks = torch.randint(0, arch.vocab_size - 1, (T,), device=dev)
        labels = toks.roll(-1)
        ca, _ = packed_ctx(lens, dev)
        cb, _ = packed_ctx(lens, dev)
        lp_a, ent_a = ma.logprobs(toks, labels, ca)
        lp_b, ent_b = sb.logprobs(toks, labels, cb)
        la = -(lp_a.sum() + 0.01 * ent_a.sum()) / T
        lb = -(lp_b.sum() + 0.01 * ent_b.sum()) / T
        la.backward(); lb.backward()
        res["loss"].append((la.item(), lb.item()))
    na, nb = sa.step(), sb.step()
    res["norm"].append((float(na), float(nb)))
# scoring pass as the trainer runs it: no tape, residual adds fused into the following norms
with torch.no_grad():
    lens = [90, 200]
    toks = torch.randint(0, arch.vocab_size - 1, (sum(lens),), device=dev)
    c1, _ = packed_ctx(lens, dev); c2, _ = packed_ctx(lens, dev)
    c1.fuse_add_norm = c2.fuse_add_norm = True
    res["score_diff"] = (ma.logprobs(toks, toks.roll(-1), c1)[0] - sb.logprobs(toks, toks.roll(-1), c2)[0]).abs().max().item()
torch.cuda.synchronize()
with sb.all_gathered() as whole:
    diffs = [(x.flat.float() - y.flat.float()).abs().max().item() for x, y in zip(ma.blocks, whole.blocks)]
    mism = sum(int((x.flat != y.flat).sum()) for x, y in zip(ma.blocks, whole.blocks)) / sum(b.numel for b in ma.blocks)
res["param_diff"], res["param_mismatch_frac"] = max(diffs), mism
res["status"] = int(sb.symm_gather.status()) if sb.symm_gather is not None else 0
res["resident_param_bytes"] = sum(s.param_shard.numel() * 2 for s in sb.states)
res["whole_param_bytes"] = sum(b.numel * 2 for b in ma.blocks)
if rank == 0:
    print("RESULT " + json.dumps(res), flush=True)
shutdown()
