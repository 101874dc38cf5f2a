"""Expert-parallel rollout on two GPUs: NCCL all-to-all path vs peer-memory dispatch (run under
torchrun with CLB200_SYMM_EP=0 / 1; prints greedy tokens' checksum and the time per decode step)."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from chatlearn_b200.launcher.initialize import init_distributed, shutdown  # noqa: E402
from chatlearn_b200.models.nn import PRESETS, CausalLM  # noqa: E402
from chatlearn_b200.parallel.expert_parallel import ExpertParallel  # noqa: E402
from chatlearn_b200.parallel.groups import Group  # noqa: E402
from chatlearn_b200.rollout import RolloutEngine, SamplingParams  # noqa: E402

init_distributed()
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
torch.cuda.set_device(dev)
g = Group(dist.group.WORLD, list(range(world)), "ep")
arch = PRESETS[os.environ.get("MODEL", "tiny_moe")]()
if os.environ.get("LAYERS"):
    arch.num_hidden_layers = int(os.environ["LAYERS"])
model = CausalLM(arch, dtype=torch.bfloat16, device=dev, ep=world, ep_rank=rank).init_weights(3)
eng = RolloutEngine(model, ep_group=ExpertParallel(g), lockstep_group=g, block_size=16, num_blocks=4096,
                    max_num_seqs=64, max_num_batched_tokens=4096, max_model_len=512, seed=5)
B, new = int(os.environ.get("BATCH", "32")), int(os.environ.get("NEW", "24"))
gen = torch.Generator().manual_seed(100 + rank)
prompts = [torch.randint(0, arch.vocab_size - 1, (int(torch.randint(8, 40, (1,), generator=gen)),), generator=gen).tolist()
           for _ in range(B)]
sp = SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True)
eng.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
torch.cuda.synchronize(); dist.barrier()
t0 = time.perf_counter()
seqs = eng.generate(prompts, sp)
torch.cuda.synchronize()
dt = time.perf_counter() - t0
toks = [t for s in seqs for t in s.output]
res = {"rank": rank, "symm_ep": eng.ep_symm is not None, "tokens": len(toks), "first": toks[:12],
       "checksum": int(sum((i + 1) * t for i, t in enumerate(toks)) % 1000003),
       "ms_per_decode_step": round(eng.stats["decode_s"] / max(eng.stats["decode_steps"], 1) * 1e3, 3), "total_s": round(dt, 3)}
print("RESULT " + json.dumps(res), flush=True)
shutdown()
