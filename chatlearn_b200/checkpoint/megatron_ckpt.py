"""Megatron-layout checkpoints.

The reference calls Megatron-Core's ``save_checkpoint`` into
``{output_dir}/save_model/{name}`` (chatlearn/models/megatron_module.py:175-190) and
resumes by flipping ``no_load_optim/rng/scheduler`` (megatron_policy_trainer.py:77-85).
The directory convention written here is Megatron's:

    {root}/latest_checkpointed_iteration.txt
    {root}/iter_{iteration:07d}/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt
    {root}/iter_{iteration:07d}/mp_rank_.../distrib_optim_dp{dp:03d}.pt   (optimizer shards)

``model_optim_rng.pt`` holds ``{"iteration", "model": {local leaf name: tensor},
"layout": {leaf name: HF rectangles}, "rng_state", "args"}``; the model part is
written once per model-parallel rank (data-parallel rank 0).  Because the leaf →
HF rectangle layout travels with the file, a checkpoint can be re-assembled into
HF tensors offline (``offline_ckpt_converter``) without this framework's classes.
"""
import os

import torch

from chatlearn_b200.configs import to_container

LATEST = "latest_checkpointed_iteration.txt"


def mp_rank_dir(tp: int, pp: int, ep: int, pp_size: int, ep_size: int) -> str:
    d = f"mp_rank_{tp:02d}"
    if pp_size > 1:
        d += f"_{pp:03d}"
    if ep_size > 1:
        d += f"_{ep:03d}"
    return d


def save_megatron_checkpoint(module, root: str, iteration: int):
    c = module.mesh.coords
    d = os.path.join(root, f"iter_{iteration:07d}",
                     mp_rank_dir(c["tp"], c["pp"], c["ep"], module.pp_size, module.ep_size))
    os.makedirs(d, exist_ok=True)
    dp = c["dp"] * module.cp_size + c["cp"]
    if dp == 0 or (module.ep_size > 1 and c["edp"] == 0 and c["cp"] == 0):
        model_sd, layout = {}, {}
        for name, p, lf, _ in module.model.named_leaves():
            model_sd[name] = p.detach().cpu()
            layout[name] = [(s.hf_name, s.hf_shape, s.src_start, s.extent, s.dst_start, s.dst_index)
                            for s in lf.segments]
        torch.save({"iteration": iteration, "model": model_sd, "layout": layout,
                    "rng_state": module.get_rng_state(), "checkpoint_version": 3.0,
                    "args": to_container(module.module_args)}, os.path.join(d, "model_optim_rng.pt"))
    if module.state is not None:
        torch.save(module.state.state_dict(), os.path.join(d, f"distrib_optim_dp{dp:03d}.pt"))
    if module.get_rank() == module.placement[0]:
        tmp = os.path.join(root, LATEST + f".tmp{os.getpid()}")
        with open(tmp, "w", encoding="utf-8") as f:
            f.write(str(iteration))
        os.replace(tmp, os.path.join(root, LATEST))


def load_megatron_checkpoint(module, root: str, iteration=None) -> bool:
    if iteration is None:
        p = os.path.join(root, LATEST)
        if not os.path.exists(p):
            return False
        with open(p, "r", encoding="utf-8") as f:
            iteration = int(f.read().strip())
    c = module.mesh.coords
    d = os.path.join(root, f"iter_{iteration:07d}",
                     mp_rank_dir(c["tp"], c["pp"], c["ep"], module.pp_size, module.ep_size))
    mp = os.path.join(d, "model_optim_rng.pt")
    if not os.path.exists(mp):
        return False
    sd = torch.load(mp, weights_only=False)
    with torch.no_grad():
        for name, p, _, _ in module.model.named_leaves():
            p.copy_(sd["model"][name])
    dp = c["dp"] * module.cp_size + c["cp"]
    op = os.path.join(d, f"distrib_optim_dp{dp:03d}.pt")
    no_load_optim = bool(getattr(module.module_args, "no_load_optim", False)) and not module._resume_training
    if module.state is not None and os.path.exists(op) and not no_load_optim:
        module.state.load_state_dict(torch.load(op, weights_only=False))
    elif module.state is not None:
        for s in module.state.states:        # fresh optimizer on the loaded weights
            s.master.copy_(s.block.flat[s.lo:s.hi])
    if not (getattr(module.module_args, "no_load_rng", False) and not module._resume_training):
        module.set_rng_state(sd["rng_state"])
    return True
