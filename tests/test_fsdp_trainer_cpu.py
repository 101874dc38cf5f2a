"""The data-parallel trainer with Ulysses sequence parallelism, hybrid sharding or sharded parameters must reproduce
the single-rank result: same log-probs, same loss statistics, same weights after one optimizer step."""
import os
import subprocess
import sys

import pytest
import torch

from chatlearn_b200.utils.utils import get_free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "tests", "fsdp_trainer_driver.py")


def _run(out_dir, tag, world, **env):
    port = get_free_port()
    procs = []
    for r in range(world):
        e = dict(os.environ, OUT_DIR=str(out_dir), TAG=tag, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world),
                 MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CHATLEARN_FORCE_CPU="1", OMP_NUM_THREADS="2")
        e.update({k: str(v) for k, v in env.items()})
        procs.append(subprocess.Popen([sys.executable, DRIVER], env=e, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2500:] for o in outs)
    return torch.load(os.path.join(out_dir, f"{tag}.pt"), weights_only=False)


_BASE = {}


@pytest.fixture(scope="module")
def base_dir(tmp_path_factory):
    return tmp_path_factory.mktemp("single_rank")


def _base(base_dir, **env):
    """The single-rank result for one set of model settings (computed once per module)."""
    key = tuple(sorted((k, str(v)) for k, v in env.items()))
    if key not in _BASE:
        d = base_dir / f"base{len(_BASE)}"
        d.mkdir()
        _BASE[key] = _run(d, "base", 1, **env)
    return _BASE[key]


def _compare(a, b, tol=5e-4, outliers=2):
    """Adam's first step moves an element by the learning rate times the sign of its gradient, so a gradient at
    rounding level can land on either side (at most 2 * lr apart): a few such elements per tensor are allowed."""
    for x, y in zip(a["logprobs"], b["logprobs"]):
        assert (x - y).abs().max().item() < 1e-4
    assert set(a["sd"]) == set(b["sd"])
    for k in a["sd"]:
        d = (a["sd"][k] - b["sd"][k]).abs()
        assert int((d >= tol).sum()) <= outliers and d.max().item() < 2.1e-3, (k, d.max().item(), int((d >= tol).sum()))
    for k in ("pg_loss", "kl_loss", "entropy_loss", "grad_norm"):
        assert abs(a["metrics"][k] - b["metrics"][k]) < 5e-4 * max(1.0, abs(a["metrics"][k])), (k, a["metrics"], b["metrics"])


@pytest.mark.parametrize("name,world,env", [
    ("dp2", 2, dict()),
    ("ulysses2", 2, dict(ULYSSES=2)),                    # every packed row split over the two ranks
    ("ulysses2_gspo", 2, dict(ULYSSES=2, GSPO=1)),
    ("ulysses2_resharded", 2, dict(ULYSSES=2, RESHARD=1)),
    ("ulysses4_replicated_kv_heads", 4, dict(ULYSSES=4)),   # four ranks, two key/value heads
    # hybrid sharding: two shard groups of two ranks with sharded parameters
    ("hsdp2x2_resharded", 4, dict(FSDP=2, RESHARD=1)),
])
def test_dense_matches_single(tmp_path, base_dir, name, world, env):
    base = _base(base_dir, **{k: v for k, v in env.items() if k == "GSPO"})
    par = _run(tmp_path, name, world, **env)
    _compare(base, par)


@pytest.mark.parametrize("name,world,env", [
    ("moe_ulysses2", 2, dict(PRESET="tiny_moe", ULYSSES=2)),
    ("moe_ulysses2_balancing_loss", 2, dict(PRESET="tiny_moe", ULYSSES=2, AUX=1)),   # statistics over both ranks' rows
    # sharded parameters: the segments' forward runs without a tape, the balancing losses are back-propagated from
    # the re-run inside each segment's backward
    ("moe_resharded_ulysses2_balancing_loss", 2, dict(PRESET="tiny_moe", ULYSSES=2, RESHARD=1, AUX=1)),
    # latent attention: queries, (decompressed) keys and values trade rows for heads after the rotary parts were rotated
    ("mla_ulysses2", 2, dict(PRESET="tiny_mla_moe", ULYSSES=2)),
    # Qwen3-Next: the convolution and the recurrence of the delta-net layers run per head over whole sequences
    ("hybrid_ulysses2", 2, dict(PRESET="tiny_qwen3_next", ULYSSES=2))])
def test_moe_matches_single(tmp_path, base_dir, name, world, env):
    base = _base(base_dir, **{k: v for k, v in env.items() if k in ("PRESET", "AUX")})
    par = _run(tmp_path, name, world, **env)
    _compare(base, par)


@pytest.mark.parametrize("name,world,env", [
    ("vl_ulysses2", 2, dict(PRESET="tiny_qwen2_5_vl", ULYSSES=2)),
    # Qwen3-VL: deep-stack taps at the image rows this rank holds; the tower's weights trained
    ("vl3_ulysses2_trained_tower", 2, dict(PRESET="tiny_qwen3_vl", ULYSSES=2, TRAIN_TOWER=1)),
    # sharded parameters: the tower's output enters inside the first segment (embedding and tower blocks gathered)
    ("vl_resharded_trained_tower", 2, dict(PRESET="tiny_qwen2_5_vl", RESHARD=1, TRAIN_TOWER=1)),
    ("vl3_resharded_ulysses2", 2, dict(PRESET="tiny_qwen3_vl", RESHARD=1, ULYSSES=2)),
    # ... and the deep-stack taps of a trained tower cross the segment boundaries as outputs / inputs
    ("vl3_resharded_trained_tower", 2, dict(PRESET="tiny_qwen3_vl", RESHARD=1, TRAIN_TOWER=1))])
def test_vision_language_matches_single(tmp_path, base_dir, name, world, env):
    """Rows with image patches under Ulysses: embeddings and positions are built for the whole packed row, a rank
    keeps its rows of the embeddings and the whole positions (the attention runs on all rows of its heads)."""
    base = _base(base_dir, **{k: v for k, v in env.items() if k in ("PRESET", "TRAIN_TOWER")})
    par = _run(tmp_path, name, world, **env)
    _compare(base, par)
