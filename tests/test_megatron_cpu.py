"""The TP / PP / CP / EP trainer must reproduce the single-rank result: same
log-probs, same loss statistics, same weights after one optimizer step."""
import os
import subprocess
import sys

import pytest
import torch

from chatlearn_b200.utils.utils import get_free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "tests", "megatron_driver.py")


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


def _compare(a, b, tol=5e-4, outliers=0):
    """``outliers``: how many elements per tensor may differ by more than ``tol`` (Adam's first step moves an
    element by the learning rate times the sign of its gradient, so a gradient at rounding level can land on either
    side: at most 2 * lr apart)."""
    assert set(a["sd"]) == set(b["sd"])
    for k in a["sd"]:
        d = (a["sd"][k] - b["sd"][k]).abs()
        if outliers:
            assert int((d >= tol).sum()) <= outliers and d.max().item() < 2.1e-3, (k, d.max().item(), int((d >= tol).sum()))
        else:
            assert d.max().item() < tol, (k, d.max().item())
    for k in ("pg_loss", "kl_loss", "entropy_loss", "grad_norm"):
        assert abs(a["metrics"][k] - b["metrics"][k]) < 5e-4 * max(1.0, abs(a["metrics"][k])), (k, a["metrics"], b["metrics"])


@pytest.mark.parametrize("name,world,env", [
    ("tp2", 2, dict(TP=2)),                      # rows split over the tensor-parallel ranks between the layers
    ("tp2_no_seq_par", 2, dict(TP=2, SEQ_PAR=0)),
    ("tp2pp2", 4, dict(TP=2, PP=2)),
    ("tp2cp2", 4, dict(TP=2, CP=2)),
    ("pp2", 2, dict(PP=2)),
    ("cp2", 2, dict(CP=2)),
    ("dp2", 2, dict()),
    ("tp2_gspo", 2, dict(TP=2, GSPO=1)),
    ("cp2_gspo", 2, dict(CP=2, GSPO=1)),         # sequence-level ratios need every rank's rows of a sequence
    # tied input / output embeddings: the first and the last stage hold copies and exchange their gradients
    ("pp2_tied", 2, dict(PP=2, ARCH_JSON='{"tie_word_embeddings": true}')),
    ("tp2pp2_tied", 4, dict(TP=2, PP=2, ARCH_JSON='{"tie_word_embeddings": true}')),
    # two model chunks per stage, interleaved one-forward-one-backward over a global time table
    ("pp2vpp2", 2, dict(PP=2, VPP=2, LAYERS=4)),
    # ... and with four of the six layers on the first stage: chunks of two layers there, of one layer on the second
    ("pp2vpp2_uneven", 2, dict(PP=2, VPP=2, LAYERS=6, FIRST=4)),
    # more ranks than key/value heads: two ranks hold each head, and the gradients of its rows are summed over them
    ("tp4_replicated_kv_heads", 4, dict(TP=4)),
])
def test_dense_parallel_matches_single(tmp_path, base_dir, name, world, env):
    base_env = {k: v for k, v in env.items() if k in ("GSPO", "LAYERS", "ARCH_JSON")}
    base = _base(base_dir, **base_env)
    par = _run(tmp_path, name, world, **env)
    _compare(base, par)


@pytest.mark.parametrize("name,world,env", [("ep2", 2, dict(EP=2)), ("tp2ep2", 4, dict(TP=2, EP=2)),
                                            ("tp2etp2", 2, dict(TP=2, ETP=2)), ("tp2etp2ep2", 4, dict(TP=2, ETP=2, EP=2)),
                                            ("tp2_replicated_experts", 2, dict(TP=2))])
def test_moe_parallel_matches_single(tmp_path, base_dir, name, world, env):
    base = _base(base_dir, PRESET="tiny_moe", NOAUX=1)
    par = _run(tmp_path, name, world, PRESET="tiny_moe", NOAUX=1, **env)
    _compare(base, par, tol=5e-4)


@pytest.mark.parametrize("name,world,env", [
    ("tp2", 2, dict(TP=2)), ("tp2_no_seq_par", 2, dict(TP=2, SEQ_PAR=0)), ("tp2pp2", 4, dict(TP=2, PP=2)),
    # four key heads in the delta-net layers, two key/value heads (each on two ranks) in the attention layers
    ("tp4", 4, dict(TP=4, ARCH_JSON='{"linear_num_key_heads": 4}')),
    # context parallelism: the delta-net layers exchange their zig-zag rows for all rows of half of the heads, the
    # attention layers gather keys and values
    ("cp2", 2, dict(CP=2)), ("tp2cp2", 4, dict(TP=2, CP=2, ARCH_JSON='{"linear_num_key_heads": 4}'))])
def test_hybrid_parallel_matches_single(tmp_path, base_dir, name, world, env):
    """Qwen3-Next: the heads of the gated delta-net layers (input projections, convolution channels, decay
    parameters, recurrent state) and of the gated attention layers split over the tensor-parallel ranks."""
    base = _base(base_dir, PRESET="tiny_qwen3_next", NOAUX=1, **{k: v for k, v in env.items() if k == "ARCH_JSON"})
    par = _run(tmp_path, name, world, PRESET="tiny_qwen3_next", NOAUX=1, **env)
    _compare(base, par, tol=5e-4, outliers=2)


@pytest.mark.parametrize("name,world,env", [
    ("cp2", 2, dict(CP=2)), ("tp2", 2, dict(TP=2)), ("pp2", 2, dict(PP=2)),
    # sequence-parallel rows and a context-parallel slice at once, with the tower's weights trained
    ("tp2cp2_trained_tower", 4, dict(TP=2, CP=2, TRAIN_TOWER=1)),
    # Qwen3-VL: the tower's deep-stack taps are added to the first layers at the image rows this rank holds
    ("deepstack_cp2", 2, dict(CP=2, PRESET="tiny_qwen3_vl"))])
def test_vision_language_parallel_matches_single(tmp_path, base_dir, name, world, env):
    """Rows with image patches: the tower's embeddings and the (time, row, column) positions are built for the whole
    packed row; a context-parallel rank keeps its zig-zag slice of both, later pipeline stages only the positions."""
    env = dict(env)
    preset = env.pop("PRESET", "tiny_qwen2_5_vl")
    base = _base(base_dir, PRESET=preset, **{k: v for k, v in env.items() if k == "TRAIN_TOWER"})
    par = _run(tmp_path, name, world, PRESET=preset, **env)
    _compare(base, par, tol=5e-4, outliers=2)


@pytest.mark.parametrize("name,world,env", [
    ("tp2", 2, dict(TP=2)), ("cp2", 2, dict(CP=2)), ("tp2ep2", 4, dict(TP=2, EP=2)),
    # compressed queries as well: their down-projection and norm feed this rank's heads only
    ("tp2_q_lora", 2, dict(TP=2, ARCH_JSON='{"q_lora_rank": 24}'))])
def test_latent_attention_parallel_matches_single(tmp_path, base_dir, name, world, env):
    """DeepSeek-V3 / Moonlight layers: the latent, the rotary key and the compressed query are shared by all heads, of
    which a tensor-parallel rank sees its own, so the gradients of those projections and norms are summed over the
    group."""
    benv = dict(PRESET="tiny_mla_moe", NOAUX=1, **{k: v for k, v in env.items() if k == "ARCH_JSON"})
    base = _base(base_dir, **benv)
    par = _run(tmp_path, name, world, **benv, **{k: v for k, v in env.items() if k != "ARCH_JSON"})
    _compare(base, par, outliers=2)


@pytest.mark.parametrize("name,world,env", [("tp2", 2, dict(TP=2)), ("cp2", 2, dict(CP=2))])
def test_balancing_loss_covers_all_rows_of_a_micro_batch(tmp_path, base_dir, name, world, env):
    """Router load-balancing loss switched on: where the rows of a micro-batch are split over sequence-parallel or
    context-parallel ranks, the routed fractions and mean probabilities are those of all its rows (alignment padding
    left out), and the ranks together apply the loss once."""
    base = _base(base_dir, PRESET="tiny_moe")
    par = _run(tmp_path, name, world, PRESET="tiny_moe", **env)
    _compare(base, par, outliers=2)
