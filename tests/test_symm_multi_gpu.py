"""In-kernel collectives on two GPUs (all-reduce, fused all-reduce+residual+RMSNorm, pull
reduce-scatter + AdamW push, the sharded train state on them, peer weight-sync pull).
Runs ``tests/symm_driver.py`` under torchrun; skipped on boxes with fewer than two GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

from chatlearn_b200.utils.utils import get_free_port as free_port

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_symm_collectives_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "symm_driver.py")],
                       capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-2000:]
    r = json.loads(lines[-1][7:])
    for key in ("allreduce_ok", "ar_residual_rmsnorm_ok", "zero_step_ok", "zero_state_symm_enabled", "zero_state_ok", "symm_moe_ok",
                "weight_sync_ok"):
        assert r[key], (key, r)
    assert r["status"] == 0 and r["status_after_graph"] == 0 and r["zero_state_status"] == 0 and r["symm_moe_status"] == 0


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_rollout_paths_agree():
    outs = {}
    for flag in ("0", "1"):
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", CLB200_SYMM_EP=flag)
        p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                            "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "ep_rollout_driver.py")],
                           capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
        res = [json.loads(l[7:]) for l in p.stdout.splitlines() if l.startswith("RESULT ")]
        assert p.returncode == 0 and len(res) == 2, p.stdout[-2000:] + p.stderr[-2000:]
        outs[flag] = {r["rank"]: r for r in res}
    assert all(outs["1"][r]["symm_ep"] and not outs["0"][r]["symm_ep"] for r in (0, 1))
    assert all(outs["1"][r]["checksum"] == outs["0"][r]["checksum"] for r in (0, 1))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_exchange_two_gpus():
    """All-gather and equal-split all-to-all by peer stores agree bit for bit with NCCL, alone and
    inside the Ulysses head/sequence exchange with gradients."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "exchange_driver.py")],
                       capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-2000:]
    r = json.loads(lines[-1][7:])
    for key in ("all_gather_ok", "all_to_all_ok", "fallback_ok", "ulysses_ok", "gemm_reduce_scatter_ok"):
        assert r[key], (key, r)
    assert r["status"] == 0


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_parameter_sharded_state_two_gpus():
    """FSDP2-style state (blocks pulled from the peers' parameter slices per segment, gradients reduce-scattered
    by the pull kernel after every segment's backward) against the replicated state on NCCL."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "fsdp2_driver.py")],
                       capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-2000:]
    r = json.loads(lines[-1][7:])
    assert r["symm_pull"] and r["status"] == 0, r
    for la, lb in r["loss"]:
        assert abs(la - lb) < 2e-2 * max(1.0, abs(la)), r
    for na, nb in r["norm"]:
        assert abs(na - nb) < 2e-2 * max(1.0, abs(na)), r
    # bf16 weights after two AdamW steps: a last-bit difference in a gradient moves an update by a bf16 ulp
    assert r["param_diff"] < 2e-2 and r["param_mismatch_frac"] < 0.05, r
    assert r["resident_param_bytes"] * 2 == r["whole_param_bytes"]
    assert r["score_diff"] < 5e-2, r          # the two models differ by a few bf16 ulps after two steps
