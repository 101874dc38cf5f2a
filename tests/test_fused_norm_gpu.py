"""Residual add fused with RMSNorm, and the in-place inference path of the decoder built on it."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H", [(1, 4096), (333, 2048), (64, 8192), (17, 256)])
def test_add_rmsnorm_matches_reference(T, H):
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import reference as ref
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = torch.randn(T, H, device=dev).bfloat16()
    d = torch.randn(T, H, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
    x1, x0 = x.clone(), x.clone()
    before = ops.launch_counts["add_residual_rmsnorm"]
    h1 = ops.add_rmsnorm_(x1, d, w, 1e-6)
    assert ops.launch_counts["add_residual_rmsnorm"] == before + 1
    h0 = ref.add_rmsnorm_(x0, d, w, 1e-6)
    assert torch.equal(x1, x0)                       # bf16(x + d) both ways
    assert torch.allclose(h1.float(), h0.float(), rtol=2e-2, atol=2e-2)
    x2 = x.clone()
    assert ops.add_rmsnorm_(x2, d, None, 1e-6) is None and torch.equal(x2, x0)


@pytest.mark.parametrize("preset", ["tiny_qwen3", "tiny_moe"])
def test_fused_inference_path_matches_plain(preset):
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.models.nn.model import packed_ctx
    dev = torch.device("cuda", 0)
    arch = PRESETS[preset]()
    m = CausalLM(arch, dtype=torch.bfloat16, device=dev).init_weights(2)
    lens = [37, 5, 64]
    toks = torch.randint(0, arch.vocab_size - 1, (sum(lens),), device=dev)
    with torch.no_grad():
        ctx0, _ = packed_ctx(lens, dev)
        h0 = m.hidden_states(toks, ctx0)
        ctx1, _ = packed_ctx(lens, dev, fuse_add_norm=True)
        h1 = m.hidden_states(toks, ctx1)
    assert ctx1.pending is None
    assert torch.allclose(h1.float(), h0.float(), rtol=3e-2, atol=3e-2)
