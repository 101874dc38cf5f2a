"""tcgen05/TMEM GEMM against an fp32 matmul.  Needs a B200."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def native():
    from chatlearn_b200.ops import native as n
    return n


def _close(a, b, rtol, atol):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.allclose(a, b, rtol=rtol, atol=atol), f"max abs diff {(a - b).abs().max().item():.3e}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 264, 136), (4096, 4096, 4096),
                                    (128, 6144, 4096), (16, 4096, 12288), (100, 24576, 4096)])
@pytest.mark.parametrize("out_fp32", [False, True])
def test_gemm_tcgen05(native, M, N, K, out_fp32):
    torch.manual_seed(9)
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
    c = native.gemm_nt(a, b, out_fp32)
    torch.cuda.synchronize()
    assert native.C.gemm_last_status() == 0, "a bounded wait inside the GEMM kernel timed out"
    c_ref = a.float() @ b.float().t()
    tol = 1e-3 if out_fp32 else 2e-2
    _close(c, c_ref, tol, tol * K ** 0.5 * 0.25)


def test_gemm_splitk_is_deterministic_in_shape(native):
    """Small-M problems take the split-K path (fp32 partial sums in a workspace that the
    finalize kernel clears): two calls in a row must agree with each other and with fp32."""
    torch.manual_seed(11)
    a = (torch.randn(64, 4096, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(4096, 4096, device=DEV) * 0.5).bfloat16()
    c1 = native.gemm_nt(a, b, True)
    c2 = native.gemm_nt(a, b, True)
    torch.cuda.synchronize()
    assert native.C.gemm_last_status() == 0
    ref = a.float() @ b.float().t()
    _close(c1, ref, 1e-3, 2e-2)
    _close(c2, ref, 1e-3, 2e-2)
