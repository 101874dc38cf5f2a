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
    """Small-M problems take the split-K path (fp32 partial planes in a workspace, added in slice order by the
    finalize kernel): two calls in a row must agree bit for bit with each other and, within bf16 rounding,
    with fp32."""
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
    assert torch.equal(c1, c2), "the plane sum must not depend on which CTA finishes last"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 264, 136), (2048, 4096, 6144), (100, 1024, 4096),
                                    (4096, 4096, 12288)])
def test_gemm_nn_input_gradient_layout(native, M, N, K):
    """C[M, N] = A[M, K] B[K, N] with B row-major (dx = dy W): B is fetched as MN-major tiles."""
    torch.manual_seed(12)
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(K, N, device=DEV) * 0.5).bfloat16()
    c = native.gemm_nn(a, b)
    torch.cuda.synchronize()
    assert native.C.gemm_last_status() == 0
    _close(c, a.float() @ b.float(), 2e-2, 2e-2 * K ** 0.5 * 0.25)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 200), (264, 136, 300), (4096, 6144, 2048), (1024, 4096, 100),
                                    (4096, 12288, 4097)])
def test_gemm_tn_weight_gradient_layout(native, M, N, K):
    """C[M, N] = A[K, M]^T B[K, N] (dW = dy^T x): both operands MN-major; bf16 result, fp32 result, and
    accumulation into an fp32 buffer twice in a row (beta = 1 epilogue)."""
    torch.manual_seed(13)
    a = (torch.randn(K, M, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(K, N, device=DEV) * 0.5).bfloat16()
    ref = a.float().t() @ b.float()
    c = native.gemm_tn(a, b)
    _close(c, ref, 2e-2, 2e-2 * K ** 0.5 * 0.25)
    acc = torch.ones(M, N, device=DEV)
    native.gemm_tn(a, b, out=acc, accumulate=True)
    native.gemm_tn(a, b, out=acc, accumulate=True)
    torch.cuda.synchronize()
    assert native.C.gemm_last_status() == 0
    _close(acc, 1.0 + 2.0 * ref, 1e-3, 1e-3 * K ** 0.5)
    plain = torch.full((M, N), float("nan"), device=DEV)
    native.gemm_tn(a, b, out=plain)
    _close(plain, ref, 1e-3, 1e-3 * K ** 0.5 * 0.25)


def test_linear_backward_runs_on_the_kernel_and_accumulates_into_main_grad(native):
    """dx and dW of the linear op against fp32 autograd; a parameter with an fp32 ``main_grad`` buffer
    receives its gradient there (added by the GEMM epilogue) and none through autograd."""
    torch.manual_seed(14)
    T, K, N = 520, 512, 768
    x = (torch.randn(T, K, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(N, K, device=DEV) * 0.1).bfloat16().requires_grad_(True)
    dy = (torch.randn(T, N, device=DEV) * 0.5).bfloat16()
    before = dict(native.library_counts)
    y = native.linear(x, w)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (xr @ wr.t()).backward(dy.float())
    _close(x.grad, xr.grad, 2e-2, 2e-2 * N ** 0.5 * 0.1)
    _close(w.grad, wr.grad, 2e-2, 2e-2 * T ** 0.5 * 0.25)
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.zeros(N, K, device=DEV)
    for _ in range(2):
        native.linear(x.detach(), w2).backward(dy)
    assert w2.grad is None
    _close(w2.main_grad, 2.0 * wr.grad, 1e-3, 1e-3 * T ** 0.5)
    assert dict(native.library_counts) == before, "the backward must not fall back to a library GEMM"
    assert native.C.gemm_last_status() == 0
