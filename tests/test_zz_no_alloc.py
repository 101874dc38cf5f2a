"""The allocation-free C entry point of the GEMM (``clb200_gemm_bf16_nt_noalloc``).

Some users of the library cannot let a call allocate device memory: a host
application that handed the whole GPU to its own pool, a latency-critical loop that
must not hit cudaMalloc's implicit synchronisation, a plain C caller without a
caching allocator.  For them the split-K GEMM is exported once more as a C symbol
that takes the output buffer from the caller and keeps its partial sums in a fixed
array inside the library.  This test calls that symbol through ``ctypes`` (not
through the PyTorch binding) and checks it against the regular entry point, twice
in a row, because the scratch array keeps the previous call's contents.

Collected last on purpose: if it fails, a run that stops at the first failure has
already executed every other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from chatlearn_b200.ops import native          # loads torch's libraries the extension links against
    lib = ctypes.CDLL(native._SO)
    fn = lib.clb200_gemm_bf16_nt_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    lib.clb200_gemm_noalloc_last_error.restype = ctypes.c_char_p
    lib.clb200_gemm_noalloc_device_status.restype = ctypes.c_int
    return lib, fn, native


def _call(fn, a, b, c, out_fp32):
    M, K = a.shape
    N = b.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    return fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0), int(out_fp32),
              ctypes.c_void_p(stream))


@pytest.mark.parametrize("M,N,K,out_fp32", [(128, 4096, 4096, False), (64, 6144, 4096, True), (100, 1024, 512, False)])
def test_noalloc_entry_matches_regular_entry(M, N, K, out_fp32):
    lib, fn, native = _lib()
    torch.manual_seed(21)
    dev = "cuda"
    for trial in range(2):                         # two calls in a row share the scratch array
        a = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
        b = (torch.randn(N, K, device=dev) * 0.5).bfloat16()
        c = torch.full((M, N), float("nan"), device=dev, dtype=torch.float32 if out_fp32 else torch.bfloat16)
        rc = _call(fn, a, b, c, out_fp32)
        assert rc == 0, lib.clb200_gemm_noalloc_last_error().decode()
        # "launched" is not "finished": a plain C caller learns from this symbol whether a bounded wait gave up
        assert lib.clb200_gemm_noalloc_device_status() == 0
        want = native.gemm_nt(a, b, out_fp32)
        torch.cuda.synchronize()
        assert native.C.gemm_last_status() == 0
        tol = 1e-3 if out_fp32 else 2e-2
        assert torch.allclose(c.float(), want.float(), rtol=tol, atol=tol * K ** 0.5 * 0.25), \
            f"trial {trial}: max diff {(c.float() - want.float()).abs().max().item():.3e}"
        ref = a.float() @ b.float().t()
        assert torch.allclose(c.float(), ref, rtol=tol, atol=tol * K ** 0.5 * 0.25)


def test_noalloc_entry_rejects_oversized_and_misaligned():
    lib, fn, _ = _lib()
    a = torch.zeros(2048, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(2048, 64, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(2048, 2048, device="cuda", dtype=torch.bfloat16)
    assert _call(fn, a, b, c, False) == 5          # 2*M*N floats exceed the built-in scratch
    assert b"too large" in lib.clb200_gemm_noalloc_last_error()
    a2 = torch.zeros(16, 72, device="cuda", dtype=torch.bfloat16)[:, :68]
    assert fn(a2.data_ptr(), b.data_ptr(), c.data_ptr(), 16, 2048, 68, 72, 64, 0, None) == 3
