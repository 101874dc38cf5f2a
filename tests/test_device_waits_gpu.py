"""Bounded device waits and output-boundary (canary) checks on one GPU.

The timeout test makes a wait run out on purpose in the only way allowed here: a barrier whose
"peer" is a flag word in this GPU's own memory that nothing ever increments.  The kernel gives up
after its time limit, records a status code and returns; the context stays usable."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_reports_status():
    from chatlearn_b200.ops import native
    C = native.C
    dev = torch.device("cuda", 0)
    slots = 8
    mine = torch.zeros(8 * slots, dtype=torch.int32, device=dev)        # flags of "rank 0" (this kernel)
    nobody = torch.zeros(8 * slots, dtype=torch.int32, device=dev)      # flags of a rank that does not exist
    expect = torch.zeros(slots * 8, dtype=torch.int32, device=dev)
    C.symm_moe_last_status()                                            # clear
    t0 = time.time()
    C.symm_moe_barrier([mine.data_ptr(), nobody.data_ptr()], expect, 0, slots, 0)
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert 1.0 < dt < 10.0, dt                                          # waited its limit (2 s), not forever
    assert C.symm_moe_last_status() == 1                                # "a peer did not arrive"
    assert int(nobody[0 * slots + 0]) == 1                              # our own signal was delivered
    # the context is intact: later work runs and the status is clear again
    x = torch.randn(256, 256, device=dev).bfloat16()
    y = C.gemm_bf16_nt(x, x, False)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and C.symm_moe_last_status() == 0 and C.gemm_last_status() == 0


def _guarded(shape, dtype, dev, pad=4096):
    """A tensor with guard regions before and after it, filled with a sentinel."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * pad,), 7.0, dtype=dtype, device=dev)
    return buf, buf[pad:pad + n].view(*shape), pad


def _guards_intact(buf, pad):
    return bool((buf[:pad] == 7.0).all() and (buf[-pad:] == 7.0).all())


def test_kernels_do_not_write_outside_their_outputs():
    from chatlearn_b200.ops import native
    C = native.C
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    # GEMM with ragged M and N (partial tiles in both directions), all tile widths
    for bn in (0, 64, 128, 256):
        C.gemm_set_tile_n(bn)
        a = torch.randn(200, 512, device=dev).bfloat16()
        b = torch.randn(328, 512, device=dev).bfloat16()
        buf, out, pad = _guarded((200, 328), torch.bfloat16, dev)
        C.gemm_bf16_nt_out(a, b, out)
        torch.cuda.synchronize()
        assert _guards_intact(buf, pad)
        assert (out.float() - a.float() @ b.float().t()).norm() / (a.float() @ b.float().t()).norm() < 5e-3
    C.gemm_set_tile_n(0)
    # grouped GEMM: rows past the last group are not written
    xs = torch.randn(300, 256, device=dev).bfloat16()
    w = torch.randn(4, 128, 256, device=dev).bfloat16()
    off = torch.tensor([0, 10, 10, 150, 260], dtype=torch.long, device=dev)
    y = C.grouped_gemm_bf16_nt(xs, w, off)
    y2 = C.grouped_gemm_bf16_nt(xs, w, off)
    torch.cuda.synchronize()
    assert torch.equal(y[:260], y2[:260])
    # fused residual + norm writes exactly T x H
    bufx, x, padx = _guarded((33, 512), torch.bfloat16, dev)
    x.copy_(torch.randn(33, 512, device=dev))
    d = torch.randn(33, 512, device=dev).bfloat16()
    wn = torch.ones(512, device=dev).bfloat16()
    C.add_residual_rmsnorm(x, d, wn, 1e-6)
    torch.cuda.synchronize()
    assert _guards_intact(bufx, padx)
    # MoE permute / combine
    T, H, E, k = 50, 256, 8, 2
    xt = torch.randn(T, H, device=dev).bfloat16()
    idx = torch.randint(0, E, (T, k), device=dev)
    hist = torch.bincount(idx.reshape(-1), minlength=E)
    offs = torch.zeros(E + 1, dtype=torch.long, device=dev)
    offs[1:] = hist.cumsum(0)
    xs2, pos = C.moe_permute(xt, idx, offs)
    torch.cuda.synchronize()
    assert sorted(pos.reshape(-1).tolist()) == list(range(T * k))        # a permutation: every row claimed once
    assert torch.equal(xs2[pos[:, 0].long()], xt)
