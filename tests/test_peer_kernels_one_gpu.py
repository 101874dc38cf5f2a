"""The peer-memory kernels on ONE GPU: the ranks of a group are emulated by distinct buffers on the same device.

Every kernel that reads or writes a peer takes a table of per-rank base pointers; here the table points at
ordinary tensors of the one device, one per emulated rank, and the kernel of each "rank" is launched in turn.
The kernels' flag barriers exist to order one rank's loads after its peers' stores; in this emulation all
inputs are in place before the first launch, so the flag words are pre-set to a count that every wait already
finds reached: no launch ever waits for another launch (kernels that wait on one another must not share a
GPU).  What is checked is the data path: pointer tables, offsets, the reduction order and the arithmetic,
against fp32 PyTorch statements.  The synchronisation itself is exercised by the two-GPU tests.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
W = 4
SLOTS = 1024
DEV = "cuda"


@pytest.fixture(scope="module")
def native():
    from chatlearn_b200.ops import native as n
    return n


def _flags(world=W, slots=SLOTS):
    """Per-rank flag arrays whose counters are already far ahead of any round the kernels will wait for."""
    flags = [torch.full((8 * slots,), 1 << 20, dtype=torch.int32, device=DEV) for _ in range(world)]
    expect = [torch.zeros(slots * 8, dtype=torch.int32, device=DEV) for _ in range(world)]
    return flags, [f.data_ptr() for f in flags], expect


def test_oneshot_allreduce_every_rank_gets_the_same_sum(native):
    torch.manual_seed(0)
    flags, fptr, expect = _flags()
    for n in (8, 4096 * 128, 4096 * 64 + 24):
        bufs = [torch.randn(n, device=DEV).bfloat16() for _ in range(W)]
        want = sum(b.float() for b in bufs)
        outs = []
        for r in range(W):
            out = torch.empty(n, device=DEV, dtype=torch.bfloat16)
            native.C.symm_allreduce([b.data_ptr() for b in bufs], fptr, expect[r], out, n, r, SLOTS)
            outs.append(out)
        torch.cuda.synchronize()
        assert native.C.symm_last_status() == 0
        for o in outs:
            assert torch.allclose(o.float(), want, rtol=2e-2, atol=2e-2)
            assert torch.equal(o, outs[0])              # fixed summation order: bit-identical on every rank


def test_allreduce_residual_rmsnorm(native):
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(1)
    flags, fptr, expect = _flags()
    T, H = 77, 4096
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    parts = [(0.5 * torch.randn(T, H, device=DEV)).bfloat16() for _ in range(W)]
    resid0 = torch.randn(T, H, device=DEV).bfloat16()
    want_res = (sum(p.float() for p in parts) + resid0.float()).bfloat16()
    for r in range(W):
        resid = resid0.clone()
        h = native.C.symm_ar_residual_rmsnorm([p.data_ptr() for p in parts], fptr, expect[r], resid, w, 1e-6, r, SLOTS)
        torch.cuda.synchronize()
        assert torch.allclose(resid.float(), want_res.float(), rtol=2e-2, atol=2e-2)
        assert torch.allclose(h.float(), ref.rmsnorm(resid, w, 1e-6).float(), rtol=2e-2, atol=2e-2)
    assert native.C.symm_last_status() == 0


def test_pull_reduce_scatter_then_adamw_with_pushed_all_gather(native):
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(2)
    flags, fptr, expect = _flags()
    N = 1 << 18
    shard = N // W
    grads = [torch.randn(N, device=DEV) for _ in range(W)]
    full0 = torch.randn(N, device=DEV)
    params = [full0.bfloat16().clone() for _ in range(W)]                    # every rank's copy of the parameters
    want_g = sum(grads)
    shards, sq = [], torch.zeros((), device=DEV)
    for r in range(W):
        g = torch.empty(shard, device=DEV)
        part = native.C.symm_rs_pull_sumsq([x.data_ptr() for x in grads], fptr, expect[r], g, r * shard, r, SLOTS)
        shards.append(g)
        sq = sq + part.sum()
    torch.cuda.synchronize()
    for r in range(W):
        assert torch.allclose(shards[r], want_g[r * shard:(r + 1) * shard], rtol=1e-5, atol=1e-5)
    assert torch.allclose(sq, want_g.pow(2).sum(), rtol=1e-4)
    scale = torch.clamp(1.0 / (sq.sqrt() + 1e-6), max=1.0).reshape(1)
    want_param = torch.empty(N, device=DEV, dtype=torch.bfloat16)
    for r in range(W):
        lo = r * shard
        master = full0[lo:lo + shard].clone()
        m, v = torch.zeros(shard, device=DEV), torch.zeros(shard, device=DEV)
        mr, m_r, v_r = master.clone(), m.clone(), v.clone()
        native.C.symm_adamw_push(master, shards[r], m, v, [p.data_ptr() for p in params], fptr, expect[r], lo, True, 1,
                                 1e-2, 0.9, 0.95, 1e-8, 0.01, scale, r, SLOTS)
        ref.adamw_step(mr, want_g[lo:lo + shard], m_r, v_r, want_param[lo:lo + shard], 1, 1e-2, 0.9, 0.95, 1e-8, 0.01, scale)
        torch.cuda.synchronize()
        assert torch.allclose(master, mr, rtol=1e-4, atol=1e-5)
    for p in params:                                                          # the push reached every rank's buffer
        assert (p.float() - want_param.float()).abs().max() < 1e-2
        assert torch.equal(p, params[0])
    assert native.C.symm_last_status() == 0


@pytest.mark.parametrize("all_to_all", [False, True])
def test_push_chunks_all_gather_and_all_to_all(native, all_to_all):
    torch.manual_seed(3)
    flags, fptr, expect = _flags()
    chunk = 4096 * 16                                                         # bytes per chunk
    n = chunk // 2
    srcs = [torch.randn(n * (W if all_to_all else 1), device=DEV).bfloat16() for _ in range(W)]
    recv = [torch.zeros(W * chunk, dtype=torch.uint8, device=DEV) for _ in range(W)]
    for r in range(W):
        native.C.symm_push_chunks(srcs[r], [x.data_ptr() for x in recv], chunk, all_to_all, r)
        native.C.symm_group_barrier(fptr, expect[r], SLOTS - 1, SLOTS, r)
    torch.cuda.synchronize()
    for r in range(W):
        got = recv[r].view(torch.bfloat16).view(W, n)
        for s in range(W):
            want = srcs[s][r * n:(r + 1) * n] if all_to_all else srcs[s]
            assert torch.equal(got[s], want)
    assert native.C.symm_last_status() == 0


def test_expert_parallel_dispatch_gemm_combine(native):
    """Two emulated expert-parallel ranks: remote-atomic dispatch into the owners' regions, grouped tcgen05 GEMMs
    over the occupied rows, pull combine."""
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(4)
    world, E, H, F, k, T = 2, 8, 256, 128, 2, 150
    El = E // world
    cap = 256
    rows = El * cap
    w13 = (torch.randn(E, 2 * F, H, device=DEV) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, F, device=DEV) * 0.05).bfloat16()
    xs = [torch.randn(T, H, device=DEV).bfloat16() for _ in range(world)]
    routed = [ref.moe_router(torch.randn(T, E, device=DEV), k) for _ in range(world)]
    recv_x = [torch.zeros(rows * H, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    recv_y = [torch.zeros(rows * H, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    cursor = [torch.zeros(max(El, 4), dtype=torch.int32, device=DEV) for _ in range(world)]
    where = [native.C.symm_moe_dispatch(xs[r], routed[r][1].contiguous(), [t.data_ptr() for t in recv_x],
                                        [c.data_ptr() for c in cursor], El, cap) for r in range(world)]
    for r in range(world):
        table, count = native.C.symm_moe_region_table(cursor[r][:El], cap, 2 * F)
        h13 = torch.empty(rows, 2 * F, dtype=torch.bfloat16, device=DEV)
        act = torch.empty(rows, F, dtype=torch.bfloat16, device=DEV)
        native.C.grouped_gemm_bf16_nt_table(recv_x[r].view(rows, H), w13[r * El:(r + 1) * El].contiguous(), table, count, h13)
        native.C.symm_moe_swiglu(h13, act, table, count)
        table2, count2 = native.C.symm_moe_region_table(cursor[r][:El], cap, H)
        native.C.grouped_gemm_bf16_nt_table(act, w2[r * El:(r + 1) * El].contiguous(), table2, count2, recv_y[r].view(rows, H))
    for r in range(world):
        got = native.C.symm_moe_combine([t.data_ptr() for t in recv_y], where[r], routed[r][0].float(), H, rows)
        want = ref.moe_experts(xs[r].float(), w13.float(), w2.float(), routed[r][0], routed[r][1])
        torch.cuda.synchronize()
        rel = float((got.float() - want).norm() / want.norm())
        assert rel < 2e-2, rel
    assert native.C.symm_moe_last_status() == 0 and native.C.gemm_last_status() == 0


def test_weight_sync_pulls_remote_shards_into_the_rollout_layout(native):
    """Trainer shards (fp32, 1/W of every block per emulated rank) are pulled into a tensor-parallel rollout
    layout (bf16): most descriptors of a destination rank name another rank's buffer."""
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.synchronizer.kernel_executor import KernelExecutor
    from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
    from chatlearn_b200.synchronizer.plan import build_plan, validate_plan
    world = 2
    arch = PRESETS["tiny_qwen3"]()
    full = CausalLM(arch, dtype=torch.float32, device=DEV, pad_to=world).init_weights(3)
    shards = {b.name: b.numel // world for b in full.blocks}
    src_bufs = [{f"s/{b.name}": b.flat[r * shards[b.name]:(r + 1) * shards[b.name]].clone() for b in full.blocks}
                for r in range(world)]
    src_lays = [layout_of_model(full, r, lambda name, r=r: (r * shards[name], (r + 1) * shards[name]), "s/") for r in range(world)]
    dst_lays = [layout_of_model(CausalLM(arch, dtype=torch.bfloat16, device="meta", tp=world, tp_rank=r, allocate=False), r,
                                prefix="d/") for r in range(world)]
    plan = build_plan(src_lays, dst_lays)
    validate_plan(plan, dst_lays)

    class Emulated(KernelExecutor):
        def _peer_ptr(self, bufs, name, src_rank):          # the "peer" is another tensor of this device
            return src_bufs[src_rank][name].data_ptr()

    for r in range(world):
        dst = CausalLM(arch, dtype=torch.bfloat16, device=DEV, tp=world, tp_rank=r)
        want = CausalLM(arch, dtype=torch.bfloat16, device=DEV, tp=world, tp_rank=r)
        want.load_hf_state_dict(full.hf_state_dict())
        ex = Emulated(plan, r, world)
        assert sum(1 for d in ex.descs if d.src_rank != r) > 0
        ex.needs_peers = False                               # no process group here: nothing to order
        ex.run(src_bufs[r], {f"d/{b.name}": b.flat for b in dst.blocks})
        torch.cuda.synchronize()
        assert all(torch.equal(a.flat, b.flat) for a, b in zip(dst.blocks, want.blocks))
