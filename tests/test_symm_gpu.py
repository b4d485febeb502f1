"""Symmetric-memory kernels: one-GPU emulation (all "ranks" are buffers of one device; these kernels
never wait on one another), the bounded barrier wait, and the real 2-GPU paths over NVLink."""
import ctypes as C

import pytest
import torch

from tests.dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_reduce_scatter_sumsq_emulated():
    from cverl_b200 import _native as nv
    world, n_full = 4, 4 * 50_000
    g = torch.Generator(device="cuda").manual_seed(0)
    grads = [torch.randn(n_full, device="cuda", generator=g) for _ in range(world)]
    shard = n_full // world
    for rank in range(world):
        out = torch.empty(shard, device="cuda")
        sq = torch.zeros(1, device="cuda")
        nv.check(nv.cuda().cvb_reduce_scatter_sumsq(_ptrs(grads), world, rank, rank * shard, shard, 1.0 / world,
                                                    out.data_ptr(), sq.data_ptr(), nv.stream()), "rs")
        ref = torch.stack([x[rank * shard:(rank + 1) * shard] for x in grads]).double().mean(0)
        torch.testing.assert_close(out.double(), ref, rtol=1e-6, atol=1e-6)
        assert abs(sq.item() - ref.pow(2).sum().item()) < 1e-4 * ref.pow(2).sum().item()


@pytest.mark.parametrize("master", [True, False])
def test_adamw_allgather_emulated(master):
    from cverl_b200 import _native as nv
    from cverl_b200.ops import optim as optim_ops
    world, shard = 2, 40_000
    g = torch.Generator(device="cuda").manual_seed(1)
    full0 = torch.randn(world * shard, device="cuda", generator=g).bfloat16()
    bufs = [full0.clone() for _ in range(world)]
    ref_full = full0.clone()
    clip = torch.tensor([0.5], device="cuda")
    for rank in range(world):
        sl = slice(rank * shard, (rank + 1) * shard)
        grad = torch.randn(shard, device="cuda", generator=g)
        m, v = torch.rand(shard, device="cuda", generator=g), torch.rand(shard, device="cuda", generator=g)
        mst = full0[sl].float() if master else None
        m2, v2 = m.clone(), v.clone()
        mst2 = mst.clone() if master else None
        optim_ops.flat_adamw_step(grad.clone(), mst2, ref_full[sl], m2, v2, clip=clip, grad_scale=1.0, lr=1e-2,
                                  beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=3, zero_grad=False)
        nv.check(nv.cuda().cvb_flat_adamw_allgather(grad.data_ptr(), nv.ptr(mst), m.data_ptr(), v.data_ptr(),
                                                    clip.data_ptr(), _ptrs(bufs), world, rank, rank * shard, shard,
                                                    1e-2, 0.9, 0.95, 1e-8, 0.01, 3, nv.stream()), "adam")
        torch.testing.assert_close(m, m2)
        torch.testing.assert_close(v, v2)
        if master:
            torch.testing.assert_close(mst, mst2)
    for b in bufs:
        torch.testing.assert_close(b.float(), ref_full.float(), rtol=8e-3, atol=1e-6)


def test_broadcast_store_emulated():
    from cverl_b200 import _native as nv
    src = torch.randn(1 << 20, device="cuda").bfloat16()
    dst = [torch.zeros_like(src) for _ in range(3)]
    nv.check(nv.cuda().cvb_broadcast_store(src.data_ptr(), _ptrs(dst), 3, src.numel() * 2, nv.stream()), "bcast")
    for d in dst:
        assert torch.equal(d, src)


def test_p2p_rows_skip_entries_outside_the_group_or_the_buffer():
    """Row scatter / gather with two "ranks" that are buffers of one device: an entry whose rank is not in the
    group (2 of a world of 2, although the pointer table has 8 slots) or whose row is past the buffer is skipped
    and reported through the status word; rank -1 is left out silently; the good entries move."""
    from cverl_b200 import _native as nv
    cap, hidden = 8, 64
    bufs = [torch.zeros(cap, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    rows = torch.arange(5 * hidden, device="cuda", dtype=torch.float32).view(5, hidden).bfloat16()
    st = nv.status_word()
    st.zero_()
    prank = torch.tensor([0, 1, 2, 1, -1], dtype=torch.int32, device="cuda")      # 2: outside the group
    prow = torch.tensor([3, 7, 0, 8, 0], dtype=torch.int64, device="cuda")        # 8: past the 8-row buffer
    nv.check(nv.cuda().cvb_p2p_scatter_rows(rows.data_ptr(), _ptrs(bufs), 2, prank.data_ptr(), prow.data_ptr(), 5,
                                            hidden * 2, cap, st.data_ptr(), nv.stream()), "scatter")
    torch.cuda.synchronize()
    assert torch.equal(bufs[0][3], rows[0]) and torch.equal(bufs[1][7], rows[1])
    assert int((bufs[0] != 0).any(1).sum()) == 1 and int((bufs[1] != 0).any(1).sum()) == 1   # nothing else written
    with pytest.raises(RuntimeError, match="status 7"):
        nv.check_status()
    # gather the two good rows back; no status this time
    back = torch.zeros(2, hidden, device="cuda", dtype=torch.bfloat16)
    nv.check(nv.cuda().cvb_p2p_gather_rows(back.data_ptr(), _ptrs(bufs), 2, prank[:2].contiguous().data_ptr(),
                                           prow[:2].contiguous().data_ptr(), 2, hidden * 2, cap, st.data_ptr(),
                                           nv.stream()), "gather")
    torch.cuda.synchronize()
    assert torch.equal(back, rows[:2]) and nv.check_status() == 0


def test_gemm_reduce_scatter_epilogue_emulated():
    """GEMM whose epilogue sends every row block only to its owner: two "ranks" on one device, each writing its
    partial product into slot ``rank`` of both owners' buffers; the owners' slot sums equal the fp32 product."""
    from cverl_b200 import _native as nv
    from cverl_b200.ops import gemm as G
    M, N, K, world = 1024, 256, 384, 2
    rl = M // world
    g = torch.Generator(device="cuda").manual_seed(4)
    xs = [torch.randn(M, K, device="cuda", generator=g).bfloat16() for _ in range(world)]
    ws = [(0.05 * torch.randn(N, K, device="cuda", generator=g)).bfloat16() for _ in range(world)]
    owners = [torch.zeros(world, rl, N, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    for me in range(world):
        bases = [owners[o].data_ptr() + (me * rl - o * rl) * N * 2 for o in range(world)]
        G.gemm_raw(xs[me], ws[me], None, M, N, K, a_mn=False, b_mn=False, epi=nv.EPI_STORE_BF16,
                   block_n=G._pick_block_n(M, N), scatter=(bases, rl), ldc=N)
    torch.cuda.synchronize()
    nv.check_status()
    ref = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for o in range(world):
        for me in range(world):
            part = xs[me].float() @ ws[me].float().t()
            torch.testing.assert_close(owners[o][me].float(), part[o * rl:(o + 1) * rl], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(owners[o].float().sum(0), ref[o * rl:(o + 1) * rl], rtol=2e-2, atol=4e-2)


def test_sequence_parallel_norm_kernels_emulated():
    """``sp_add_rmsnorm`` forward / backward against the fp32 statement: the inputs are ``n`` partial slots, the
    outputs go to row ``dst_row0`` of several gathered buffers (here all on one device)."""
    from cverl_b200 import _native as nv
    from cverl_b200.ops.norm import rmsnorm_ref
    world, rl, H, rank = 2, 384, 1024, 1
    g = torch.Generator(device="cuda").manual_seed(8)
    parts = torch.randn(world, rl, H, device="cuda", generator=g).bfloat16()
    resid = torch.randn(rl, H, device="cuda", generator=g).bfloat16()
    w = (0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    gathered = [torch.zeros(world * rl, H, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    resid_out = torch.empty(rl, H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.empty(rl, device="cuda")
    nv.check(nv.cuda().cvb_sp_add_rmsnorm_fwd(parts.data_ptr(), rl * H, world, resid.data_ptr(), w.data_ptr(),
                                              _ptrs(gathered), world, rank * rl, resid_out.data_ptr(),
                                              rstd.data_ptr(), rl, H, 1e-6, 1.0, nv.stream()), "sp fwd")
    torch.cuda.synchronize()
    hsum = (parts.float().sum(0) + resid.float()).requires_grad_(True)
    torch.testing.assert_close(resid_out.float(), hsum.detach(), rtol=1e-2, atol=1e-2)
    y_ref = rmsnorm_ref(resid_out.float().requires_grad_(False), w, 1e-6, 1.0)
    for buf in gathered:
        torch.testing.assert_close(buf[rank * rl:(rank + 1) * rl].float(), y_ref.float(), rtol=2e-2, atol=2e-2)
        assert float(buf[:rank * rl].abs().sum()) == 0.0                      # other ranks' rows untouched
    # backward: dy arrives as n partial slots, dres as a local tensor
    dy_parts = torch.randn(world, rl, H, device="cuda", generator=g).bfloat16()
    dres = torch.randn(rl, H, device="cuda", generator=g).bfloat16()
    dx = torch.empty(rl, H, device="cuda", dtype=torch.bfloat16)
    dxg = [torch.zeros(world * rl, H, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    dw = torch.zeros(H, device="cuda")
    nv.check(nv.cuda().cvb_sp_add_rmsnorm_bwd(dy_parts.data_ptr(), rl * H, world, resid_out.data_ptr(), w.data_ptr(),
                                              rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), _ptrs(dxg), world,
                                              rank * rl, dw.data_ptr(), rl, H, 1.0, nv.stream()), "sp bwd")
    torch.cuda.synchronize()
    h = resid_out.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    xf = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * (1.0 + wf)
    xf.backward(dy_parts.float().sum(0))
    torch.testing.assert_close(dx.float(), h.grad + dres.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(dw, wf.grad, rtol=2e-2, atol=0.5)
    for buf in dxg:
        assert torch.equal(buf[rank * rl:(rank + 1) * rl], dx)


def test_barrier_wait_runs_out_to_status():
    """A flag that nothing sets: the wait gives up within its clock budget, the kernel returns and the
    host reads the status word; the context stays usable."""
    from cverl_b200 import _native as nv
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    other = torch.zeros(8, dtype=torch.int32, device="cuda")     # stands for a silent peer's flag array
    st = nv.status_word()
    st.zero_()
    nv.check(nv.cuda().cvb_symm_barrier(_ptrs([flags, other]), 0, 2, 1, st.data_ptr(), nv.stream()), "barrier")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 5"):
        nv.check_status()
    assert int(other[0].item()) == 1 and int(flags[0].item()) == 1 and int(flags[1].item()) == 0
    assert int(st.item()) == 0                                     # cleared by the host read
    x = torch.ones(4, device="cuda") * 2                           # context still works
    assert float(x.sum().item()) == 8.0


def _fused_zero_rank(rank, world):
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.models.params import FlatParams
    from cverl_b200.optim.adamw import AdamWOptions
    from cverl_b200.parallel.symm import FusedZeroComm, P2pBroadcaster, SymmetricHeap
    from cverl_b200.parallel.zero import FlatZeroOptimizer
    dev = torch.device("cuda", rank)
    heap = SymmetricHeap(None, dev)
    fc = FusedZeroComm(heap)
    entries = [("a", (1000, 64)), ("b", (64,)), ("c", (333, 8))]
    fused = FlatParams(entries, device=dev, pad_multiple=world * 8, allocator=fc.allocator)
    plain = FlatParams(entries, device=dev, pad_multiple=world * 8)
    g = torch.Generator(device=dev).manual_seed(5)
    init = torch.randn(fused.padded_numel, device=dev, generator=g).bfloat16()
    fused.flat.copy_(init)
    plain.flat.copy_(init)
    for use_master in (True,):
        opts = AdamWOptions(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, use_master_weights=use_master)
        kw = dict(dp_group=None, dp_rank=rank, dp_size=world, norm_group=None, norm_world=world, max_grad_norm=1.0)
        of = FlatZeroOptimizer(fused, opts, fused_comm=fc, **kw)
        op = FlatZeroOptimizer(plain, opts, **kw)
        gr = torch.Generator(device=dev).manual_seed(100 + rank)
        for _ in range(3):
            grad = torch.randn(fused.padded_numel, device=dev, generator=gr)
            fused.main_grad.copy_(grad)
            plain.main_grad.copy_(grad)
            of.step()
            op.step()
            torch.cuda.synchronize()
            nv.check_status()
            torch.testing.assert_close(fused.flat.float(), plain.flat.float(), rtol=8e-3, atol=1e-6)
            torch.testing.assert_close(of.last_metrics, op.last_metrics, rtol=1e-4, atol=1e-6)
            assert float(fused.main_grad.abs().sum()) == 0.0
    # weight push: rank 0 -> rank 1
    bc = P2pBroadcaster(heap, 1 << 20)
    mine = bc.tensor(1 << 19, torch.bfloat16)
    if rank == 0:
        src = torch.arange(1 << 19, device=dev).bfloat16()
        bc.push(src, [1])
    bc.sync()
    torch.cuda.synchronize()
    nv.check_status()
    if rank == 1:
        assert torch.equal(mine, torch.arange(1 << 19, device=dev).bfloat16())
    dist.barrier()
    heap.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_zero_and_push_two_gpus():
    run_ranks(_fused_zero_rank, 2, backend="nccl", timeout=300)


def _tp_symm_rank(rank, world):
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.ops import gemm as G
    from cverl_b200.parallel import tp_symm
    dev = torch.device("cuda", rank)
    tps = tp_symm.TpSymm(None, dev, max_rows=640, max_cols=256)
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    for it in range(5):                                   # more uses than buffers: exercises the alternation
        rows = 640 if it % 2 == 0 else 300
        x = torch.randn(rows, 384, device=dev, generator=g).bfloat16().requires_grad_(True)
        w_row = (0.05 * torch.randn(256, 384, device=dev, generator=g)).bfloat16().requires_grad_(True)
        y = tp_symm.row_parallel_linear(x, w_row, tps)
        ref = (x.detach().float() @ w_row.detach().float().t())
        dist.all_reduce(ref)
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
        # column parallel: replicated input, all-reduced input gradient
        xr = torch.randn(rows, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(77 + it))
        xr = xr.bfloat16().requires_grad_(True)
        w_col = (0.05 * torch.randn(384, 256, device=dev, generator=g)).bfloat16().requires_grad_(True)
        yc = tp_symm.column_parallel_linear(xr, w_col, tps)
        dy = torch.randn(yc.shape, device=dev, generator=g).bfloat16()
        yc.backward(dy)
        dref = dy.float() @ w_col.detach().float()
        dist.all_reduce(dref)
        torch.testing.assert_close(xr.grad.float(), dref, rtol=2e-2, atol=3e-2)
        torch.testing.assert_close(w_col.grad.float(), dy.float().t() @ xr.detach().float(), rtol=2e-2, atol=5e-2)
    torch.cuda.synchronize()
    nv.check_status()
    dist.barrier()
    tps.heap.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_fused_linear_two_gpus():
    run_ranks(_tp_symm_rank, 2, backend="nccl", timeout=300)


def _tp_sp_model_rank(rank, world):
    """Sequence-parallel tensor parallelism (GEMM -> reduce-scatter epilogue, norm -> all-gather stores) against
    the same model on one GPU: response log-probs and every parameter gradient."""
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.params import shard_tensor
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.parallel.mesh import build_context
    from cverl_b200.parallel.tp_sp import TpSp
    dev = torch.device("cuda", rank)
    cfg = Qwen35TextConfig(vocab_size=4096, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, intermediate_size=512, linear_key_head_dim=128,
                           linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=2)
    B, S, P = 4, 256, 64
    ctx = build_context(world, rank, tp=world, dp=1)
    ctx.tp_sp = TpSp(ctx.tp_group, dev, B * S, cfg.hidden_size, arena_slots=2 * cfg.num_hidden_layers + 1)
    tp_model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=8)
    tp_model.init_weights(seed=7)
    dense = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, pad_multiple=8)
    dense.init_weights(seed=7)
    assert tp_model.sequence_parallel and not dense.sequence_parallel
    g = torch.Generator(device=dev).manual_seed(3)
    failures = []                                          # asserted after both ranks are past every collective
    for it in range(2):                                    # twice: the arena and the double buffers are reused
        ids = torch.randint(1, cfg.vocab_size, (B, S), device=dev, generator=g)
        seed = torch.randn(B, S - P, device=dev, generator=g)
        lp = tp_model.response_logprobs(ids, P)
        lp.backward(seed)
        tp_model.sync_replicated_grads()
        lp_d = dense.response_logprobs(ids, P)
        lp_d.backward(seed)
        torch.cuda.synchronize()
        nv.check_status()
        if (lp.float() - lp_d.float()).abs().max().item() >= 0.1:
            failures.append(("log-probs", it))
        bad, err_sq, tot_sq = [], 0.0, 0.0
        pairs = []
        for spec in tp_model.specs:
            full = dense.flat.params[spec.name].main_grad
            want = shard_tensor(spec, full, rank, world).float()
            got = tp_model.flat.params[spec.name].main_grad.float()
            pairs.append((spec.name, got, want))
            err_sq += (got - want).pow(2).sum().item()
            tot_sq += want.pow(2).sum().item()
        if (err_sq / tot_sq) ** 0.5 >= 0.03:                                  # all gradients as one vector
            failures.append(("all gradients", it, (err_sq / tot_sq) ** 0.5))
        for name, got, want in pairs:
            # per tensor, for every tensor that carries more than 0.1 % of the gradient norm.  The decay-gate
            # inputs (a-projection, A_log, dt_bias) are sums with heavy cancellation: two bf16 runs that group the
            # heads differently agree less closely on them than on the rest
            if want.norm().item() < 1e-3 * tot_sq ** 0.5:
                continue
            gate = name.endswith(("in_proj_a.weight", "A_log", "dt_bias"))
            rel = ((got - want).norm() / want.norm()).item()
            if rel >= (0.5 if gate else 0.08):
                bad.append((name, round(rel, 4), round(got.norm().item(), 5), round(want.norm().item(), 5)))
        failures += bad[:12]
        tp_model.flat.main_grad.zero_()
        dense.flat.main_grad.zero_()
    dist.barrier()
    ctx.tp_sp.heap.close()
    assert not failures, failures


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_parallel_tp_model_two_gpus():
    run_ranks(_tp_sp_model_rank, 2, backend="nccl", timeout=300)


def _zero2_gpu_rank(rank, world, fused):
    """Bucketed ZeRO-2 on GPUs: per-layer gradient buckets reduced from inside the backward pass on a side stream
    (peer-memory kernels or NCCL), against a full-gradient model whose gradients are all-reduced afterwards."""
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.optim import AdamWOptions
    from cverl_b200.parallel.mesh import build_context
    from cverl_b200.parallel.symm import SymmetricHeap
    from cverl_b200.parallel.zero import FlatZeroOptimizer
    from cverl_b200.parallel.zero2 import BucketedZero2Optimizer, FusedZero2Comm
    dev = torch.device("cuda", rank)
    cfg = Qwen35TextConfig(vocab_size=4096, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=128, intermediate_size=512, linear_key_head_dim=128,
                           linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=2)
    B, S, P = 2, 256, 64
    ctx = build_context(world, rank, tp=1, dp=world)
    heap = SymmetricHeap(ctx.dp_group, dev) if fused else None
    comm = FusedZero2Comm(heap) if fused else None
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=world * 8, grad_buckets=True,
                        bucket_align=world * 8, grad_slots=2, flat_allocator=comm.allocator if comm else None)
    model.init_weights(seed=7)
    ref = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx, pad_multiple=world * 8)
    ref.init_weights(seed=7)
    opts = AdamWOptions(lr=1e-3, beta2=0.95, use_master_weights=False)
    opt = BucketedZero2Optimizer(model, opts, dp_group=ctx.dp_group, dp_rank=rank, dp_size=world, norm_group=None,
                                 norm_world=world, max_grad_norm=1.0, fused_comm=comm)
    ropt = FlatZeroOptimizer(ref.flat, opts, dp_group=ctx.dp_group, dp_rank=rank, dp_size=world, norm_group=None,
                             norm_world=world, max_grad_norm=1.0)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    failures = []
    for it in range(2):
        for mb in range(2):
            ids = torch.randint(1, cfg.vocab_size, (B, S), device=dev, generator=g)
            seed = torch.randn(B, S - P, device=dev, generator=g) * 0.5
            model.response_logprobs(ids, P).backward(seed)
            ref.response_logprobs(ids, P).backward(seed)
        for p in list(ref.flat.params.values()) + list(ref.fused.values()):   # gradients that came through autograd
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        opt.finish_backward()
        want = ref.flat.main_grad.clone()
        dist.all_reduce(want, group=ctx.dp_group)
        want /= world
        torch.cuda.synchronize()
        nv.check_status()
        err_sq = tot_sq = 0.0
        for b in model.flat.bucket_ids:
            lo, _ = model.flat.bucket_ranges[b]
            c = opt.chunk[b]
            got = opt.grad_shard[opt.piece_off[b]: opt.piece_off[b] + c]
            # the same elements in the reference layout: walk the entries of this bucket that fall into the piece
            for name, (off, n) in model.flat.offsets.items():
                a, e = max(off, lo + rank * c), min(off + n, lo + (rank + 1) * c)
                if a >= e:
                    continue
                roff = ref.flat.offsets[name][0]
                w = want[roff + (a - off): roff + (e - off)]
                gt = got[a - lo - rank * c: e - lo - rank * c]
                err_sq += (gt - w).pow(2).sum().item()
                tot_sq += w.pow(2).sum().item()
        if not (tot_sq > 0 and (err_sq / tot_sq) ** 0.5 < 1e-4):   # fp32 atomics in another order: rounding only
            failures.append(("shard gradient", it, err_sq, tot_sq))
        if any(float(buf.abs().max()) != 0.0 for buf in model.flat.grad_buffers):
            failures.append(("bucket buffers not cleared", it))
        if opt.reduced_buckets != (it + 1) * 2 * cfg.num_hidden_layers:
            failures.append(("reductions from inside backward", opt.reduced_buckets))
        opt.step()
        ropt.step()
        torch.cuda.synchronize()
        nv.check_status()
        # one AdamW step moves every element by about lr = 1e-3: a piece that missed its update or its all-gather
        # would differ by that much everywhere; elements whose near-zero gradient changed sign may differ singly
        off_cnt = tot_cnt = 0
        for name, t in model.flat.named_tensors():
            d = (t.float() - ref.flat.params[name].data.float()).abs()
            if d.max().item() > 2.5e-3 * (it + 1):
                failures.append((name, it, d.max().item()))
            off_cnt += int((d > 5e-4).sum())
            tot_cnt += d.numel()
        if off_cnt > 0.02 * tot_cnt:
            failures.append(("parameters off by a whole update", it, off_cnt, tot_cnt))
        # every rank holds the same parameters after the all-gather
        chk = model.flat.flat.float().sum().reshape(1)
        both = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(both, chk, group=ctx.dp_group)
        if any(float(x) != float(both[0]) for x in both):
            failures.append(("parameters differ between ranks", it))
        # start the next round from identical parameters again: a bf16 rounding that fell differently in the two
        # optimizers would otherwise show up, amplified by the recurrent layers, as a gradient difference
        with torch.no_grad():
            for name, t in model.flat.named_tensors():
                t.copy_(ref.flat.params[name].data)
    dist.barrier()
    torch.cuda.synchronize()
    if heap is not None:
        heap.close()
    assert not failures, failures[:10]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", [False, True])
def test_bucketed_zero2_two_gpus(fused):
    run_ranks(_zero2_gpu_rank, 2, fused, backend="nccl", timeout=300)


def _nvls_rank(rank, world):
    """NVSwitch multicast kernels (multimem.st / multimem.ld_reduce) against the library collectives."""
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.parallel import nvls
    dev = torch.device("cuda", rank)
    group = dist.group.WORLD
    try:
        bc = nvls.NvlsBroadcaster(group, dev, 1 << 22)
    except RuntimeError as exc:                       # no multicast support on this machine: nothing to test
        print(f"NVLS unavailable: {exc}")
        return
    failures = []
    g = torch.Generator(device=dev).manual_seed(5)                     # the same stream of numbers on both ranks
    src = torch.randn(1 << 20, device=dev, generator=g).bfloat16()
    dst = bc.tensor(1 << 20, torch.bfloat16, 1 << 21)
    if rank == 0:
        bc.push(src, 1 << 21)
    bc.sync()
    torch.cuda.synchronize()
    if not torch.equal(dst, src):
        failures.append("multicast store")
    if float(bc.tensor(1 << 20, torch.bfloat16, 0).abs().max()) != 0.0:
        failures.append("multicast store wrote outside its range")
    n = 1 << 20
    rs = nvls.NvlsReduceScatter(group, dev, n)
    rs.grad.copy_(torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(10 + rank)))
    shard = n // world
    got = torch.full((shard,), 0.5, device=dev)
    sq = rs.reduce(got, rank * shard, accumulate=True).clone()
    want = torch.empty(shard, device=dev)
    dist.reduce_scatter_tensor(want, rs.grad.clone(), op=dist.ReduceOp.AVG)
    torch.cuda.synchronize()
    if not torch.allclose(got, want + 0.5, rtol=1e-5, atol=1e-6):
        failures.append(("reducing load", float((got - want - 0.5).abs().max())))
    if abs(float(sq) - float((want + 0.5).pow(2).sum())) > 1e-3 * float((want + 0.5).pow(2).sum()):
        failures.append("squared norm")
    ar = nvls.NvlsAllReduce(group, dev, 40 * 1024 + 8)
    x = torch.randn(40 * 1024 + 8, device=dev, generator=torch.Generator(device=dev).manual_seed(20 + rank)).bfloat16()
    ar.data.copy_(x)
    y = ar.all_reduce().clone()
    ref = x.float()
    dist.all_reduce(ref)
    torch.cuda.synchronize()
    if not torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2):
        failures.append(("all-reduce", float((y.float() - ref).abs().max())))
    nv.check_status()
    dist.barrier()
    torch.cuda.synchronize()
    for o in (bc, rs, ar):
        o.close()
    assert not failures, failures


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_nvls_multicast_kernels_two_gpus():
    run_ranks(_nvls_rank, 2, backend="nccl", timeout=300)


def _zigzag_native_rank(rank, world):
    """Zig-zag context-parallel attention on the tcgen05 kernels (hops with unequal query / key lengths, the fp32
    merge kernel) against dense causal attention in fp32: outputs and gradients."""
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.ops.attention import causal_attention_ref
    from cverl_b200.parallel.cp_zigzag import zigzag_chunks, zigzag_ring_attention
    from cverl_b200.utils import fallbacks
    dev = torch.device("cuda", rank)
    failures = []
    for D in (128, 256):
        B, Hq, Hkv, h = 1, 4, 2, 256
        S = 2 * h * world
        g = torch.Generator(device=dev).manual_seed(3)                  # the same tensors on every rank
        q, k, v, w = (torch.randn(B, S, n, D, device=dev, generator=g).bfloat16().float() for n in (Hq, Hkv, Hkv, Hq))
        qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
        dense = causal_attention_ref(qd.reshape(B * S, Hq, D), kd.reshape(B * S, Hkv, D), vd.reshape(B * S, Hkv, D),
                                     B, S).view(B, S, Hq, D)
        (dense * w).sum().backward()
        c0, c1 = zigzag_chunks(rank, world)
        rows = torch.cat([torch.arange(c0 * h, (c0 + 1) * h), torch.arange(c1 * h, (c1 + 1) * h)]).to(dev)
        ql, kl, vl = (t[:, rows].bfloat16().requires_grad_(True) for t in (q, k, v))
        out = zigzag_ring_attention(ql, kl, vl, dist.group.WORLD, rank, world)
        (out.float() * w[:, rows]).sum().backward()
        torch.cuda.synchronize()
        nv.check_status()
        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-20)).item()
        errs = {"out": rel(out, dense.detach()[:, rows]), "dq": rel(ql.grad, qd.grad[:, rows]),
                "dk": rel(kl.grad, kd.grad[:, rows]), "dv": rel(vl.grad, vd.grad[:, rows])}
        if any(e > 2e-2 for e in errs.values()):
            failures.append((D, errs))
    if fallbacks.total() != 0:
        failures.append(("library fallbacks", fallbacks.total()))
    dist.barrier()
    assert not failures, failures


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_zigzag_ring_attention_native_two_gpus():
    run_ranks(_zigzag_native_rank, 2, backend="nccl", timeout=300)


def _ring_native_rank(rank, world, pull=False):
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.ops import attention
    from cverl_b200.parallel.context_parallel import ring_attention
    dev = torch.device("cuda", rank)
    B, S, Hq, Hkv, D = 2, 256 * world, 4, 2, 128
    L = S // world
    g = torch.Generator(device=dev).manual_seed(21)           # same full tensors on every rank
    qf = torch.randn(B, Hq, S, D, device=dev, generator=g).bfloat16()
    kf = torch.randn(B, Hkv, S, D, device=dev, generator=g).bfloat16()
    vf = torch.randn(B, Hkv, S, D, device=dev, generator=g).bfloat16()
    wf = torch.randn(B, Hq, S, D, device=dev, generator=g).bfloat16()
    sl = slice(rank * L, (rank + 1) * L)
    q, k, v = (t[:, :, sl].contiguous().requires_grad_(True) for t in (qf, kf, vf))
    symm = None
    if pull:
        from cverl_b200.parallel.cp_symm import CpSymm
        symm = CpSymm(dist.group.WORLD, dev)
    out = ring_attention(q, k, v, dist.group.WORLD, rank, world, S, symm=symm, key=0)
    (out.float() * wf[:, :, sl].float()).sum().backward()
    torch.cuda.synchronize()
    nv.check_status()
    # oracle: full causal attention in fp32 on the whole sequence
    qr, kr, vr = (t.float().requires_grad_(True) for t in (qf, kf, vf))
    o_r = attention.causal_attention_ref(qr.transpose(1, 2).reshape(B * S, Hq, D), kr.transpose(1, 2).reshape(B * S, Hkv, D),
                                         vr.transpose(1, 2).reshape(B * S, Hkv, D), B, S)
    o_r = o_r.view(B, S, Hq, D).transpose(1, 2)
    (o_r * wf.float()).sum().backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(out, o_r[:, :, sl]) < 1e-2
    assert rel(q.grad, qr.grad[:, :, sl]) < 2e-2
    assert rel(k.grad, kr.grad[:, :, sl]) < 2e-2
    assert rel(v.grad, vr.grad[:, :, sl]) < 2e-2
    dist.barrier()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ring_attention_native_hops_two_gpus():
    run_ranks(_ring_native_rank, 2, backend="nccl", timeout=300)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ring_attention_peer_pull_two_gpus():
    """Same oracle, but K / V are pulled from the owner's peer-mapped buffer by the attention kernels' TMA loads
    and dK | dV come home through the staged pull-reduce."""
    run_ranks(_ring_native_rank, 2, True, backend="nccl", timeout=300)


def _ep_symm_rank(rank, world):
    """MoE layer with expert parallelism: dispatch / combine over peer memory against the NCCL all-to-all path."""
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.parallel.ep_symm import EpSymm
    from cverl_b200.parallel.mesh import build_context
    dev = torch.device("cuda", rank)
    cfg = Qwen35TextConfig.tiny(moe=True, layers=2)
    outs = []
    for mode in ("all_to_all", "symm", "symm_fused"):       # fused: the combine rides on the down projection's epilogue
        ctx = build_context(world, rank, tp=1, dp=1, ep=world)
        if mode != "all_to_all":
            ctx.ep_symm = EpSymm(ctx.ep_group, dev, capacity_rows=2 * 24 * cfg.num_experts_per_tok * world,
                                 hidden=cfg.hidden_size)
            ctx.ep_symm.fuse_combine = mode == "symm_fused"
        model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx)
        model.init_weights(seed=5)
        ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(100 + rank)).to(dev)
        for _ in range(2):                                   # twice: the return buffer is reused layer after layer
            model.flat.main_grad.zero_()
            lp = model.response_logprobs(ids, 8)
            lp.sum().backward()
        for p in list(model.flat.params.values()) + list(model.fused.values()):
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        torch.cuda.synchronize()
        nv.check_status()
        if mode != "all_to_all":
            ctx.ep_symm.check()
            assert ctx.ep_symm.fused_combines == (2 * cfg.num_hidden_layers if mode == "symm_fused" else 0)
        outs.append((lp.detach().float().clone(), model.flat.main_grad.clone()))
    (lp_a, g_a) = outs[0]
    for lp_b, g_b in outs[1:]:
        torch.testing.assert_close(lp_b, lp_a, rtol=2e-2, atol=2e-2)
        assert ((g_b - g_a).norm() / g_a.norm()).item() < 2e-2
    dist.barrier()


def _ep_overflow_rank(rank, world):
    """A receive buffer too small for the routed rows: the entries that do not fit are dropped (their outputs and
    gradients read as zeros, never as uninitialised memory), nothing is written past a buffer, and the overflow
    is reported when the trainer would read its metrics."""
    import torch.distributed as dist
    from cverl_b200 import _native as nv
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.parallel.ep_symm import EpSymm
    from cverl_b200.parallel.mesh import build_context
    dev = torch.device("cuda", rank)
    cfg = Qwen35TextConfig.tiny(moe=True, layers=2)
    ctx = build_context(world, rank, tp=1, dp=1, ep=world)
    ctx.ep_symm = EpSymm(ctx.ep_group, dev, capacity_rows=32, hidden=cfg.hidden_size)     # 96 entries are routed
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, ctx=ctx)
    model.init_weights(seed=5)
    # poison the allocator's free memory, so that an uninitialised output row would show up as NaN
    junk = torch.full((1 << 22,), float("nan"), device=dev, dtype=torch.bfloat16)
    del junk
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(100 + rank)).to(dev)
    failures = []
    for _ in range(2):
        lp = model.response_logprobs(ids, 8)
        lp.sum().backward()
        torch.cuda.synchronize()
        if not bool(torch.isfinite(lp).all()):
            failures.append("non-finite log-probs")
        if not bool(torch.isfinite(model.flat.main_grad).all()):
            failures.append("non-finite gradients")
    try:
        nv.check_status()
    except RuntimeError as exc:
        failures.append(f"status word: {exc}")
    try:
        ctx.ep_symm.check()
        failures.append("overflow not reported")
    except RuntimeError as exc:
        if "capacity" not in str(exc):
            failures.append(str(exc))
    dist.barrier()
    assert not failures, failures


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_receive_overflow_is_dropped_and_reported_two_gpus():
    run_ranks(_ep_overflow_rank, 2, backend="nccl", timeout=300)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_symm_matches_all_to_all_two_gpus():
    run_ranks(_ep_symm_rank, 2, backend="nccl", timeout=300)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("push", ["nccl", "symm", "nvls"])
def test_static_split_on_gpus_with_each_weight_push(push):
    """The static trainer / rollout split on two GPUs with the weight push by library send / recv, by the peer-store
    kernel and by one multicast store through the NVSwitch: weights agree on both ranks afterwards and the rollout
    rank generates with the pushed version."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    port = {"nccl": "29780", "symm": "29781", "nvls": "29782"}[push]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", port, "-m", "cverl_b200.cli.static_split", "--backend", "nccl", "--trainers",
           "1", "--steps", "2", "--weight-push", push]
    p = subprocess.run(cmd, cwd=root, env=dict(os.environ, PYTHONPATH=str(root)), capture_output=True, text=True,
                       timeout=120)
    if push == "nvls" and "NVLS unavailable" in (p.stdout + p.stderr):
        pytest.skip("no NVSwitch multicast on this machine")
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    assert "weights_in_sync=True" in p.stdout and "weight_version=1" in p.stdout
