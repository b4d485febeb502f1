"""Tensor parallelism and ZeRO sharding on CPU ranks (gloo) and with scripted fake collectives."""
import pytest
import torch

from cverl_b200.models.config import Qwen35TextConfig
from cverl_b200.models.params import model_param_specs, shard_tensor, unshard_tensor
from cverl_b200.models.qwen3_5 import Qwen35Model
from cverl_b200.optim import AdamWOptions, FlatAdamW, Fp32MasterAdamW
from cverl_b200.parallel.collectives import Collectives, ReduceOp, SingleProcessCollectives
from cverl_b200.parallel.zero import (FlatZeroOptimizer, flat_sharded_adamw_step, flatten_parameter_shard,
                                      greedy_parameter_owners)
from dist_utils import run_ranks


def _fold(model):
    for p in list(model.flat.params.values()) + list(model.fused.values()):
        if p.grad is not None:
            p.main_grad.add_(p.grad.float())
            p.grad = None


def _tp_worker(rank, world, moe):
    from cverl_b200.parallel.mesh import build_context
    torch.manual_seed(0)
    cfg = Qwen35TextConfig.tiny(moe=moe, layers=4)
    ctx = build_context(world, rank, tp=2, dp=1)
    tp_model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx)
    tp_model.init_weights(seed=11)
    dense = Qwen35Model(cfg, dtype=torch.float32)
    dense.init_weights(seed=11)
    ids = torch.randint(0, cfg.vocab_size, (2, 20), generator=torch.Generator().manual_seed(3))
    w = torch.randn(2, 12, generator=torch.Generator().manual_seed(4))
    lp_tp = tp_model.response_logprobs(ids, 8)
    lp_d = dense.response_logprobs(ids, 8)
    torch.testing.assert_close(lp_tp, lp_d, rtol=1e-4, atol=1e-4)
    (lp_tp * w).sum().backward()
    (lp_d * w).sum().backward()
    _fold(tp_model)
    _fold(dense)
    tp_model.sync_replicated_grads()
    # every local gradient equals the matching shard of the dense gradient (correct TP backward)
    for spec in dense.specs:
        if spec.expert >= 0:
            continue
        full = dense.flat.params[spec.name].main_grad
        local = shard_tensor(spec, full, ctx.tp_rank, 2).reshape(tp_model.flat.params[spec.name].shape)
        torch.testing.assert_close(tp_model.flat.params[spec.name].main_grad, local, rtol=2e-3, atol=2e-5,
                                   msg=lambda m: f"{spec.name}: {m}")


def test_tp2_matches_dense_forward_and_backward():
    run_ranks(_tp_worker, 2, False)


def test_shard_unshard_roundtrip():
    cfg = Qwen35TextConfig.tiny(layers=4)
    for spec in model_param_specs(cfg):
        full = torch.randn(spec.full_shape)
        shards = [shard_tensor(spec, full, r, 2) for r in range(2)]
        assert tuple(shards[0].shape) == spec.local_shape(2)
        torch.testing.assert_close(unshard_tensor(spec, shards), full)


def _zero_worker(rank, world):
    import torch.distributed as dist
    from cverl_b200.parallel.mesh import build_context
    cfg = Qwen35TextConfig.tiny(layers=2)
    ctx = build_context(world, rank, tp=1, dp=2)
    model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx, pad_multiple=2 * 8)
    model.init_weights(seed=5)
    ref = Qwen35Model(cfg, dtype=torch.float32, pad_multiple=2 * 8)
    ref.init_weights(seed=5)
    opts = AdamWOptions(lr=1e-2, beta2=0.95, use_master_weights=True)
    opt = FlatZeroOptimizer(model.flat, opts, dp_group=ctx.dp_group, dp_rank=rank, dp_size=2, norm_group=None,
                            norm_world=2, max_grad_norm=0.5)
    ropt = FlatZeroOptimizer(ref.flat, opts, max_grad_norm=0.5)
    gen = torch.Generator().manual_seed(9)
    for step in range(2):
        grads = [torch.randn(model.flat.padded_numel, generator=gen) for _ in range(2)]
        for g in grads:
            g[model.flat.numel:] = 0
        model.flat.main_grad.copy_(grads[rank])
        ref.flat.main_grad.copy_((grads[0] + grads[1]) / 2)
        opt.step()
        ropt.step()
        torch.testing.assert_close(model.flat.flat, ref.flat.flat, rtol=1e-5, atol=2e-5)
        # the global norm is the norm of the averaged gradient: shards' squared norms add up
        assert abs(opt.last_metrics[1].item() - ropt.last_metrics[1].item()) < 1e-3 * ropt.last_metrics[1].item()
        assert model.flat.main_grad.abs().max().item() == 0.0


def test_flat_zero_dp2_matches_single_rank():
    run_ranks(_zero_worker, 2)


class SliceCollectives(Collectives):
    """Simulates one rank of a DP group: reduce_scatter sums scripted peer tensors and returns this
    rank's slice, all_gather returns scripted shards.  Records every call."""

    def __init__(self, rank, world, peer_flat_grads=None, gathered=None):
        self._rank, self._world = rank, world
        self.peer_flat_grads, self.gathered = peer_flat_grads, gathered
        self.calls = []

    def rank(self): return self._rank
    def world_size(self): return self._world
    def barrier(self, group=None): self.calls.append(("barrier",))
    def broadcast(self, tensor, root, group=None): return tensor.clone()

    def all_reduce(self, tensor, op=ReduceOp.SUM, group=None):
        self.calls.append(("all_reduce", op, tensor.dtype))
        return tensor * self._world if op == ReduceOp.SUM else tensor.clone()

    def all_gather(self, tensor, group=None):
        self.calls.append(("all_gather", tensor.dtype))
        parts = list(self.gathered)
        parts[self._rank] = tensor
        return torch.cat(parts)

    def reduce_scatter(self, tensor, op=ReduceOp.SUM, group=None):
        self.calls.append(("reduce_scatter", op, tensor.dtype))
        total = tensor.clone()
        for r, g in enumerate(self.peer_flat_grads):
            if r != self._rank:
                total += g.to(tensor.dtype)
        if op == ReduceOp.MEAN:
            total /= self._world
        n = total.numel() // self._world
        return total[self._rank * n:(self._rank + 1) * n].clone()

    def all_to_all(self, tensor, group=None): return tensor.clone()
    def send(self, tensor, dst): raise RuntimeError
    def recv_like(self, like, src): raise RuntimeError


def test_flat_sharded_adamw_two_simulated_ranks_equals_dense():
    torch.manual_seed(0)
    shapes = [(5, 3), (7,), (4, 4)]
    params0 = [torch.randn(s) for s in shapes]
    grads = [[torch.randn(s) for s in shapes] for _ in range(2)]
    opts = AdamWOptions(lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.01, use_master_weights=True)
    dense_p = [p.clone().requires_grad_(True) for p in params0]
    dense = Fp32MasterAdamW(dense_p, opts)
    for p, g0, g1 in zip(dense_p, grads[0], grads[1]):
        p.grad = (g0 + g1) / 2
    dense.step()
    total = sum(p.numel() for p in params0)
    padded = (total + 1) // 2 * 2

    def flat_of(gs):
        f = torch.zeros(padded)
        f[:total] = torch.cat([g.reshape(-1) for g in gs])
        return f
    new_shards = []
    for rank in range(2):
        ps = [p.clone().requires_grad_(True) for p in params0]
        for p, g in zip(ps, grads[rank]):
            p.grad = g.clone()
        shard = flatten_parameter_shard(ps, rank, 2, dtype=torch.float32)
        assert (shard.original_numel, shard.padded_numel) == (total, padded)
        comm = SliceCollectives(rank, 2, peer_flat_grads=[flat_of(grads[0]), flat_of(grads[1])],
                                gathered=[torch.zeros(padded // 2)] * 2)
        opt = FlatAdamW(shard.shard.clone(), opts)
        res = flat_sharded_adamw_step(ps, shard, opt, comm, [0, 1], comm, [0, 1], max_grad_norm=0.0,
                                      apply_parameters=False)
        assert ("reduce_scatter", ReduceOp.MEAN, torch.float32) in comm.calls
        assert all(p.grad is None for p in ps)
        assert res.grad_clip_scale == 1.0
        new_shards.append(shard.shard.clone())
    flat_new = torch.cat(new_shards)[:total]
    dense_flat = torch.cat([p.detach().reshape(-1) for p in dense_p])
    torch.testing.assert_close(flat_new, dense_flat, rtol=1e-5, atol=2e-5)


def test_dp1_skips_collectives_and_clipping():
    torch.manual_seed(1)
    ps = [torch.randn(6, 2).requires_grad_(True)]
    ps[0].grad = torch.full((6, 2), 10.0)
    shard = flatten_parameter_shard(ps, 0, 1)
    comm = SingleProcessCollectives()
    opt = FlatAdamW(shard.shard.clone(), AdamWOptions(lr=1e-3, use_master_weights=False))
    res = flat_sharded_adamw_step(ps, shard, opt, comm, [0], comm, [0], max_grad_norm=1.0)
    norm = (10.0 ** 2 * 12) ** 0.5
    assert res.global_grad_norm == pytest.approx(norm, rel=1e-5)
    assert res.grad_clip_scale == pytest.approx(1.0 / (norm + 1e-6), rel=1e-5)


def test_greedy_owners_balance():
    owners = greedy_parameter_owners([100, 90, 50, 40, 10, 5], 2)
    load = [0, 0]
    for n, o in zip([100, 90, 50, 40, 10, 5], owners):
        load[o] += n
    assert owners[0] != owners[1] and abs(load[0] - load[1]) <= 15


def test_adamw_master_keeps_small_updates_and_load_state():
    p = torch.ones(16, dtype=torch.bfloat16)
    opts = AdamWOptions(lr=1e-5, weight_decay=0.0, use_master_weights=True)
    opt = FlatAdamW(p, opts)
    opt.step(torch.ones(16))
    assert (opt.master < 1.0).all()          # fp32 master moved
    assert (p == 1.0).all()                  # bf16 rounds the tiny update away
    nomaster = FlatAdamW(torch.ones(16, dtype=torch.bfloat16), AdamWOptions(use_master_weights=False))
    assert nomaster.master is None and nomaster.parameter_shard.dtype == torch.bfloat16
    opt2 = FlatAdamW(torch.zeros(16), opts)
    opt2.load_state(opt.master, opt.exp_avg, opt.exp_avg_sq, opt.step_count)
    opt.step(torch.ones(16))
    opt2.step(torch.ones(16))
    torch.testing.assert_close(opt.master, opt2.master)
    with pytest.raises(ValueError):
        opt2.load_state(opt.master[:4], opt.exp_avg, opt.exp_avg_sq, 1)


class _ScriptedDp:
    """Plays rank ``rank`` of a data-parallel group of ``n``: every peer's gradient is this rank's scaled by a
    known factor, so reductions have closed forms; calls and their dtypes / sizes are recorded."""

    def __init__(self, rank, n, factors):
        from cverl_b200.parallel.collectives import Collectives
        self._rank, self._n, self.factors, self.calls = rank, n, factors, []

    def rank(self):
        return self._rank

    def world_size(self):
        return self._n

    def all_reduce(self, t, op, group):
        from cverl_b200.parallel.collectives import ReduceOp
        self.calls.append(("all_reduce", t.dtype, t.numel()))
        total = t.float() * sum(self.factors) / self.factors[self._rank]
        return (total / self._n if op == ReduceOp.MEAN else total).to(t.dtype)

    def reduce_scatter(self, t, op, group):
        from cverl_b200.parallel.collectives import ReduceOp
        self.calls.append(("reduce_scatter", t.dtype, t.numel()))
        total = t.float() * sum(self.factors) / self.factors[self._rank]
        total = total / self._n if op == ReduceOp.MEAN else total
        k = t.numel() // self._n
        return total[self._rank * k:(self._rank + 1) * k].to(t.dtype)

    def broadcast(self, t, root, group):
        self.calls.append(("broadcast", root, t.numel()))
        return t.clone() if root == self._rank else torch.full_like(t, float(root + 100))


def test_bucketed_dp_gradient_sync_and_owner_broadcast():
    """Bucket boundaries, single-tensor buckets, forced communication dtype, a group of one, reduce-scatter
    padding and the ZeRO-1 owner broadcast, each against a scripted rank (reference behaviour:
    src/distributed/parallel_ops.cc:226-321)."""
    from cverl_b200.parallel import dp_sync
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(n)) for n in (100, 300, 50, 1000, 7)]
    for p in params:
        p.grad = torch.randn_like(p)
    want = [p.grad.clone() * (1.0 + 3.0) / 2.0 for p in params]
    fake = _ScriptedDp(0, 2, [1.0, 3.0])
    calls = dp_sync.data_parallel_sync_gradients(params, fake, [0, 1], True, bucket_bytes=1700)
    # 100+300 floats fit 1700 bytes, 50 opens the next bucket with nothing else fitting beside 1000, then 7
    assert calls == 4 and [c[2] for c in fake.calls] == [400, 50, 1000, 7]
    for p, w in zip(params, want):
        assert torch.allclose(p.grad, w, atol=1e-6)
    # forced bf16 communication halves the bytes per element, so more fits a bucket, and the wire dtype is bf16
    fake = _ScriptedDp(1, 2, [1.0, 3.0])
    dp_sync.data_parallel_sync_gradients(params, fake, [0, 1], False, bucket_bytes=1700, comm_dtype=torch.bfloat16)
    assert all(c[1] == torch.bfloat16 for c in fake.calls) and [c[2] for c in fake.calls] == [450, 1000, 7]
    # a data group of one issues nothing; a non-member is refused
    lone = _ScriptedDp(0, 1, [1.0])
    assert dp_sync.data_parallel_sync_gradients(params, lone, [0]) == 0 and not lone.calls
    with pytest.raises(ValueError):
        dp_sync.data_parallel_sync_gradients(params, _ScriptedDp(5, 2, [1.0, 1.0]), [0, 1])
    with pytest.raises(ValueError):
        dp_sync.data_parallel_sync_gradients(params, fake, [0, 1], bucket_bytes=0)
    # reduce-scatter buckets: padded to the group size, this rank's slice of the mean
    for p in params:
        p.grad = torch.ones_like(p)
    fake = _ScriptedDp(1, 2, [1.0, 1.0])
    buckets = dp_sync.data_parallel_reduce_scatter_gradients(params, fake, [0, 1], True, bucket_bytes=10 ** 9)
    assert len(buckets) == 1 and buckets[0].original_numel == 1457 and buckets[0].padded_numel == 1458
    assert buckets[0].parameter_indices == [0, 1, 2, 3, 4] and buckets[0].shard.numel() == 729
    assert float(buckets[0].shard[:-1].min()) == 1.0 and float(buckets[0].shard[-1]) == 0.0     # the padding
    # owner broadcast: rank 0 owns parameters 0 and 3, rank 1 the rest; rank 0 keeps its own and receives the others
    owners = [0, 1, 1, 0, 1]
    vals = [torch.full((n,), float(i)) for i, n in enumerate((100, 300, 50, 1000, 7))]
    fake = _ScriptedDp(0, 2, [1.0, 1.0])
    calls = dp_sync.broadcast_owner_parameters(vals, owners, fake, [0, 1], bucket_bytes=10 ** 9)
    assert calls == 2 and [c[1] for c in fake.calls] == [0, 1]
    assert float(vals[0][0]) == 0.0 and float(vals[3][0]) == 3.0 and all(float(vals[i][0]) == 101.0 for i in (1, 2, 4))
    # flat bucket ranges cut at parameter boundaries
    assert dp_sync.flat_bucket_ranges([100, 300, 50, 1000, 7], [0, 104, 408, 464, 1464], 1700, 4) == \
        [(0, 404), (408, 458), (464, 1464), (1464, 1471)]


def test_ep_row_plan_and_overflow_flag():
    """Destination rows of the peer-memory expert dispatch: rows for one destination are stacked by source
    rank; a destination that would overflow its buffer raises the flag and the surplus entries are left out
    (rank -1) instead of being written over the last row."""
    from cverl_b200.parallel.ep_symm import plan_rows
    dst = [torch.tensor([0, 1, 1, 0, 1]), torch.tensor([1, 1, 0, 1, 1])]         # routed entries of ranks 0 and 1
    table = torch.stack([torch.bincount(d, minlength=2) for d in dst]).to(torch.int64)   # [src, dst]
    r0 = plan_rows(table, 0, dst[0], capacity_rows=16)
    r1 = plan_rows(table, 1, dst[1], capacity_rows=16)
    assert r0[0].tolist() == [0, 1, 1, 0, 1] and r0[1].tolist() == [0, 0, 1, 1, 2] and int(r0[2]) == 0
    assert r1[1].tolist() == [3, 4, 2, 5, 6]            # after rank 0's 3 rows at destination 1, 2 rows at 0
    rows_at_1 = sorted([r for k, r in zip(r0[0].tolist(), r0[1].tolist()) if k == 1] +
                       [r for k, r in zip(r1[0].tolist(), r1[1].tolist()) if k == 1])
    assert rows_at_1 == list(range(7))                  # dense, no collisions
    # capacity 5 < 7 rows bound for rank 1: flag set on every rank, surplus entries dropped, none clamped
    o0 = plan_rows(table, 0, dst[0], capacity_rows=5)
    o1 = plan_rows(table, 1, dst[1], capacity_rows=5)
    assert int(o0[2]) == 1 and int(o1[2]) == 1
    assert o1[0].tolist() == [1, 1, 0, -1, -1] and o1[1].tolist() == [3, 4, 2, 0, 0]
    assert all(r < 5 for r in o0[1].tolist() + o1[1].tolist())


def _zero2_worker(rank, world, moe):
    """Bucketed ZeRO-2 (gradients reduced per layer from inside the backward pass) against the flat optimizer on
    one rank that sees both ranks' batches."""
    from cverl_b200.parallel.mesh import build_context
    from cverl_b200.parallel.zero2 import BucketedZero2Optimizer
    cfg = Qwen35TextConfig.tiny(moe=moe, layers=3)
    ctx = build_context(world, rank, tp=1, dp=2)
    model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx, pad_multiple=2 * 8, grad_buckets=True, bucket_align=2 * 8,
                        grad_slots=2)
    model.init_weights(seed=5)
    assert model.flat.main_grad is None and model.flat.bucket_ids == list(range(cfg.num_hidden_layers + 1))
    ref = Qwen35Model(cfg, dtype=torch.float32, pad_multiple=2 * 8)
    ref.init_weights(seed=5)
    opts = AdamWOptions(lr=1e-2, beta2=0.95, use_master_weights=False)
    opt = BucketedZero2Optimizer(model, opts, dp_group=ctx.dp_group, dp_rank=rank, dp_size=2, norm_group=None,
                                 norm_world=2, max_grad_norm=0.5)
    ropt = FlatZeroOptimizer(ref.flat, opts, max_grad_norm=0.5)
    gen = torch.Generator().manual_seed(11)
    for step in range(2):
        # two micro-batches per rank: buckets are reduced and accumulated once per backward pass
        ids = torch.randint(0, cfg.vocab_size, (2, 2, 2, 12), generator=gen)       # [rank, micro-batch, B, S]
        w = torch.randn(2, 2, 2, 8, generator=gen)
        for mb in range(2):
            lp = model.response_logprobs(ids[rank, mb], 4)
            lp.backward(w[rank, mb] * 0.5)
        assert opt.reduced_buckets == (step * 2 + 2) * cfg.num_hidden_layers
        for r in range(2):
            for mb in range(2):
                lp = ref.response_logprobs(ids[r, mb], 4)
                lp.backward(w[r, mb] * 0.25)
        _fold(ref)
        opt.step()
        ropt.step()
        for name, t in model.flat.named_tensors():
            # AdamW moves every element by about lr = 1e-2; an element whose gradient is near zero turns the last
            # bits of the two summation orders into a visible fraction of that, so the bound is 1 % of a step
            torch.testing.assert_close(t, ref.flat.params[name].data, rtol=2e-4, atol=1e-4, msg=lambda m: f"{name}: {m}")
        assert abs(opt.last_metrics[1].item() - ropt.last_metrics[1].item()) < 1e-3 * ropt.last_metrics[1].item()
        assert all(float(g.abs().max()) == 0.0 for g in model.flat.grad_buffers)
        assert float(opt.grad_shard.abs().max()) == 0.0
    # state round trip: a second optimizer loaded from the first continues identically
    sd = opt.state_dict()
    opt.load_state_dict(sd)
    assert opt.step_count == 2 and int(sd["bucket_chunks"].sum()) == opt.shard_numel


@pytest.mark.parametrize("moe", [False, True])
def test_bucketed_zero2_dp2_matches_single_rank(moe):
    run_ranks(_zero2_worker, 2, moe)


def test_flat_params_gradient_buckets_layout():
    from cverl_b200.models.params import FlatParams
    entries = [("emb", (5, 4)), ("l0.a", (3, 8)), ("l0.b", (8,)), ("l1.a", (3, 8)), ("l1.b", (8,)), ("l2.a", (3, 8))]
    fp = FlatParams(entries, dtype=torch.float32, pad_multiple=16, grad_buckets=[0, 1, 1, 2, 2, 3], bucket_align=16,
                    grad_slots=2, pinned_buckets=(0,))
    assert fp.bucket_ranges == {0: (0, 32), 1: (32, 64), 2: (64, 96), 3: (96, 128)} and fp.padded_numel == 128
    assert fp.grad_slot_of == {1: 1, 2: 0, 3: 1} and len(fp.grad_buffers) == 3
    # buckets 1 and 3 share a slot: the same memory backs both parameters' gradients
    assert fp.params["l0.a"].main_grad.data_ptr() == fp.params["l2.a"].main_grad.data_ptr()
    assert fp.params["l1.a"].main_grad.data_ptr() != fp.params["l0.a"].main_grad.data_ptr()
    assert fp.fused_view(["l0.a", "l0.b"], (32,)).main_grad.numel() == 32
    with pytest.raises(ValueError):
        fp.fused_view(["l0.b", "l1.a"], (32,))                  # crosses a bucket boundary
    with pytest.raises(ValueError):
        FlatParams(entries, grad_buckets=[0, 1, 0, 2, 2, 3])    # bucket ids must not decrease


def _tp_decode_worker(rank, world):
    """Cached decode (prefill + one-token steps: KV cache, convolution tail, recurrent state) under tensor
    parallelism against the same model on one rank: the logits of every step agree."""
    from cverl_b200.models import decode
    from cverl_b200.parallel.mesh import build_context
    cfg = Qwen35TextConfig.tiny(layers=4)
    ctx = build_context(world, rank, tp=world, dp=1)
    tp_model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx)
    tp_model.init_weights(seed=9)
    dense = Qwen35Model(cfg, dtype=torch.float32)
    dense.init_weights(seed=9)
    prompt = torch.randint(0, cfg.vocab_size, (2, 7), generator=torch.Generator().manual_seed(4))
    st_tp, lg_tp = decode.prefill(tp_model, prompt, 12)
    st_d, lg_d = decode.prefill(dense, prompt, 12)
    torch.testing.assert_close(lg_tp, lg_d, rtol=2e-4, atol=2e-4)
    assert lg_tp.shape == (2, cfg.vocab_size)
    for _ in range(4):
        tok = lg_d.argmax(-1)
        lg_tp = decode.decode_step(tp_model, st_tp, tok)
        lg_d = decode.decode_step(dense, st_d, tok)
        torch.testing.assert_close(lg_tp, lg_d, rtol=2e-4, atol=2e-4)
    assert st_tp.length == st_d.length == 11


def test_cached_decode_under_tensor_parallelism():
    run_ranks(_tp_decode_worker, 2)


def _zero2_bf16_comm_worker(rank, world):
    """Buckets reduced in bf16: the shard gradient equals the fp32 reduction up to bf16 rounding of each addend."""
    from cverl_b200.parallel.mesh import build_context
    from cverl_b200.parallel.zero2 import BucketedZero2Optimizer
    cfg = Qwen35TextConfig.tiny(layers=2)
    ctx = build_context(world, rank, tp=1, dp=2)
    opts = AdamWOptions(lr=1e-2, beta2=0.95, use_master_weights=False)
    shards = []
    for cd in (None, torch.bfloat16):
        model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx, pad_multiple=16, grad_buckets=True, bucket_align=16)
        model.init_weights(seed=5)
        opt = BucketedZero2Optimizer(model, opts, dp_group=ctx.dp_group, dp_rank=rank, dp_size=2, norm_world=2,
                                     max_grad_norm=0.0, comm_dtype=cd)
        ids = torch.randint(0, cfg.vocab_size, (2, 12), generator=torch.Generator().manual_seed(20 + rank))
        model.response_logprobs(ids, 4).sum().backward()
        opt.finish_backward()
        shards.append(opt.grad_shard.clone())
    rel = ((shards[1] - shards[0]).norm() / shards[0].norm()).item()
    assert 0 < rel < 1e-2, rel
    with pytest.raises(ValueError):
        BucketedZero2Optimizer(model, opts, dp_size=2, fused_comm=object(), comm_dtype=torch.bfloat16)


def test_bucketed_zero2_low_precision_gradient_communication():
    run_ranks(_zero2_bf16_comm_worker, 2)


def test_peer_memory_weight_push_slices_cover_the_buffer_once():
    """The multicast weight push: trainer t sends slice t; over all trainers the slices tile the padded flat buffer
    exactly once, each starting on a 16-byte boundary; the peer-store mode sends the whole buffer to the served ranks."""
    from cverl_b200.parallel.weight_sync import ParameterView, PeerMemoryWeightPush

    class FakeBroadcaster:
        def __init__(self):
            self.pushed, self.syncs = [], 0

        def push(self, src, second=0):
            self.pushed.append((src.clone(), second))

        def sync(self):
            self.syncs += 1

    params = [ParameterView(f"p{i}", torch.arange(n, dtype=torch.float32) + 100 * i) for i, n in enumerate((5, 13, 7))]
    for trainers in (1, 2, 3):
        got = torch.full((32,), -1.0)
        for rank in range(trainers):
            push = object.__new__(PeerMemoryWeightPush)
            push.params, push.dtype, push.numel, push.trainers, push.world, push.mode = params, torch.float32, 25, trainers, 6, "nvls"
            push.bc, push.recv = FakeBroadcaster(), torch.zeros(25)
            push.push(rank, [])
            assert push.bc.syncs == 1
            for src, off in push.bc.pushed:
                assert off % 16 == 0 and src.numel() % 4 == 0
                assert (got[off // 4: off // 4 + src.numel()] == -1).all()        # nobody wrote here before
                got[off // 4: off // 4 + src.numel()] = src
        flat = torch.cat([p.tensor for p in params])
        assert torch.equal(got[:25], flat) and (got[25:32] == 0).all()
    push = object.__new__(PeerMemoryWeightPush)
    push.params, push.dtype, push.numel, push.trainers, push.world, push.mode = params, torch.float32, 25, 2, 4, "symm"
    push.bc, push.recv = FakeBroadcaster(), torch.zeros(25)
    push.push(1, [3])
    (src, dsts), = push.bc.pushed
    assert dsts == [3] and src.numel() == 32 and torch.equal(src[:25], torch.cat([p.tensor for p in params]))
    push.bc = FakeBroadcaster()
    push.push(2, [])                                  # a rollout rank: no send, one barrier, parameters loaded
    assert push.bc.pushed == [] and push.bc.syncs == 1


def test_multicast_allreduce_slices_tile_the_buffer():
    from cverl_b200.parallel.nvls import allreduce_slice
    for n in (8, 40, 40968, 83886080):
        for world in (2, 3, 4, 8):
            pos = 0
            for r in range(world):
                lo, length = allreduce_slice(n, world, r)
                assert lo == pos and lo % 8 == 0 and length >= 0
                pos += length
            assert pos == n
