"""Context parallelism on gloo ranks: sharding, ring schedule, streaming vs dense attention,
ring attention forward/backward, and the full hybrid model (halo + state carry) vs a dense run."""
import math

import pytest
import torch

from cverl_b200.models.config import Qwen35TextConfig
from cverl_b200.models.qwen3_5 import Qwen35Model
from cverl_b200.ops.attention import causal_attention_ref
from cverl_b200.parallel.context_parallel import (padded_shard_len, ring_schedule, shard_sequence,
                                                  streaming_attention)
from dist_utils import run_ranks


def test_shard_and_schedule():
    x = torch.arange(10).view(1, 10)
    parts = [shard_sequence(x, r, 3, 1) for r in range(3)]
    assert padded_shard_len(10, 3) == 4
    assert parts[2].tolist() == [[8, 9, 0, 0]]
    assert [o for o, _, _ in ring_schedule(1, 3)] == [1, 0, 2]
    assert ring_schedule(2, 4)[0][1:] == (3, 1)


def test_streaming_attention_order_independent_and_padded():
    torch.manual_seed(0)
    B, Hq, Hkv, S, D = 2, 4, 2, 12, 8
    q, k, v = torch.randn(B, Hq, S, D), torch.randn(B, Hkv, S, D), torch.randn(B, Hkv, S, D)
    dense = causal_attention_ref(q.transpose(1, 2).reshape(B * S, Hq, D), k.transpose(1, 2).reshape(B * S, Hkv, D),
                                 v.transpose(1, 2).reshape(B * S, Hkv, D), B, S).view(B, S, Hq, D).transpose(1, 2)
    ks, vs = list(k.split(4, dim=2)), list(v.split(4, dim=2))
    for order in ([0, 1, 2], [2, 0, 1]):
        out, lse = streaming_attention(q, [ks[i] for i in order], [vs[i] for i in order], 0, [4 * i for i in order], S)
        torch.testing.assert_close(out, dense, rtol=1e-4, atol=1e-5)
    # a padded tail: keys >= original_len are ignored, queries of a later shard see everything before them
    out_tail, _ = streaming_attention(q[:, :, 8:], ks, vs, 8, [0, 4, 8], S)
    torch.testing.assert_close(out_tail, dense[:, :, 8:], rtol=1e-4, atol=1e-5)


def _ring_worker(rank, world):
    import torch.distributed as dist
    from cverl_b200.parallel.context_parallel import ring_attention
    torch.manual_seed(1)
    B, Hq, Hkv, S, D = 2, 4, 2, 4 * world - 1, 8          # ragged: the last shard is padded
    q, k, v = (torch.randn(B, h, S, D) for h in (Hq, Hkv, Hkv))
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    dense = causal_attention_ref(qd.transpose(1, 2).reshape(B * S, Hq, D), kd.transpose(1, 2).reshape(B * S, Hkv, D),
                                 vd.transpose(1, 2).reshape(B * S, Hkv, D), B, S).view(B, S, Hq, D).transpose(1, 2)
    w = torch.randn(B, Hq, S, D)
    (dense * w).sum().backward()
    s_loc = padded_shard_len(S, world)
    ql, kl, vl = (shard_sequence(t, rank, world, 2).clone().requires_grad_(True) for t in (q, k, v))
    out = ring_attention(ql, kl, vl, dist.group.WORLD, rank, world, S)
    ref = shard_sequence(dense.detach(), rank, world, 2)
    wl = shard_sequence(w, rank, world, 2)
    n_real = min(s_loc, S - rank * s_loc)
    torch.testing.assert_close(out[:, :, :n_real], ref[:, :, :n_real], rtol=1e-4, atol=1e-5)
    (out * wl).sum().backward()
    for got, full in ((ql, qd), (kl, kd), (vl, vd)):
        want = shard_sequence(full.grad, rank, world, 2)
        torch.testing.assert_close(got.grad[:, :, :n_real], want[:, :, :n_real], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_matches_dense(world):
    run_ranks(_ring_worker, world)


def _model_cp_worker(rank, world):
    from cverl_b200.parallel.mesh import build_context
    cfg = Qwen35TextConfig.tiny(layers=4)
    ctx = build_context(world, rank, cp=world, dp=1)
    cp_model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx)
    cp_model.init_weights(seed=6)
    dense = Qwen35Model(cfg, dtype=torch.float32)
    dense.init_weights(seed=6)
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(2))
    w = torch.randn(2, 16, generator=torch.Generator().manual_seed(3))
    lp = cp_model.response_logprobs(ids, 8)
    lpd = dense.response_logprobs(ids, 8)
    torch.testing.assert_close(lp, lpd, rtol=2e-4, atol=2e-4)
    # every rank holds the same loss; dividing by cp makes the CP-summed gradient the dense one
    ((lp * w).sum() / world).backward()
    (lpd * w).sum().backward()
    for m in (cp_model, dense):
        for p in list(m.flat.params.values()) + list(m.fused.values()):
            if p.grad is not None:
                p.main_grad.add_(p.grad)
                p.grad = None
    import torch.distributed as dist
    dist.all_reduce(cp_model.flat.main_grad)
    torch.testing.assert_close(cp_model.flat.main_grad, dense.flat.main_grad, rtol=5e-3, atol=5e-5)


def test_hybrid_model_context_parallel_matches_dense():
    run_ranks(_model_cp_worker, 2)


def _zigzag_worker(rank, world):
    """Zig-zag sharded ring attention (one equally sized launch per hop and rank) against dense causal attention:
    outputs and all three gradients, through the resharding in both directions."""
    import torch.distributed as dist
    from cverl_b200.parallel.cp_zigzag import zigzag_chunks, zigzag_reshard, zigzag_ring_attention
    torch.manual_seed(1)
    B, Hq, Hkv, D = 2, 4, 2, 8
    h = 3
    S = 2 * h * world
    q, k, v = (torch.randn(B, S, n, D) for n in (Hq, Hkv, Hkv))
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    dense = causal_attention_ref(qd.reshape(B * S, Hq, D), kd.reshape(B * S, Hkv, D), vd.reshape(B * S, Hkv, D), B,
                                 S).view(B, S, Hq, D)
    w = torch.randn(B, S, Hq, D)
    (dense * w).sum().backward()
    T = S // world
    cont = slice(rank * T, (rank + 1) * T)
    ql, kl, vl = (t[:, cont].clone().requires_grad_(True) for t in (q, k, v))
    packed = torch.cat([ql.reshape(B, T, -1), kl.reshape(B, T, -1), vl.reshape(B, T, -1)], dim=-1)
    z = zigzag_reshard(packed, dist.group.WORLD, rank, world, True)
    c0, c1 = zigzag_chunks(rank, world)
    want_rows = torch.cat([torch.arange(c0 * h, (c0 + 1) * h), torch.arange(c1 * h, (c1 + 1) * h)])
    torch.testing.assert_close(z[..., :Hq * D], q[:, want_rows].reshape(B, T, -1))      # the layout itself
    zq, zk, zv = z.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    out = zigzag_ring_attention(zq.reshape(B, T, Hq, D), zk.reshape(B, T, Hkv, D), zv.reshape(B, T, Hkv, D),
                                dist.group.WORLD, rank, world)
    torch.testing.assert_close(out, dense.detach()[:, want_rows], rtol=1e-4, atol=1e-5)
    back = zigzag_reshard(out.reshape(B, T, -1), dist.group.WORLD, rank, world, False).reshape(B, T, Hq, D)
    torch.testing.assert_close(back, dense.detach()[:, cont], rtol=1e-4, atol=1e-5)
    (back * w[:, cont]).sum().backward()
    for got, full in ((ql, qd), (kl, kd), (vl, vd)):
        torch.testing.assert_close(got.grad, full.grad[:, cont], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("world", [2, 3, 4])
def test_zigzag_ring_attention_matches_dense(world):
    run_ranks(_zigzag_worker, world)


def _model_zigzag_worker(rank, world):
    from cverl_b200.parallel.mesh import build_context
    cfg = Qwen35TextConfig.tiny(layers=4)
    ctx = build_context(world, rank, cp=world, dp=1)
    ctx.cp_zigzag = True
    cp_model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx)
    cp_model.init_weights(seed=6)
    dense = Qwen35Model(cfg, dtype=torch.float32)
    dense.init_weights(seed=6)
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(2))
    w = torch.randn(2, 16, generator=torch.Generator().manual_seed(3))
    lp = cp_model.response_logprobs(ids, 8)
    lpd = dense.response_logprobs(ids, 8)
    torch.testing.assert_close(lp, lpd, rtol=2e-4, atol=2e-4)
    ((lp * w).sum() / world).backward()
    (lpd * w).sum().backward()
    for m in (cp_model, dense):
        for p in list(m.flat.params.values()) + list(m.fused.values()):
            if p.grad is not None:
                p.main_grad.add_(p.grad)
                p.grad = None
    import torch.distributed as dist
    dist.all_reduce(cp_model.flat.main_grad)
    torch.testing.assert_close(cp_model.flat.main_grad, dense.flat.main_grad, rtol=5e-3, atol=5e-5)


def test_hybrid_model_zigzag_context_parallel_matches_dense():
    run_ranks(_model_zigzag_worker, 2)


@pytest.mark.parametrize("cp", [2, 3, 4, 8])
def test_zigzag_hop_plans_cover_the_causal_mask_once_and_balance_the_work(cp):
    """Over all ranks and owners, the one-launch-per-hop plans visit every (query half-chunk, key half-chunk) pair
    below the diagonal exactly once, the diagonal pairs causally, nothing above it - and every rank does the same
    amount of work per hop."""
    from cverl_b200.parallel.cp_zigzag import _hop_plan, zigzag_chunks
    from cverl_b200.parallel.context_parallel import ring_schedule
    h = 1
    seen = torch.zeros(2 * cp, 2 * cp, dtype=torch.int64)          # [query half-chunk, key half-chunk]
    causal_pairs = set()
    for rank in range(cp):
        mine = zigzag_chunks(rank, cp)
        work = []
        for owner, _, _ in ring_schedule(rank, cp):
            theirs = zigzag_chunks(owner, cp)
            (q0, q1), (k0, k1), causal = _hop_plan(owner, rank, h)
            qs = [mine[i] for i in range(2) if q0 <= i * h < q1]
            ks = [theirs[i] for i in range(2) if k0 <= i * h < k1]
            for qi, qc in enumerate(qs):
                for ki, kc in enumerate(ks):
                    if causal and ki > qi:
                        continue                                   # masked by the local causal rule
                    seen[qc, kc] += 1
                    if causal and ki == qi:
                        causal_pairs.add((qc, kc))
            work.append(len(qs) * len(ks))
        assert len(set(work)) <= 2 and set(work) <= {2, 4}          # 2 h^2 scores per hop (4 half-masked on the diagonal)
    want = torch.tril(torch.ones(2 * cp, 2 * cp, dtype=torch.int64))
    assert torch.equal(seen, want)
    assert causal_pairs == {(c, c) for c in range(2 * cp)}
