"""Qwen3-MoE: grouped path vs the dense expert loop; expert parallelism over gloo ranks."""
import pytest
import torch

from cverl_b200.models.config import Qwen35TextConfig
from cverl_b200.models.moe import moe_mlp, moe_mlp_dense_loop, router, sort_by_expert
from cverl_b200.models.qwen3_5 import Qwen35Model, _packed_moe_names
from dist_utils import run_ranks


def test_sort_by_expert_layout():
    ids = torch.tensor([3, 0, 3, 1, 3, 0])
    order, dest, tile_group, offsets, m_pad = sort_by_expert(ids, 4)
    assert offsets.tolist() == [0, 128, 256, 256, 384]
    assert ids[order].tolist() == [0, 0, 1, 3, 3, 3]
    assert dest.tolist() == [0, 1, 128, 256, 257, 258]
    assert tile_group[:3].tolist() == [0, 1, 3] and (tile_group[3:] == -1).all()
    assert m_pad % 128 == 0 and m_pad >= 384


def test_router_modes():
    x, g = torch.randn(5, 8), torch.randn(6, 8)
    idx, w = router(x, g, 2, True)
    assert torch.allclose(w.sum(-1), torch.ones(5))
    idx2, w2 = router(x, g, 2, False)
    full = torch.softmax(x @ g.t(), -1)
    assert torch.equal(idx, idx2) and torch.allclose(w2, full.gather(-1, idx))


def test_moe_grouped_matches_dense_loop_with_grads():
    cfg = Qwen35TextConfig.tiny(moe=True, layers=1)
    m = Qwen35Model(cfg, dtype=torch.float32)
    m.init_weights(seed=2)
    x = torch.randn(40, cfg.hidden_size, requires_grad=True)
    y = moe_mlp(m, x, 0)
    gu, dn = (m.param(n) for n in _packed_moe_names(0))
    ref = moe_mlp_dense_loop(x, m.param(f"{cfg.layer_root}0.mlp.gate.weight"), gu, dn, cfg.num_experts_per_tok,
                             cfg.norm_topk_prob)
    torch.testing.assert_close(y, ref, rtol=1e-4, atol=1e-5)
    gy = torch.randn_like(y)
    (gx,) = torch.autograd.grad(y, x, gy, retain_graph=True)
    (gr,) = torch.autograd.grad(ref, x, gy)
    torch.testing.assert_close(gx, gr, rtol=1e-4, atol=1e-5)


def test_moe_model_forward_backward():
    cfg = Qwen35TextConfig.tiny(moe=True, layers=2)
    m = Qwen35Model(cfg, dtype=torch.float32)
    m.init_weights(seed=3)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    lp = m.response_logprobs(ids, 6)
    lp.sum().backward()
    assert torch.isfinite(lp).all()
    # untied head, full rotary, no output gate
    assert "lm_head.weight" in m.flat.params and cfg.rotary_dim == cfg.head_dim


def _ep_worker(rank, world):
    from cverl_b200.parallel.mesh import build_context
    cfg = Qwen35TextConfig.tiny(moe=True, layers=1)
    ctx = build_context(world, rank, ep=2, dp=1)
    ep_model = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx)
    ep_model.init_weights(seed=4)
    dense = Qwen35Model(cfg, dtype=torch.float32)
    dense.init_weights(seed=4)
    # EP ranks see different micro-batches
    x = torch.randn(24, cfg.hidden_size, generator=torch.Generator().manual_seed(10 + rank)).requires_grad_(True)
    y = moe_mlp(ep_model, x, 0)
    yd = moe_mlp(dense, x, 0)
    torch.testing.assert_close(y, yd, rtol=1e-4, atol=1e-5)
    gy = torch.randn(24, cfg.hidden_size, generator=torch.Generator().manual_seed(20 + rank))
    (gx,) = torch.autograd.grad(y, x, gy)
    (gd,) = torch.autograd.grad(yd, x, gy)
    torch.testing.assert_close(gx, gd, rtol=1e-4, atol=1e-5)


def test_expert_parallel_matches_single_rank():
    run_ranks(_ep_worker, 2)


@pytest.mark.parametrize("moe", [False, True])
def test_activation_checkpointing_same_gradients_fewer_saved_bytes(moe):
    """A checkpointed layer keeps only its input: the gradients are those of the plain model (the recomputation is
    the same arithmetic), and the bytes autograd holds between the passes drop."""
    cfg = Qwen35TextConfig.tiny(moe=moe, layers=4)
    ids = torch.randint(0, cfg.vocab_size, (2, 24))
    grads, held = [], []
    for ckpt in (False, True):
        m = Qwen35Model(cfg, dtype=torch.float32, activation_checkpointing=ckpt)
        m.init_weights(seed=5)
        seen = {}

        def pack(t):
            if t.untyped_storage().data_ptr() not in params:
                seen[t.untyped_storage().data_ptr()] = t.untyped_storage().nbytes()
            return t
        params = {p.untyped_storage().data_ptr() for p in m.parameters()}
        with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
            lp = m.response_logprobs(ids, 8)
        held.append(sum(seen.values()))
        lp.sum().backward()
        m_grads = {n: (p.main_grad.clone() if getattr(p, "main_grad", None) is not None else None)
                   for n, p in m.flat.params.items()}
        for n, p in m.flat.params.items():
            if p.grad is not None:
                m_grads[n] = p.grad.clone() if m_grads[n] is None else m_grads[n] + p.grad
        grads.append(m_grads)
    assert held[1] < 0.6 * held[0], held
    assert set(grads[0]) == set(grads[1])
    checked = 0
    for n, g in grads[0].items():
        if g is None:
            assert grads[1][n] is None
            continue
        torch.testing.assert_close(grads[1][n], g, rtol=1e-6, atol=1e-7)
        checked += int(g.abs().sum() > 0)
    assert checked > 10
    # no graph, no checkpointing: inference and cached decode go straight through
    m.eval()
    with torch.no_grad():
        assert torch.isfinite(m.response_logprobs(ids, 8)).all()


@pytest.mark.parametrize("moe", [False, True])
def test_sharded_ranks_read_only_their_bytes(moe, tmp_path):
    """A tensor-parallel rank reads its rows of row-sharded tensors, an expert-parallel rank skips the other ranks'
    experts: the loaded shard equals what slicing the full tensors gives, from a fraction of the bytes."""
    from cverl_b200.models.hf_io import HfModelLoader, load_model_weights, synthesize_model_dir
    from cverl_b200.parallel.context import ParallelContext
    cfg = Qwen35TextConfig.tiny(moe=moe, layers=2)
    d = synthesize_model_dir(cfg, tmp_path / "m", dtype=torch.float32)
    full_loader = HfModelLoader(d).load_metadata()
    total = sum(full_loader.info(n).nbytes for n in full_loader.names())
    for rank in (0, 1):
        ctx = ParallelContext(tp_rank=rank, tp_size=2, ep_rank=rank if moe else 0, ep_size=2 if moe else 1)
        a = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx, with_main_grad=False)
        b = Qwen35Model(cfg, dtype=torch.float32, ctx=ctx, with_main_grad=False)
        loader = HfModelLoader(d)
        load_model_weights(a, loader)
        for spec in b.specs:                                   # the plain way: read everything, slice
            b.load_full_tensor(spec.name, full_loader.load_tensor(spec.name))
        assert torch.equal(a.flat.flat, b.flat.flat) and a.flat.flat.abs().sum() > 0
        assert loader.bytes_read < (0.62 if moe else 0.8) * total, (loader.bytes_read, total)
    rows = full_loader.load_rows(cfg.embed_name, 3, 9, threads=3)
    assert torch.equal(rows, full_loader.load_tensor(cfg.embed_name)[3:9])
    assert full_loader.load_rows(cfg.embed_name, 5, 5).shape[0] == 0
    with pytest.raises(ValueError):
        full_loader.load_rows(cfg.embed_name, 0, cfg.vocab_size + 1)
