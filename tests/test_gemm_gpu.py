"""tcgen05 GEMM, linear autograd and fused LM-head log-prob against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from cverl_b200 import _native as nv
    if torch.cuda.is_available():
        nv.check_status()


# ------------------------------- GEMM ---------------------------------------
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 1000, 520), (4096, 1024, 1024),
                                   (130, 72, 136), (5000, 3584, 1024)])
def test_gemm_nt(M, N, K):
    from cverl_b200.ops import gemm_nt
    torch.manual_seed(0)
    a = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(N, K, device=_dev(), dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = gemm_nt(a, b)
    assert _rel_err(out, ref) < 6e-3
    out32 = gemm_nt(a, b, out_dtype=torch.float32)
    assert _rel_err(out32, ref) < 1e-4


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (512, 1024, 384), (1000, 520, 1000), (4096, 1024, 2048)])
def test_gemm_nn(M, N, K):
    from cverl_b200.ops import gemm_nn
    torch.manual_seed(1)
    a = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(K, N, device=_dev(), dtype=torch.bfloat16)
    ref = a.float() @ b.float()
    assert _rel_err(gemm_nn(a, b, out_dtype=torch.float32), ref) < 1e-4


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 4096), (1024, 1024, 20000), (520, 1000, 1000)])
def test_gemm_tn_accumulate(M, N, K):
    from cverl_b200.ops import gemm_tn_acc
    torch.manual_seed(2)
    a = torch.randn(K, M, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(K, N, device=_dev(), dtype=torch.bfloat16)
    acc = torch.ones(M, N, device=_dev(), dtype=torch.float32)
    ref = 1.0 + a.float().t() @ b.float()
    gemm_tn_acc(a, b, acc)
    assert _rel_err(acc, ref) < 1e-4


def test_linear_autograd():
    from cverl_b200.ops import linear
    torch.manual_seed(3)
    x = torch.randn(3, 300, 512, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(768, 512, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 6e-3
    assert _rel_err(x.grad, xr.grad) < 6e-3
    assert _rel_err(w.grad, wr.grad) < 6e-3
    # main_grad accumulation path
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.zeros(w2.shape, device=_dev(), dtype=torch.float32)
    linear(x.detach(), w2).backward(dy)
    linear(x.detach(), w2).backward(dy)
    assert w2.grad is None
    assert _rel_err(w2.main_grad, 2 * wr.grad) < 1e-4


# ------------------------------- LM head ------------------------------------
@pytest.mark.parametrize("M,V,K", [(300, 1000, 256), (1024, 5000, 1024)])
def test_lmhead_logprob(M, V, K):
    from cverl_b200.ops import lmhead_logprob
    from cverl_b200.ops.lmhead import lmhead_logprob_ref
    torch.manual_seed(12)
    h = (0.5 * torch.randn(M, K, device=_dev())).to(torch.bfloat16).requires_grad_(True)
    emb = (0.1 * torch.randn(V, K, device=_dev())).to(torch.bfloat16).requires_grad_(True)
    tgt = torch.randint(0, V, (M,), device=_dev())
    lp = lmhead_logprob(h, emb, tgt)
    g = torch.randn(M, device=_dev())
    lp.backward(g)
    hr, er = h.detach().float().requires_grad_(True), emb.detach().float().requires_grad_(True)
    lpr = lmhead_logprob_ref(hr, er, tgt)
    lpr.backward(g)
    assert (lp - lpr).abs().max().item() < 2e-3
    assert _rel_err(h.grad, hr.grad) < 1.5e-2
    assert _rel_err(emb.grad, er.grad) < 1.5e-2




# --------------------------- Gated-DeltaNet scans ---------------------------
def _gdn_scan_inputs(B=2, H=3, n=5, seed=0):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s, sc=1.0: (sc * torch.randn(*s, generator=g)).to(torch.bfloat16).float().to(_dev())
    W = mk(B, H, n, 64, 128, sc=0.1)
    U = mk(B, H, n, 64, 128)
    Kd = mk(B, H, n, 64, 128, sc=0.1)
    Qd = mk(B, H, n, 64, 128, sc=0.1)
    egam = torch.exp(-torch.rand(B, H, n, generator=g)).to(_dev())
    S0 = (0.1 * torch.randn(B, H, 128, 128, generator=g)).to(_dev())
    return W, U, Kd, Qd, egam, S0


def test_gdn_scan_fwd_kernel():
    from cverl_b200.ops import gdn, gdn_native
    W, U, Kd, Qd, egam, S0 = _gdn_scan_inputs()
    Vn, Ss, Sf = gdn_native.scan_fwd(W, U, Kd, egam, S0)
    Vr, Sr, Sfr = gdn.scan_fwd_ref(W, U, Kd, egam, S0)
    assert _rel_err(Vn, Vr) < 1e-2
    assert _rel_err(Ss, Sr) < 1e-2
    assert _rel_err(Sf, Sfr) < 1e-2
    Vn0, _, _ = gdn_native.scan_fwd(W, U, Kd, egam, None)
    Vr0, _, _ = gdn.scan_fwd_ref(W, U, Kd, egam, torch.zeros_like(S0))
    assert _rel_err(Vn0, Vr0) < 1e-2


def test_gdn_scan_bwd_kernel():
    from cverl_b200.ops import gdn, gdn_native
    W, U, Kd, Qd, egam, S0 = _gdn_scan_inputs(seed=1)
    dO = (0.5 * U.flip(2)).to(torch.bfloat16).float()
    P = (0.2 * torch.randn(*U.shape[:3], 64, 64, device=U.device)).tril().to(torch.bfloat16).float()
    dVn, dSn, dS0 = gdn_native.scan_bwd(P, Kd, Qd, W, dO, egam, S0)
    rV, rS, r0 = gdn.scan_bwd_ref(P.transpose(-1, -2) @ dO, Kd, Qd, W, dO, egam, S0)
    assert _rel_err(dVn, rV) < 1e-2
    assert _rel_err(dSn, rS) < 1e-2
    assert _rel_err(dS0, r0) < 1e-2


def test_gdn_fused_matches_recurrence_on_gpu():
    from cverl_b200.ops import gdn
    torch.manual_seed(5)
    B, T, H = 2, 200, 2
    q = torch.randn(B, T, H, 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, H, 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, H, 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    beta = torch.sigmoid(torch.randn(B, T, H, device=_dev())).requires_grad_(True)
    g = (-0.5 * torch.rand(B, T, H, device=_dev())).requires_grad_(True)
    scale = 128 ** -0.5
    o, Sf = gdn.gated_delta_rule_fused(q, k, v, beta, g, None, scale=scale)
    do = torch.randn_like(o)
    o.backward(do)
    ins = [t.detach().float().cpu().requires_grad_(True) for t in (q, k, v, beta, g)]
    qq, kk, vv, bb, gg = ins
    o_r, S_r = gdn.gdn_recurrent_ref((gdn.l2norm(qq) * scale).transpose(1, 2), gdn.l2norm(kk).transpose(1, 2),
                                     vv.transpose(1, 2), bb.transpose(1, 2), gg.transpose(1, 2))
    o_r = o_r.transpose(1, 2)
    o_r.backward(do.float().cpu())
    assert _rel_err(o.cpu(), o_r) < 2e-2
    assert _rel_err(Sf.cpu(), S_r) < 2e-2
    for a, b in zip((q, k, v, beta, g), ins):
        assert _rel_err(a.grad.cpu(), b.grad) < 4e-2


# ------------------------------ grouped (MoE) GEMM ---------------------------
def test_grouped_linear_fwd_bwd():
    from cverl_b200.models.moe import sort_by_expert
    from cverl_b200.ops.grouped_gemm import grouped_linear, grouped_linear_ref
    torch.manual_seed(21)
    E, N, K, n = 6, 192, 256, 700
    ids = torch.randint(0, E, (n,), device=_dev())
    ids[ids == 4] = 3                                   # an expert without tokens
    order, dest, tile_group, offsets, m_pad = sort_by_expert(ids, E)
    rows = torch.randn(n, K, device=_dev(), dtype=torch.bfloat16)
    x = torch.zeros(m_pad, K, device=_dev(), dtype=torch.bfloat16).index_copy(0, dest, rows[order]).requires_grad_(True)
    w = (0.1 * torch.randn(E, N, K, device=_dev())).to(torch.bfloat16).requires_grad_(True)
    y = grouped_linear(x, w, tile_group, offsets)
    ref = grouped_linear_ref(x.detach(), w.detach(), tile_group)
    assert _rel_err(y, ref) < 6e-3
    dy = torch.randn_like(y)
    dy[(tile_group.long().repeat_interleave(128) < 0)] = 0
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    rows_group = tile_group.long().repeat_interleave(128)
    yr = torch.zeros(m_pad, N, device=_dev())
    for e in range(E):
        sel = (rows_group == e).nonzero().squeeze(-1)
        if sel.numel():
            yr = yr.index_add(0, sel, xr[sel] @ wr[e].t())
    yr.backward(dy.float())
    assert _rel_err(x.grad, xr.grad) < 8e-3
    assert _rel_err(w.grad, wr.grad) < 8e-3


def test_expert_layout_kernel_matches_tensor_ops():
    """The bookkeeping kernels (stable counting sort into 128-row padded expert segments) give the same rows, segment
    bounds and tile table as the argsort / bincount / cumsum / searchsorted version, for experts without tokens,
    unused entries (id == E), one block and many blocks; an id outside the table is reported, not followed."""
    from cverl_b200 import _native as nv
    from cverl_b200.models.moe import expert_layout, sort_by_expert
    g = torch.Generator(device=_dev()).manual_seed(31)
    for E, n, unused in ((6, 700, False), (128, 40000, False), (16, 5000, True), (256, 300, True), (3, 1, False)):
        ids = torch.randint(0, E + (1 if unused else 0), (n,), device=_dev(), generator=g)
        if E > 4:
            ids[ids == 4] = 3                                   # an expert without tokens
        row, tile_group, offsets, m_pad = expert_layout(ids, E)
        order, dest, tg_ref, off_ref, m_ref = sort_by_expert(ids, E)
        want = torch.empty_like(order)
        want[order] = dest
        nv.check_status()
        assert m_pad == m_ref and torch.equal(offsets, off_ref) and torch.equal(tile_group, tg_ref)
        assert torch.equal(row, want)
        assert int(row.max()) < m_pad and row.unique().numel() == n
    bad = torch.tensor([0, 1, 99, -5, 2], device=_dev())
    row, _, _, m_pad = expert_layout(bad, 4)
    torch.cuda.synchronize()
    assert int(row.min()) >= 0 and int(row.max()) < m_pad          # every row stays inside the buffer
    with pytest.raises(RuntimeError):
        nv.check_status()                                          # ... and the bad ids are reported


def test_expert_parallel_row_plan_on_the_layout_kernels_matches_tensor_ops():
    """Destination rows of routed entries: the CUDA path (stable grouping by the layout kernels) equals the
    sort-based tensor-op statement, including the entries that do not fit the receive buffer."""
    from cverl_b200.parallel.ep_symm import plan_rows
    g = torch.Generator().manual_seed(4)
    for world, n, cap in ((2, 96, 1000), (8, 5000, 700), (4, 1, 10)):
        dst = torch.randint(0, world, (n,), generator=g)
        table = torch.randint(0, 300, (world, world), generator=g)
        for rank in (0, world - 1):
            table[rank] = torch.bincount(dst, minlength=world)
            want = plan_rows(table, rank, dst, cap)
            got = plan_rows(table.to(_dev()), rank, dst.to(_dev()), cap)
            for a, b in zip(got, want):
                assert torch.equal(a.cpu(), b)


def test_router_ids_stay_in_table_for_non_finite_logits():
    """Rows of NaN / infinite activations still give k distinct expert ids inside [0, E): the ids index tables
    further down the layer, so they must never leave them whatever the data."""
    from cverl_b200.ops.router import route
    torch.manual_seed(3)
    T, H, E, k = 64, 128, 32, 8
    x = torch.randn(T, H, device=_dev(), dtype=torch.bfloat16)
    x[5] = float("nan")
    x[9, :7] = float("inf")
    x[17] = float("-inf")
    gate = (0.1 * torch.randn(E, H, device=_dev())).to(torch.bfloat16)
    idx, w = route(x, gate, k, True)
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0 and int(idx.max()) < E
    assert all(len(set(row.tolist())) == k for row in idx.cpu())
    good = torch.ones(T, dtype=torch.bool)
    good[[5, 9, 17]] = False
    assert torch.isfinite(w.cpu()[good]).all()


def test_moe_model_gpu_matches_cpu():
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.qwen3_5 import Qwen35Model
    cfg = Qwen35TextConfig(model_type="qwen3_moe", vocab_size=1024, hidden_size=256, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
                           moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2, rope_theta=1e4,
                           tie_word_embeddings=False)
    gm = Qwen35Model(cfg, dtype=torch.bfloat16, device=_dev())
    gm.init_weights(seed=5)
    cm = Qwen35Model(cfg, dtype=torch.float32)
    cm.flat.flat.copy_(gm.flat.flat.float().cpu())
    ids = torch.randint(1, cfg.vocab_size, (2, 64))
    lg = gm.response_logprobs(ids.to(_dev()), 16)
    lc = cm.response_logprobs(ids, 16)
    assert (lg.cpu() - lc).abs().mean().item() < 0.03
    lg.sum().backward()


def test_gdn_chunk_kernels_strided_inputs():
    """Chunk prep / scan / output kernels on q, k, v read in place from one [B, T, 3*H*128] buffer."""
    from cverl_b200.ops import gdn, gdn_native
    torch.manual_seed(6)
    B, T, H = 2, 256, 3
    mixed = torch.randn(B, T, 3 * H * 128, device=_dev(), dtype=torch.bfloat16)
    q, k, v = (m.reshape(B, T, H, 128) for m in mixed.split(H * 128, dim=-1))
    assert gdn_native.chunk_supported(q, k, v)
    beta = torch.sigmoid(torch.randn(B, T, H, device=_dev()))
    g = -0.5 * torch.rand(B, T, H, device=_dev())
    S0 = 0.1 * torch.randn(B, H, 128, 128, device=_dev())
    scale = 128 ** -0.5
    o, Sf, Vn, SsT, _ = gdn_native.chunk_forward(q, k, v, beta, g, S0, scale)
    qq, kk, vv = (t.float().cpu() for t in (q, k, v))
    o_r, S_r = gdn.gdn_recurrent_ref((gdn.l2norm(qq) * scale).transpose(1, 2), gdn.l2norm(kk).transpose(1, 2),
                                     vv.transpose(1, 2), beta.cpu().transpose(1, 2), g.cpu().transpose(1, 2), S0.cpu())
    assert _rel_err(o.cpu(), o_r.transpose(1, 2)) < 2e-2
    assert _rel_err(Sf.cpu(), S_r) < 2e-2
    # the prep kernel against the PyTorch chunk-local algebra
    pre = gdn_native.chunk_prep(q, k, v, beta, g, scale, want_aux=True)
    blk = lambda x: x.float().transpose(1, 2).reshape(B, H, T // 64, 64, -1)
    L = gdn._chunk_local(blk(q), blk(k), blk(v), beta.transpose(1, 2).reshape(B, H, T // 64, 64),
                         g.transpose(1, 2).reshape(B, H, T // 64, 64), scale)
    for name, ref in (("W", L["W"]), ("U", L["U"]), ("Kd", L["Kdec"]), ("Qd", L["Qd"]), ("P", L["P"]), ("Tm", L["T"])):
        assert _rel_err(pre[name], ref) < 2e-2, name
    assert _rel_err(pre["egam"], L["egam"]) < 1e-4


@pytest.mark.parametrize("decay", [0.5, 8.0])
def test_gdn_chunk_backward_kernel(decay):
    """Native chunked forward + backward (prep, scans, chunk-local backward kernel) against autograd through the
    token-by-token fp32 recurrence, with an initial state and a gradient on the final state.  decay = 8: the
    cumulative log-decay of a chunk reaches -250, where e^{c} underflows and e^{-c} overflows on their own (the
    kernels may only ever exponentiate differences)."""
    from cverl_b200.ops import gdn, gdn_native
    torch.manual_seed(8)
    B, T, H = 2, 256, 3
    mixed = torch.randn(B, T, 3 * H * 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    q, k, v = (m.reshape(B, T, H, 128) for m in mixed.split(H * 128, dim=-1))
    assert gdn_native.chunk_supported(q, k, v) and gdn_native.chunk_bwd_enabled()
    beta = torch.sigmoid(torch.randn(B, T, H, device=_dev())).requires_grad_(True)
    g = (-decay * torch.rand(B, T, H, device=_dev())).requires_grad_(True)
    S0 = (0.1 * torch.randn(B, H, 128, 128, device=_dev())).requires_grad_(True)
    scale = 128 ** -0.5
    o, Sf = gdn.gated_delta_rule_fused(q, k, v, beta, g, S0, scale=scale)
    do = torch.randn_like(o)
    dSf = 0.05 * torch.randn_like(Sf)
    torch.autograd.backward([o, Sf], [do, dSf])
    from cverl_b200 import _native as nv
    nv.check_status()
    mr = mixed.detach().float().cpu().requires_grad_(True)
    qq, kk, vv = (m.reshape(B, T, H, 128) for m in mr.split(H * 128, dim=-1))
    bb, gg, ss = (t.detach().float().cpu().requires_grad_(True) for t in (beta, g, S0))
    o_r, S_r = gdn.gdn_recurrent_ref((gdn.l2norm(qq) * scale).transpose(1, 2), gdn.l2norm(kk).transpose(1, 2),
                                     vv.transpose(1, 2), bb.transpose(1, 2), gg.transpose(1, 2), ss)
    torch.autograd.backward([o_r.transpose(1, 2), S_r], [do.float().cpu(), dSf.cpu()])
    gq, gk, gv = (m for m in mixed.grad.float().cpu().split(H * 128, dim=-1))
    rq, rk, rv = (m for m in mr.grad.split(H * 128, dim=-1))
    for name, a, b in (("dq", gq, rq), ("dk", gk, rk), ("dv", gv, rv), ("dbeta", beta.grad.cpu(), bb.grad),
                       ("dg", g.grad.cpu(), gg.grad), ("dS0", S0.grad.cpu(), ss.grad)):
        assert torch.isfinite(a).all(), name
        if b.norm() < 1e-5:        # fully decayed away (strong decay): both must vanish
            assert a.norm() < 1e-3, (name, float(a.norm()))
        else:
            # under strong decay dg and dbeta are differences of nearly equal row dot products
            assert _rel_err(a, b) < (4e-2 if decay < 1 else 8e-2), (name, _rel_err(a, b))
    assert torch.isfinite(o).all() and _rel_err(o.detach().cpu(), o_r.transpose(1, 2).detach()) < 2e-2


def test_gdn_packed_entry_matches_split_entry():
    """The packed entry (gradients of q | k | v written in place into one buffer by the backward kernel) gives
    bit-identical outputs and gradients to the entry on three split views."""
    from cverl_b200.ops import gdn
    from cverl_b200 import _native as nv
    torch.manual_seed(9)
    B, T, H = 2, 192, 3
    base = torch.randn(B, T, 3 * H * 128, device=_dev(), dtype=torch.bfloat16)
    beta0 = torch.sigmoid(torch.randn(B, T, H, device=_dev()))
    g0 = -0.5 * torch.rand(B, T, H, device=_dev())
    scale = 128 ** -0.5
    res = []
    for packed in (True, False):
        mixed = base.clone().requires_grad_(True)
        beta, g = beta0.clone().requires_grad_(True), g0.clone().requires_grad_(True)
        if packed:
            o, Sf = gdn.gated_delta_rule_packed(mixed, beta, g, None, scale=scale, heads=H)
            assert type(o.grad_fn).__name__.startswith("_GdnPacked")
        else:
            q, k, v = (m.reshape(B, T, H, 128) for m in mixed.split(H * 128, dim=-1))
            o, Sf = gdn.gated_delta_rule_fused(q, k, v, beta, g, None, scale=scale)
        torch.manual_seed(10)
        o.backward(torch.randn_like(o))
        nv.check_status()
        res.append((o.detach(), Sf, mixed.grad, beta.grad, g.grad))
    for a, b in zip(*res):
        assert torch.equal(a, b)


def test_gdn_state_modes_give_identical_gradients(monkeypatch):
    """Keeping the per-chunk states for the backward pass, regenerating them with one more forward-scan launch, and
    letting a byte budget decide are the same computation: outputs and gradients agree bit for bit, with and
    without an initial state, and the regenerating mode saves less."""
    from cverl_b200.ops import gdn, gdn_native
    from cverl_b200 import _native as nv
    torch.manual_seed(11)
    B, T, H = 2, 512, 2
    base = torch.randn(B, T, 3 * H * 128, device=_dev(), dtype=torch.bfloat16)
    beta0 = torch.sigmoid(torch.randn(B, T, H, device=_dev()))
    g0 = -0.5 * torch.rand(B, T, H, device=_dev())
    S0 = 0.1 * torch.randn(B, H, 128, 128, device=_dev())
    scale = 128 ** -0.5
    for init in (None, S0):
        res, saved = [], []
        for env in ({"CVERL_LINEAR_ATTN_STATE_MODE": "full"}, {"CVERL_LINEAR_ATTN_STATE_MODE": "none"},
                    {"CVERL_LINEAR_ATTN_STATE_MODE": "chunk", "CVERL_LINEAR_ATTN_CHECKPOINT_MAX_BYTES_MB": "1"},
                    {"CVERL_LINEAR_ATTN_SAVE_STATES": "1"}):
            for key in ("CVERL_LINEAR_ATTN_STATE_MODE", "CVERL_LINEAR_ATTN_CHECKPOINT_MAX_BYTES_MB",
                        "CVERL_LINEAR_ATTN_SAVE_STATES"):
                monkeypatch.delenv(key, raising=False)
            for key, val in env.items():
                monkeypatch.setenv(key, val)
            mixed = base.clone().requires_grad_(True)
            beta, g = beta0.clone().requires_grad_(True), g0.clone().requires_grad_(True)
            s0 = init.clone().requires_grad_(True) if init is not None else None
            o, Sf = gdn.gated_delta_rule_packed(mixed, beta, g, s0, scale=scale, heads=H)
            saved.append(sum(t.numel() * t.element_size() for t in o.grad_fn.saved_tensors))
            torch.manual_seed(12)
            (o.float() * torch.randn_like(o, dtype=torch.float32)).sum().backward()
            nv.check_status()
            res.append((o.detach(), Sf.detach(), mixed.grad, beta.grad, g.grad) + ((s0.grad,) if s0 is not None else ()))
        for other in res[1:]:
            for a, b in zip(res[0], other):
                assert torch.equal(a, b)
        # 2 x 2 x 8 chunk states of 48 KB (S and V') are 1.5 MB: over the 1 MB budget, so that mode regenerates too
        assert saved[1] < saved[0] and saved[3] == saved[0] and saved[2] == saved[1]
    monkeypatch.setenv("CVERL_LINEAR_ATTN_STATE_MODE", "sometimes")
    with pytest.raises(ValueError):
        gdn_native.state_mode()
