"""sm_100a kernels against plain PyTorch fp32 references of the same ops."""
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


# ------------------------------- norms --------------------------------------
@pytest.mark.parametrize("D", [64, 128, 256, 1024, 2048, 3584])
def test_add_rmsnorm(D):
    from cverl_b200.ops import add_rmsnorm
    from cverl_b200.ops.norm import rmsnorm_ref
    torch.manual_seed(4)
    T = 333
    x = torch.randn(T, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (0.1 * torch.randn(D, device=_dev())).to(torch.bfloat16).requires_grad_(True)
    y, h = add_rmsnorm(x, r, w, 1e-6, 1.0)
    dy, dh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [dy, dh])
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    hr = (xr + rr)
    yr = rmsnorm_ref(hr, wr, 1e-6, 1.0)
    torch.autograd.backward([yr, hr], [dy.float(), dh.float()])
    assert _rel_err(h, hr) < 5e-3
    assert _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(r.grad, rr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


def test_rmsnorm_no_residual_and_main_grad():
    from cverl_b200.ops import rmsnorm
    from cverl_b200.ops.norm import rmsnorm_ref
    torch.manual_seed(5)
    x = torch.randn(100, 1024, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(1024, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w.main_grad = torch.zeros(1024, device=_dev())
    y = rmsnorm(x, w, 1e-6, 0.0)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    rmsnorm_ref(xr, wr, 1e-6, 0.0).backward(dy.float())
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.main_grad, wr.grad) < 1e-3


def test_gated_rmsnorm():
    from cverl_b200.ops import gated_rmsnorm
    from cverl_b200.ops.norm import rmsnorm_ref
    torch.manual_seed(6)
    x = torch.randn(200, 16, 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    z = torch.randn(200, 16, 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = gated_rmsnorm(x, z, w, 1e-6)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, zr, wr = (t.detach().float().requires_grad_(True) for t in (x, z, w))
    yr = rmsnorm_ref(xr, wr, 1e-6, 0.0, gate=zr)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(z.grad, zr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("D,rot,use_norm", [(256, 64, True), (128, 128, True), (128, 32, False)])
def test_headnorm_rope(D, rot, use_norm):
    from cverl_b200.ops import headnorm_rope, rope_tables
    from cverl_b200.ops.norm import headnorm_rope_ref
    torch.manual_seed(7)
    T, Hh, S = 300, 4, 100
    big = torch.randn(T, Hh, 2 * D, device=_dev(), dtype=torch.bfloat16)
    x = big[..., :D].detach().requires_grad_(True)  # strided view, as the q half of a q|gate projection
    w = (0.1 * torch.randn(D, device=_dev())).to(torch.bfloat16).requires_grad_(True)
    cos, sin = rope_tables(S, rot, 1e7, _dev())
    pos = (torch.arange(T, device=_dev()) % S).to(torch.int32)
    y = headnorm_rope(x, w, cos, sin, pos, rot, 1e-6, 1.0, use_norm)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = headnorm_rope_ref(xr, wr, cos, sin, pos.long(), rot, 1e-6, 1.0, use_norm)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2
    if use_norm:
        assert _rel_err(w.grad, wr.grad) < 2e-2


# ---------------------------- activations -----------------------------------
def test_swiglu():
    from cverl_b200.ops import swiglu
    from cverl_b200.ops.activation import swiglu_ref
    torch.manual_seed(8)
    gu = torch.randn(500, 2 * 3584, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = swiglu(gu)
    dy = torch.randn_like(y)
    y.backward(dy)
    gr = gu.detach().float().requires_grad_(True)
    yr = swiglu_ref(gr)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 6e-3
    assert _rel_err(gu.grad, gr.grad) < 8e-3


def test_siggate_strided_gate():
    from cverl_b200.ops import siggate
    torch.manual_seed(9)
    T, Hh, D = 257, 8, 256
    qg = torch.randn(T, Hh, 2 * D, device=_dev(), dtype=torch.bfloat16)
    g = qg[..., D:].detach().requires_grad_(True)
    a = torch.randn(T, Hh, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = siggate(a, g)
    dy = torch.randn_like(y)
    y.backward(dy)
    ar, gr = a.detach().float().requires_grad_(True), g.detach().float().requires_grad_(True)
    yr = ar * torch.sigmoid(gr)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 6e-3
    assert _rel_err(a.grad, ar.grad) < 8e-3
    assert _rel_err(g.grad, gr.grad) < 8e-3


@pytest.mark.parametrize("path", ["tma", "plain"])
@pytest.mark.parametrize("S,Cc,KW", [(5, 256, 4), (64, 256, 4), (200, 256, 4), (131, 320, 3), (70, 40, 4), (129, 64, 2)])
def test_conv1d_silu(S, Cc, KW, path, monkeypatch):
    """Both backward kernels (the TMA-tiled one takes C % 64 == 0 and falls back otherwise), partial channel
    tiles, sequence lengths that end inside a tile, a column slice of a wider tensor as the input."""
    from cverl_b200.ops import conv1d_silu
    from cverl_b200.ops.activation import conv1d_silu_ref
    from cverl_b200 import _native as nv
    monkeypatch.setenv("CVERL_B200_CONV_BWD", path)
    torch.manual_seed(10)
    B = 3
    wide = torch.randn(B, S, Cc + 64, device=_dev(), dtype=torch.bfloat16)
    x = wide[:, :, 32:32 + Cc].detach().requires_grad_(True)
    w = (0.5 * torch.randn(Cc, KW, device=_dev())).to(torch.bfloat16).requires_grad_(True)
    y = conv1d_silu(x, w)
    nv.check_status(_dev())
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = conv1d_silu_ref(xr, wr)
    yr.backward(dy.float())
    nv.check_status(_dev())
    assert _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


def test_embedding_fwd_bwd():
    from cverl_b200.ops import embedding
    torch.manual_seed(11)
    V, H = 1000, 256
    table = torch.randn(V, H, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    table.main_grad = torch.zeros(V, H, device=_dev())
    ids = torch.randint(0, V, (4, 77), device=_dev())
    out = embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    dout = torch.randn_like(out)
    out.backward(dout)
    ref = torch.zeros(V, H, device=_dev()).index_add_(0, ids.reshape(-1), dout.reshape(-1, H).float())
    assert _rel_err(table.main_grad, ref) < 1e-5
    # vocab-parallel shard: ids outside the shard give zero rows
    half = embedding(ids, table.detach()[500:], vocab_lo=500)
    assert torch.equal(half[ids < 500], torch.zeros_like(half[ids < 500]))


# ------------------------------- RL math ------------------------------------
def _rl_data(rows=64, cols=512, seed=0):
    g = torch.Generator().manual_seed(seed)
    lp = -2 + 0.5 * torch.randn(rows, cols, generator=g)
    old = lp + 0.05 * torch.randn(rows, cols, generator=g)
    ref = lp + 0.1 * torch.randn(rows, cols, generator=g)
    adv = torch.randn(rows, cols, generator=g)
    lens = torch.randint(32, cols + 1, (rows,), generator=g)
    mask = (torch.arange(cols)[None, :] < lens[:, None]).float()
    return [t.to(_dev()) for t in (lp, old, ref, adv, mask)]


def test_rl_masked_and_kl_kernels():
    from cverl_b200.ops import rl
    lp, old, ref, adv, mask = _rl_data()
    assert abs(rl.fused_masked_mean(lp, mask).item() - rl.masked_mean(lp, mask).item()) < 1e-5
    torch.testing.assert_close(rl.fused_masked_whiten(lp, mask), rl.masked_whiten(lp, mask), rtol=1e-4, atol=1e-5)
    for kind in ("k1", "abs", "k2", "k3"):
        torch.testing.assert_close(rl.fused_kl_penalty(lp, ref, kind), rl.kl_penalty(lp, ref, kind), rtol=1e-5,
                                   atol=1e-6)


def test_rl_gae_grpo_kernels():
    from cverl_b200.ops import rl
    lp, old, ref, adv, mask = _rl_data(rows=64, cols=128, seed=1)
    rew = torch.zeros_like(lp)
    rew[:, 5] = torch.bernoulli(torch.full((64,), 0.5, device=_dev()))
    val = torch.randn_like(lp)
    a, r = rl.fused_gae(rew, val, mask, 1.0, 0.95)
    at, rt = rl.gae_advantage_return(rew, val, mask, 1.0, 0.95)
    torch.testing.assert_close(a, at, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(r, rt, rtol=1e-5, atol=1e-5)
    gid = torch.arange(64, device=_dev()) // 8
    ga, _ = rl.fused_grpo_advantage(rew, mask, gid)
    gt, _ = rl.grpo_outcome_advantage(rew, mask, gid)
    torch.testing.assert_close(ga, gt, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("agg", [0, 1, 2])
def test_rl_ppo_loss_kernel(agg):
    from cverl_b200.ops import rl
    lp, old, ref, adv, mask = _rl_data(seed=2 + agg)
    metrics, grad = rl.fused_ppo_loss(old, lp, adv, mask, ref, agg=agg, kl_coef=0.01, kl_penalty_kind="k3")
    x = lp.clone().requires_grad_(True)
    res = rl.ppo_clipped_loss(old, x, adv, mask, agg=agg)
    kl = rl.masked_mean(rl.kl_penalty(x, ref, "k3"), mask)
    (res.pg_loss + 0.01 * kl).backward()
    want = torch.stack([res.pg_loss, res.pg_clipfrac, res.ppo_kl, res.pg_clipfrac_lower, kl]).detach()
    torch.testing.assert_close(metrics[:5], want, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(grad, x.grad, rtol=1e-4, atol=1e-8)


# ------------------------------- optimizer ----------------------------------
@pytest.mark.parametrize("master", [True, False])
def test_flat_adamw_kernel(master):
    from cverl_b200.ops import optim
    torch.manual_seed(13)
    n = 100003
    p0 = torch.randn(n, device=_dev())
    g = torch.randn(n, device=_dev())
    model = p0.to(torch.bfloat16)
    mast = p0.clone() if master else None
    m, v = torch.zeros(n, device=_dev()), torch.zeros(n, device=_dev())
    ref_p = (p0.clone() if master else model.float())
    rm, rv = torch.zeros(n), torch.zeros(n)
    rp = ref_p.cpu()
    sq = optim.sumsq(g)
    assert abs(sq.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-5
    clip = optim.clip_scale(sq, 1.0)
    assert abs(clip[0].item() - 1.0 / (sq.sqrt().item() + 1e-6)) < 1e-6
    for step in (1, 2, 3):
        gg = g.clone()
        optim.flat_adamw_step(gg, mast, model, m, v, clip=clip, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                              weight_decay=0.01, step=step, zero_grad=True)
        assert gg.abs().max().item() == 0.0
        gc = (g * clip[0]).cpu()
        rm.mul_(0.9).add_(gc, alpha=0.1)
        rv.mul_(0.95).addcmul_(gc, gc, value=0.05)
        rp = rp * (1 - 1e-2 * 0.01)
        rp = rp - (1e-2 / (1 - 0.9 ** step)) * rm / ((rv / (1 - 0.95 ** step)).sqrt() + 1e-8)
        if not master:
            rp = rp.to(torch.bfloat16).float()
    if master:
        torch.testing.assert_close(mast.cpu(), rp, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(model.float().cpu(), rp.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(m.cpu(), rm, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("norm_topk", [True, False])
def test_router_topk_kernel(norm_topk):
    from cverl_b200.ops import router
    torch.manual_seed(4)
    T, H, E, k = 1000, 256, 128, 8
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    gw = (0.2 * torch.randn(E, H, device="cuda")).bfloat16().requires_grad_(True)
    idx, w = router.route(x, gw, k, norm_topk)
    xr, gr = x.detach().float().requires_grad_(True), gw.detach().float().requires_grad_(True)
    ridx, rw = router.route_ref(xr, gr, k, norm_topk)
    # same experts (as sets; ties and bf16-vs-fp32 logits may reorder near-equal entries) on almost every token
    same = (idx.sort(-1).values == ridx.sort(-1).values).all(-1)
    assert same.float().mean() > 0.97
    order, rorder = idx.argsort(-1), ridx.argsort(-1)
    torch.testing.assert_close(w.gather(-1, order)[same], rw.gather(-1, rorder)[same], rtol=2e-2, atol=2e-3)
    assert torch.allclose(w.sum(-1), torch.ones(T, device="cuda"), atol=1e-4) or not norm_topk
    dw = torch.randn_like(w)
    w.backward(dw)
    # reference gradient with the kernel's own selection, so that differing tie-breaks do not matter
    logits = xr @ gr.t()
    sel = logits.gather(-1, idx)
    rw2 = torch.softmax(sel, -1) if norm_topk else torch.softmax(logits, -1).gather(-1, idx)
    rw2.backward(dw)
    assert ((x.grad.float() - xr.grad).norm() / xr.grad.norm()).item() < 3e-2
    assert ((gw.grad.float() - gr.grad).norm() / gr.grad.norm()).item() < 3e-2


@pytest.mark.parametrize("D,Hq,Hkv", [(256, 4, 1), (128, 4, 2)])
def test_attention_tcgen05_forward_backward(D, Hq, Hkv):
    """tcgen05 attention kernels against the fp32 eager statement (GQA, causal), forward and backward."""
    from cverl_b200.ops import attention, attention_native
    torch.manual_seed(12)
    B, S = 2, 384
    q = torch.randn(B * S, Hq, D, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B * S, Hkv, D, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B * S, Hkv, D, device="cuda").bfloat16().requires_grad_(True)
    assert attention_native.supported(q, k, v, S)
    o = attention_native.causal_attention(q, k, v, B, S)
    do = torch.randn_like(o)
    o.backward(do)
    from cverl_b200 import _native as nv
    nv.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o_r = attention.causal_attention_ref(qr, kr, vr, B, S)
    o_r.backward(do.float())
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(o, o_r) < 1e-2
    assert rel(q.grad, qr.grad) < 2e-2
    assert rel(k.grad, kr.grad) < 2e-2
    assert rel(v.grad, vr.grad) < 2e-2


def test_attention_block_offsets_merge_to_full_attention():
    """Two key ranges run as separate blocks (the second one causal with position offsets) merge, through their
    LSEs, to the full causal attention: the contract ring attention relies on."""
    from cverl_b200.ops import attention, attention_native
    torch.manual_seed(13)
    B, S, H, D = 1, 256, 2, 128
    q = torch.randn(B, S, H, D, device="cuda").bfloat16()
    k = torch.randn(B, S, H, D, device="cuda").bfloat16()
    v = torch.randn(B, S, H, D, device="cuda").bfloat16()
    scale = D ** -0.5
    q2 = q[:, 128:].contiguous()                      # queries 128..255 against keys 0..127 (all visible) and 128..255
    o1, l1 = attention_native.attention_block(q2, k[:, :128].contiguous(), v[:, :128].contiguous(), scale, False, 128, 0)
    o2, l2 = attention_native.attention_block(q2, k[:, 128:].contiguous(), v[:, 128:].contiguous(), scale, True, 128, 128)
    lse = torch.logaddexp(l1, l2)
    w1, w2 = (l1 - lse).exp().transpose(1, 2).unsqueeze(-1), (l2 - lse).exp().transpose(1, 2).unsqueeze(-1)
    merged = o1.float() * w1 + o2.float() * w2
    full = attention.causal_attention_ref(q.reshape(S, H, D), k.reshape(S, H, D), v.reshape(S, H, D), B, S)
    ref = full.view(B, S, H, D)[:, 128:].float()
    assert ((merged - ref).norm() / ref.norm()).item() < 1e-2


def test_conv1d_silu_split_matches_split_then_conv():
    """conv1d_silu_split (the backward fills one [B,S,W] gradient buffer in place) against splitting first."""
    from cverl_b200.ops import conv1d_silu, conv1d_silu_split
    from cverl_b200 import _native as nv
    torch.manual_seed(12)
    B, S, sizes = 2, 150, [384, 128, 8, 8]
    base = torch.randn(B, S, sum(sizes), device=_dev(), dtype=torch.bfloat16)
    w0 = (0.5 * torch.randn(sizes[0], 4, device=_dev())).to(torch.bfloat16)
    res = []
    for fused in (True, False):
        proj = base.clone().requires_grad_(True)
        w = w0.clone().requires_grad_(True)
        if fused:
            y, z, b, a = conv1d_silu_split(proj, w, sizes)
            assert type(y.grad_fn).__name__.startswith("_ConvSiluSplit")
        else:
            x, z, b, a = proj.split(sizes, dim=-1)
            y = conv1d_silu(x, w)
        # z gates an RMSNorm over 2 heads of 64: fused, the norm reads z in place from the projection and writes
        # dz straight into the projection-gradient buffer; unfused, both go through copies
        core = torch.linspace(-2, 2, B * S * 128, device=_dev()).view(B * S, 2, 64).to(torch.bfloat16)
        gw = torch.linspace(0.5, 1.5, 64, device=_dev()).to(torch.bfloat16)
        from cverl_b200.ops import gated_rmsnorm
        n = gated_rmsnorm(core, z if fused else z.reshape(B * S, 2, 64), gw, 1e-6)
        loss = (y.float() * torch.linspace(-1, 1, sizes[0], device=_dev())).sum() + \
            (n.float() * torch.linspace(-1, 1, 64, device=_dev())).sum() + torch.sigmoid(b.float()).sum()  # `a`: no grad
        loss.backward()
        nv.check_status(_dev())
        res.append((y.detach(), proj.grad, w.grad, n.detach()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][3], res[1][3])
    assert _rel_err(res[0][2], res[1][2]) < 1e-3          # atomics: summation order differs between runs


@pytest.mark.parametrize("through_split", [True, False])
def test_gdn_gates_kernel(through_split):
    """beta = sigmoid(b), g = -exp(A_log) softplus(a + dt_bias): the fused kernels against the torch statement,
    on column groups of a projection (gradients written through the split op's sink) and on a plain 2-D split."""
    from cverl_b200.ops import conv1d_silu_split
    from cverl_b200.ops import gdn
    from cverl_b200 import _native as nv
    torch.manual_seed(13)
    B, S, H = 2, 96, 16
    sizes = [128, 64, H, H]
    base = (2.0 * torch.randn(B, S, sum(sizes), device=_dev())).to(torch.bfloat16)
    base[0, 0, -1] = 30.0                                  # softplus above its linear threshold
    cw = (0.5 * torch.randn(sizes[0], 4, device=_dev())).to(torch.bfloat16)
    A0 = torch.log(torch.empty(H, device=_dev()).uniform_(1, 8)).to(torch.bfloat16)
    D0 = torch.empty(H, device=_dev()).uniform_(-1, 1).to(torch.bfloat16)
    wb = torch.randn(B, S, H, device=_dev())
    wg = torch.randn(B, S, H, device=_dev())
    res = []
    for fused in (True, False):
        proj = base.clone().requires_grad_(True)
        A_log, dt_bias = A0.clone().requires_grad_(True), D0.clone().requires_grad_(True)
        if through_split:
            y, z, b, a = conv1d_silu_split(proj, cw, sizes)
        else:
            y, z, b, a = proj.view(B * S, -1).split(sizes, dim=-1)
        beta, g = gdn.gdn_gates(b, a, A_log, dt_bias) if fused else gdn.gdn_gates_ref(b, a, A_log, dt_bias)
        if fused:
            assert type(beta.grad_fn).__name__.startswith("_GdnGates")
        loss = (beta.reshape(B, S, H) * wb).sum() + (g.reshape(B, S, H) * wg).sum() + y.float().sum()
        loss.backward()
        nv.check_status(_dev())
        res.append((beta.detach().reshape(-1), g.detach().reshape(-1), proj.grad[..., -2 * H:].float(),
                    A_log.grad.float(), dt_bias.grad.float()))
    for k, tol in zip(range(5), (1e-5, 1e-5, 1e-2, 2e-2, 2e-2)):
        assert torch.isfinite(res[0][k]).all()
        assert _rel_err(res[0][k], res[1][k]) < tol, (k, _rel_err(res[0][k], res[1][k]))


def test_library_fallbacks_are_counted_and_announced():
    """A CUDA call that a native kernel cannot serve warns once per (op, reason), is counted every time, and is an
    error under ``CVERL_B200_STRICT=1``."""
    import os
    import warnings
    from cverl_b200.ops import attention
    from cverl_b200.utils import fallbacks
    fallbacks.reset()
    q = torch.randn(96, 2, 128, device="cuda", dtype=torch.bfloat16)      # sequence length 96: not a multiple of 128
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        attention.causal_attention(q, q, q, 1, 96)
        attention.causal_attention(q, q, q, 1, 96)
    assert fallbacks.total() == 2 and len([w for w in seen if issubclass(w.category, fallbacks.NativeKernelFallback)]) == 1
    os.environ["CVERL_B200_STRICT"] = "1"
    try:
        with pytest.raises(RuntimeError, match="STRICT"):
            attention.causal_attention(q, q, q, 1, 96)
    finally:
        del os.environ["CVERL_B200_STRICT"]
    fallbacks.reset()
    ok = torch.randn(128, 2, 128, device="cuda", dtype=torch.bfloat16)
    attention.causal_attention(ok, ok, ok, 1, 128)
    assert fallbacks.total() == 0


def test_native_cached_decode_matches_forward_and_fp32_step():
    """Prefill + native one-token steps (tcgen05 GEMMs, decode attention over the cache, single-step scan state
    update), eager and replayed from a CUDA graph, against (a) the logits of a full forward over the grown
    sequence and (b) the fp32 PyTorch decode step on the same caches."""
    from cverl_b200 import _native as nv
    from cverl_b200.models import decode
    from cverl_b200.models.config import Qwen35TextConfig
    from cverl_b200.models.qwen3_5 import Qwen35Model
    cfg = Qwen35TextConfig(vocab_size=2048, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=256, intermediate_size=512, linear_key_head_dim=128,
                           linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=4)
    dev = _dev()
    model = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev, with_main_grad=False)
    model.init_weights(seed=9)
    assert decode.native_decode_supported(model)
    g = torch.Generator(device=dev).manual_seed(2)
    B, P, N = 3, 128, 6
    ids = torch.randint(1, cfg.vocab_size, (B, P + N), device=dev, generator=g)
    with torch.no_grad():
        full = model.forward_logits(ids).float()                       # [B, P+N, V]
        for graphed in (False, True):
            state, logits = decode.prefill(model, ids[:, :P], max_len=P + N)
            assert _rel_err(logits, full[:, P - 1]) < 3e-2
            runner = decode.GraphedDecoder(model, state, B) if graphed else None
            for t in range(N - 1):
                tok = ids[:, P + t]
                logits = runner.step(tok) if graphed else decode.decode_step(model, state, tok)
                assert state.length == P + t + 1
                ref = full[:, P + t]
                assert _rel_err(logits, ref) < 4e-2, (graphed, t, _rel_err(logits, ref))
                assert (logits.argmax(-1) == ref.argmax(-1)).float().mean() >= 0.66
            assert int(state.dev["len"]) == P + N and int(state.dev["pos"][0]) == P + N - 1
    nv.check_status()
