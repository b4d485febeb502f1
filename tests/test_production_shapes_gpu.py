"""The attention and Gated-DeltaNet kernels at the shapes the 0.8B benchmark runs them with (sequence 1280, head
dim 256, 8 query / 2 key-value heads; scan over 1280 tokens with 16 heads), against fp32 statements of the ops.
The references are evaluated on a sub-sample (a few sequences / heads) to keep the tests quick; the kernels run
on the full batch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_attention_at_benchmark_shape():
    from cverl_b200 import _native as nv
    from cverl_b200.ops import attention, attention_native
    torch.manual_seed(21)
    B, S, Hq, Hkv, D = 8, 1280, 8, 2, 256
    q = torch.randn(B * S, Hq, D, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B * S, Hkv, D, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B * S, Hkv, D, device="cuda").bfloat16().requires_grad_(True)
    assert attention_native.supported(q, k, v, S)
    o = attention_native.causal_attention(q, k, v, B, S)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    nv.check_status()
    for b in (0, B - 1):                                   # first and last sequence of the batch, fp32 eager
        sl = slice(b * S, (b + 1) * S)
        qr, kr, vr = (t.detach()[sl].float().requires_grad_(True) for t in (q, k, v))
        o_r = attention.causal_attention_ref(qr, kr, vr, 1, S)
        o_r.backward(do[sl].float())
        assert _rel(o[sl], o_r) < 1e-2
        assert _rel(q.grad[sl], qr.grad) < 2e-2
        assert _rel(k.grad[sl], kr.grad) < 2e-2
        assert _rel(v.grad[sl], vr.grad) < 2e-2


def test_gated_delta_rule_at_benchmark_shape():
    from cverl_b200 import _native as nv
    from cverl_b200.ops import gdn, gdn_native
    torch.manual_seed(22)
    B, T, H = 4, 1280, 16
    mixed = torch.randn(B, T, 3 * H * 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q, k, v = (m.reshape(B, T, H, 128) for m in mixed.split(H * 128, dim=-1))
    assert gdn_native.chunk_supported(q, k, v)
    beta = torch.sigmoid(torch.randn(B, T, H, device="cuda")).requires_grad_(True)
    g = (-0.3 * torch.rand(B, T, H, device="cuda")).requires_grad_(True)
    scale = 128 ** -0.5
    o, Sf = gdn.gated_delta_rule_packed(mixed, beta, g, None, scale=scale, heads=H)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    nv.check_status()
    assert torch.isfinite(o).all() and torch.isfinite(mixed.grad).all()
    # fp32 token-by-token recurrence on one sequence and three heads (first, middle, last)
    b, heads = B - 1, [0, H // 2, H - 1]
    gq, gk, gv = (m.reshape(B, T, H, 128) for m in mixed.grad.split(H * 128, dim=-1))
    qq, kk, vv = (t.detach()[b:b + 1, :, heads].float().cpu().requires_grad_(True) for t in (q, k, v))
    bb, gg = (t.detach()[b:b + 1, :, heads].float().cpu().requires_grad_(True) for t in (beta, g))
    o_r, S_r = gdn.gdn_recurrent_ref((gdn.l2norm(qq) * scale).transpose(1, 2), gdn.l2norm(kk).transpose(1, 2),
                                     vv.transpose(1, 2), bb.transpose(1, 2), gg.transpose(1, 2))
    o_r = o_r.transpose(1, 2)
    o_r.backward(do[b:b + 1, :, heads].float().cpu())
    assert _rel(o[b:b + 1, :, heads].cpu(), o_r) < 2e-2
    assert _rel(Sf[b:b + 1, heads].cpu(), S_r) < 2e-2
    for name, a, r in (("dq", gq, qq), ("dk", gk, kk), ("dv", gv, vv)):
        assert _rel(a[b:b + 1, :, heads].cpu(), r.grad) < 4e-2, name
    assert _rel(beta.grad[b:b + 1, :, heads].cpu(), bb.grad) < 6e-2
    assert _rel(g.grad[b:b + 1, :, heads].cpu(), gg.grad) < 8e-2
