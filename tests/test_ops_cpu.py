"""CPU statements of the fused linear-attention glue ops: the wrappers must equal the plain formulation
(values and gradients) when the native kernels are not in play."""
import torch
import torch.nn.functional as F


def test_conv1d_silu_split_cpu_equals_split_then_conv():
    from cverl_b200.ops import conv1d_silu, conv1d_silu_split
    torch.manual_seed(0)
    B, S, sizes = 2, 11, [16, 8, 4, 4]
    base = torch.randn(B, S, sum(sizes))
    w0 = 0.5 * torch.randn(sizes[0], 4)
    outs = []
    for fused in (True, False):
        proj, w = base.clone().requires_grad_(True), w0.clone().requires_grad_(True)
        if fused:
            y, z, b, a = conv1d_silu_split(proj, w, sizes)
        else:
            x, z, b, a = proj.split(sizes, dim=-1)
            y = conv1d_silu(x, w)
        (y.sum() + (z ** 2).sum() + torch.sigmoid(b).sum() + (a * 3).sum()).backward()
        outs.append((y.detach(), proj.grad, w.grad))
    for u, v in zip(*outs):
        assert torch.allclose(u, v, atol=1e-6)


def test_gdn_gates_cpu_matches_formula_and_grads():
    from cverl_b200.ops import gdn
    torch.manual_seed(1)
    b = torch.randn(3, 7, 4, requires_grad=True)
    a = (3 * torch.randn(3, 7, 4)).requires_grad_(True)
    A_log = torch.log(torch.empty(4).uniform_(1, 8)).requires_grad_(True)
    dt_bias = torch.empty(4).uniform_(-1, 1).requires_grad_(True)
    beta, g = gdn.gdn_gates(b, a, A_log, dt_bias)
    assert beta.dtype == torch.float32 and g.shape == a.shape
    assert torch.allclose(beta, torch.sigmoid(b)) and (g <= 0).all()
    assert torch.allclose(g, -torch.exp(A_log) * F.softplus(a + dt_bias))
    (beta.sum() + g.sum()).backward()
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in (b, a, A_log, dt_bias))
    assert torch.allclose(A_log.grad, g.detach().sum((0, 1)), atol=1e-5)   # dg/dA_log = g


def test_gated_delta_rule_packed_cpu_equals_split_entry():
    from cverl_b200.ops import gdn
    torch.manual_seed(2)
    B, T, H, d = 1, 70, 2, 8
    base = torch.randn(B, T, 3 * H * d)
    beta0 = torch.sigmoid(torch.randn(B, T, H))
    g0 = -0.3 * torch.rand(B, T, H)
    outs = []
    for packed in (True, False):
        mixed = base.clone().requires_grad_(True)
        beta, g = beta0.clone().requires_grad_(True), g0.clone().requires_grad_(True)
        if packed:
            o, Sf = gdn.gated_delta_rule_packed(mixed, beta, g, None, scale=d ** -0.5, heads=H)
        else:
            q, k, v = (m.reshape(B, T, H, d) for m in mixed.split(H * d, dim=-1))
            o, Sf = gdn.gated_delta_rule_fused(q, k, v, beta, g, None, scale=d ** -0.5)
        (o.sum() + 0.1 * Sf.sum()).backward()
        outs.append((o.detach(), Sf.detach(), mixed.grad, beta.grad, g.grad))
    for u, v in zip(*outs):
        assert torch.allclose(u, v, atol=1e-5)


def test_gated_rmsnorm_cpu_accepts_token_major_gate():
    from cverl_b200.ops import gated_rmsnorm
    torch.manual_seed(3)
    T, Hh, D = 9, 2, 8
    x = torch.randn(T, Hh, D, requires_grad=True)
    z = torch.randn(T, Hh * D, requires_grad=True)          # the projection's column group, not yet split by head
    w = torch.randn(D, requires_grad=True)
    y = gated_rmsnorm(x, z, w, 1e-6)
    y2 = gated_rmsnorm(x, z.reshape(T, Hh, D), w, 1e-6)
    assert torch.allclose(y, y2)
    y.sum().backward()
    assert z.grad.shape == z.shape and torch.isfinite(z.grad).all()
