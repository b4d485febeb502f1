"""Run-twice, bit-compare checks of the kernels that use no atomics: a data race between warps or CTAs of
a kernel shows up as differing bits between two identical launches."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _same(a, b):
    return a.dtype == b.dtype and torch.equal(a.view(torch.uint8) if a.dtype == torch.bfloat16 else a,
                                              b.view(torch.uint8) if b.dtype == torch.bfloat16 else b)


def test_gemm_is_bit_deterministic():
    from cverl_b200 import ops
    torch.manual_seed(0)
    a = torch.randn(1000, 512, device="cuda").bfloat16()
    b = torch.randn(768, 512, device="cuda").bfloat16()
    assert _same(ops.gemm_nt(a, b), ops.gemm_nt(a, b))
    bt = b.t().contiguous()
    assert _same(ops.gemm_nn(a, bt), ops.gemm_nn(a, bt))


def test_gdn_forward_and_backward_are_bit_deterministic():
    from cverl_b200.ops import gdn_native as gn
    torch.manual_seed(1)
    B, T, H = 2, 256, 2
    mixed = torch.randn(B, T, 3 * H * 128, device="cuda").bfloat16()
    q, k, v = (m.reshape(B, T, H, 128) for m in mixed.split(H * 128, dim=-1))
    beta = torch.sigmoid(torch.randn(B, T, H, device="cuda"))
    g = -0.3 * torch.rand(B, T, H, device="cuda")
    runs = []
    for _ in range(2):
        o, Sf, Vn, SsT, pre = gn.chunk_forward(q, k, v, beta, g, None, 128 ** -0.5, keep_prep=True)
        do = torch.ones_like(o)
        grads = gn.chunk_backward(q, k, v, beta, 128 ** -0.5, pre, Vn, SsT, Sf, do, None)
        runs.append((o, Sf, Vn) + tuple(grads[:5]))   # dq, dk, dv, dbeta, dg (dq^T uses no atomics here)
    for x, y in zip(*runs):
        assert _same(x, y)


def test_attention_forward_is_bit_deterministic():
    from cverl_b200.ops import attention_native as an
    torch.manual_seed(2)
    q = torch.randn(2, 256, 4, 128, device="cuda").bfloat16()
    k = torch.randn(2, 256, 2, 128, device="cuda").bfloat16()
    v = torch.randn(2, 256, 2, 128, device="cuda").bfloat16()
    o1, l1 = an._fwd(q, k, v, 128 ** -0.5, True, 0, 0)
    o2, l2 = an._fwd(q, k, v, 128 ** -0.5, True, 0, 0)
    assert _same(o1, o2) and _same(l1, l2)


def test_norm_conv_kernels_are_bit_deterministic():
    from cverl_b200 import ops
    torch.manual_seed(3)
    x = torch.randn(4, 300, 512, device="cuda").bfloat16()
    w = torch.randn(512, 4, device="cuda").bfloat16()
    with torch.no_grad():
        assert _same(ops.conv1d_silu(x, w), ops.conv1d_silu(x, w))
        h, r = torch.randn(1200, 512, device="cuda").bfloat16(), torch.randn(1200, 512, device="cuda").bfloat16()
        nw = torch.randn(512, device="cuda").bfloat16()
        y1, s1 = ops.add_rmsnorm(h, r, nw, 1e-6, 1.0)
        y2, s2 = ops.add_rmsnorm(h, r, nw, 1e-6, 1.0)
        assert _same(y1, y2) and _same(s1, s2)
