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


