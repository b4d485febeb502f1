"""Tiny hybrid model on the native kernels against the same model in fp32 PyTorch ops on CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(head_dim=128):
    from cverl_b200.models.config import Qwen35TextConfig
    return Qwen35TextConfig(vocab_size=2048, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                            num_key_value_heads=2, head_dim=head_dim, intermediate_size=512, linear_key_head_dim=128,
                            linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=2)


@pytest.mark.parametrize("head_dim,seq,prompt", [(128, 96, 32), (128, 256, 64), (256, 256, 64)])
def test_forward_backward_matches_cpu_fp32(head_dim, seq, prompt):
    """``seq = 96`` runs the PyTorch paths of attention and the scan (shapes the kernels do not take); ``seq = 256``
    runs every native kernel, which the fallback counter confirms."""
    from cverl_b200 import _native as nv
    from cverl_b200.models.qwen3_5 import Qwen35Model
    from cverl_b200.utils import fallbacks
    fallbacks.reset()
    cfg = _cfg(head_dim)
    dev = torch.device("cuda", 0)
    gm = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev)
    gm.init_weights(seed=7)
    cm = Qwen35Model(cfg, dtype=torch.float32, device="cpu")
    cm.flat.flat.copy_(gm.flat.flat.float().cpu())
    ids = torch.randint(1, cfg.vocab_size, (2, seq))
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", fallbacks.NativeKernelFallback)
        lp_g = gm.response_logprobs(ids.to(dev), prompt)
    assert (fallbacks.total() == 0) == (seq % 128 == 0)
    lp_c = cm.response_logprobs(ids, prompt)
    assert (lp_g.cpu() - lp_c).abs().max().item() < 0.15
    assert (lp_g.cpu() - lp_c).abs().mean().item() < 0.03
    w = torch.randn_like(lp_c)
    lp_g.backward(w.to(dev))
    lp_c.backward(w)
    for p in list(cm.flat.params.values()) + list(cm.fused.values()):
        if p.grad is not None:
            p.main_grad.add_(p.grad)
    nv.check_status(dev)
    g, c = gm.flat.main_grad.cpu(), cm.flat.main_grad
    rel = ((g - c).norm() / c.norm()).item()
    assert rel < 0.06, rel


def test_smoke_entry():
    import __graft_entry__ as ge
    ge.smoke()
