"""Tiny hybrid model on the native kernels against the same model in fp32 PyTorch ops on CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg():
    from cverl_b200.models.config import Qwen35TextConfig
    return Qwen35TextConfig(vocab_size=2048, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                            num_key_value_heads=2, head_dim=128, intermediate_size=512, linear_key_head_dim=128,
                            linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=2)


def test_forward_backward_matches_cpu_fp32():
    from cverl_b200 import _native as nv
    from cverl_b200.models.qwen3_5 import Qwen35Model
    cfg = _cfg()
    dev = torch.device("cuda", 0)
    gm = Qwen35Model(cfg, dtype=torch.bfloat16, device=dev)
    gm.init_weights(seed=7)
    cm = Qwen35Model(cfg, dtype=torch.float32, device="cpu")
    cm.flat.flat.copy_(gm.flat.flat.float().cpu())
    ids = torch.randint(1, cfg.vocab_size, (2, 96))
    lp_g = gm.response_logprobs(ids.to(dev), 32)
    lp_c = cm.response_logprobs(ids, 32)
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
