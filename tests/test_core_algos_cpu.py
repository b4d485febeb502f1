"""Public C ABI (libcverl.so) against the PyTorch statements of the same math and
against hand-computed values, plus the invalid-argument matrix."""
import ctypes as C
import math

import pytest
import torch

from cverl_b200.ops import rl
from cverl_b200.ops.rl import _T2, c_abi


def _data(rows=6, cols=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    lp = -2 + 0.5 * torch.randn(rows, cols, generator=g)
    old = lp + 0.3 * torch.randn(rows, cols, generator=g)
    ref = lp + 0.1 * torch.randn(rows, cols, generator=g)
    adv = torch.randn(rows, cols, generator=g)
    lens = torch.randint(1, cols + 1, (rows,), generator=g)
    mask = (torch.arange(cols)[None, :] < lens[:, None]).float()
    return lp, old, ref, adv, mask


def test_masked_ops_match_torch():
    lp, _, _, _, mask = _data()
    assert abs(c_abi.masked_sum(lp, mask) - rl.masked_sum(lp, mask).item()) < 1e-4
    assert abs(c_abi.masked_mean(lp, mask) - rl.masked_mean(lp, mask).item()) < 1e-6
    for shift in (True, False):
        torch.testing.assert_close(c_abi.masked_whiten(lp, mask, shift), rl.masked_whiten(lp, mask, shift),
                                   rtol=1e-5, atol=1e-5)


def test_masked_mean_hand_value():
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    m = torch.tensor([[1.0, 0.0, 1.0, 0.0]])
    assert c_abi.masked_sum(v, m) == pytest.approx(4.0)
    assert c_abi.masked_mean(v, m) == pytest.approx(2.0, abs=1e-6)
    # unbiased variance of {1,3} = 2 -> whitened = (+-1)/sqrt(2)
    w = c_abi.masked_whiten(v, m)
    assert w[0, 0].item() == pytest.approx(-1 / math.sqrt(2), abs=1e-5)
    assert w[0, 2].item() == pytest.approx(1 / math.sqrt(2), abs=1e-5)


@pytest.mark.parametrize("kind", ["k1", "abs", "k2", "k3"])
def test_kl_forward_backward(kind):
    lp, _, ref, _, _ = _data()
    torch.testing.assert_close(c_abi.kl_penalty(lp, ref, kind), rl.kl_penalty(lp, ref, kind), rtol=1e-5, atol=1e-6)
    x = lp.clone().requires_grad_(True)
    rl.kl_penalty(x, ref, kind).sum().backward()
    torch.testing.assert_close(c_abi.kl_penalty(lp, ref, kind, backward=True), x.grad, rtol=1e-5, atol=1e-6)


def test_kl_k3_clamps():
    lp = torch.tensor([[0.0, -30.0, 30.0]])
    ref = torch.tensor([[0.0, 0.0, 0.0]])
    out = c_abi.kl_penalty(lp, ref, "k3")
    assert out[0, 0].item() == 0.0
    assert out[0, 1].item() == pytest.approx(10.0)  # exp(20)-20-1 clamped to 10
    assert out[0, 2].item() == pytest.approx(math.exp(-20) + 20 - 1, rel=1e-5) or out[0, 2].item() == 10.0


def test_gae_matches_torch():
    g = torch.Generator().manual_seed(3)
    rew = torch.randn(5, 12, generator=g)
    val = torch.randn(5, 12, generator=g)
    mask = (torch.arange(12)[None, :] < torch.tensor([12, 7, 3, 9, 1])[:, None]).float()
    adv, ret = c_abi.gae(rew, val, mask, 1.0, 0.95)
    adv_t, ret_t = rl.gae_advantage_return(rew, val, mask, 1.0, 0.95)
    torch.testing.assert_close(adv, adv_t, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ret, ret_t, rtol=1e-5, atol=1e-5)


def test_grpo_groups_and_singletons():
    rew = torch.zeros(5, 4)
    rew[:, -1] = torch.tensor([1.0, 0.0, 1.0, 1.0, 5.0])
    mask = torch.ones(5, 4)
    gid = torch.tensor([7, 7, 9, 9, 11])  # last group has one member
    adv, ret = c_abi.grpo(rew, mask, gid, 1e-6, True)
    adv_t, _ = rl.grpo_outcome_advantage(rew, mask, gid, 1e-6, True)
    torch.testing.assert_close(adv, adv_t, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ret, adv)
    # group 7: scores {1,0}: mean .5, unbiased std sqrt(.5)
    assert adv[0, 0].item() == pytest.approx(0.5 / (math.sqrt(0.5) + 1e-6), rel=1e-5)
    # group 9: identical scores -> 0
    assert adv[2, 0].item() == pytest.approx(0.0, abs=1e-6)
    # singleton: mean 0, std 1 -> raw score
    assert adv[4, 0].item() == pytest.approx(5.0 / (1 + 1e-6), rel=1e-5)
    adv_ns, _ = c_abi.grpo(rew, mask, gid, 1e-6, False)
    assert adv_ns[0, 0].item() == pytest.approx(0.5)


@pytest.mark.parametrize("agg", [0, 1, 2])
def test_ppo_loss_and_backward(agg):
    lp, old, _, adv, mask = _data(rows=8, cols=20, seed=agg)
    mask[3] = 0  # an empty row exercises the sequence-mean modes
    got = c_abi.ppo_loss(old, lp, adv, mask, 0.2, -1.0, -1.0, 3.0, agg)
    x = lp.clone().requires_grad_(True)
    res = rl.ppo_clipped_loss(old, x, adv, mask, 0.2, -1.0, -1.0, 3.0, agg)
    want = (res.pg_loss.item(), res.pg_clipfrac.item(), res.ppo_kl.item(), res.pg_clipfrac_lower.item())
    for a, b in zip(got, want):
        assert a == pytest.approx(b, rel=1e-5, abs=1e-6)
    res.pg_loss.backward()
    torch.testing.assert_close(c_abi.ppo_loss_backward(old, lp, adv, mask, 0.2, -1.0, -1.0, 3.0, agg), x.grad,
                               rtol=1e-5, atol=1e-6)


def test_ppo_ratio_one_gradient():
    # old == new: ratio 1, loss = -A, gradient = -A * weight
    lp = torch.full((2, 3), -1.0)
    adv = torch.tensor([[1.0, -2.0, 0.5], [0.0, 1.0, 1.0]])
    mask = torch.ones(2, 3)
    g = c_abi.ppo_loss_backward(lp.clone(), lp, adv, mask)
    torch.testing.assert_close(g, -adv / 6.0, rtol=1e-5, atol=1e-6)
    loss = c_abi.ppo_loss(lp.clone(), lp, adv, mask)[0]
    assert loss == pytest.approx(-adv.mean().item(), abs=1e-6)


def test_invalid_arguments():
    lib = c_abi.lib
    v = torch.zeros(2, 3)
    ok = _T2(v.data_ptr(), 0, 0, 2, 3)
    out = C.c_float()
    assert lib.cverl_masked_sum_f32_cpu(ok, ok, C.byref(out)) == 0
    assert lib.cverl_masked_sum_f32_cpu(ok, ok, None) == 1                      # null out
    assert lib.cverl_masked_sum_f32_cpu(_T2(None, 0, 0, 2, 3), ok, C.byref(out)) == 1   # null data
    assert lib.cverl_masked_sum_f32_cpu(_T2(v.data_ptr(), 1, 0, 2, 3), ok, C.byref(out)) == 1  # dtype
    assert lib.cverl_masked_sum_f32_cpu(_T2(v.data_ptr(), 0, 1, 2, 3), ok, C.byref(out)) == 1  # device
    assert lib.cverl_masked_sum_f32_cpu(_T2(v.data_ptr(), 0, 0, 3, 2), ok, C.byref(out)) == 1  # shape
    assert lib.cverl_masked_sum_f32_cpu(_T2(v.data_ptr(), 0, 0, -1, 3), ok, C.byref(out)) == 1
    res = rl._PpoOut()
    assert lib.cverl_ppo_clipped_loss_f32_cpu(ok, ok, ok, ok, 0.2, -1.0, -1.0, 1.0, 0, C.byref(res)) == 1  # c <= 1
    assert lib.cverl_ppo_clipped_loss_f32_cpu(ok, ok, ok, ok, 0.2, -1.0, -1.0, 3.0, 0, C.byref(res)) == 0
    assert lib.cverl_status_string(0) == b"ok"
    assert lib.cverl_status_string(1) == b"invalid argument"


def test_actor_loss_cpu_path_matches_c_abi():
    lp, old, ref, adv, mask = _data(seed=5)
    metrics, grad = rl.actor_loss(old, lp, adv, mask, None)
    assert metrics[0].item() == pytest.approx(c_abi.ppo_loss(old, lp, adv, mask)[0], rel=1e-5, abs=1e-6)
    torch.testing.assert_close(grad, c_abi.ppo_loss_backward(old, lp, adv, mask), rtol=1e-5, atol=1e-6)


def test_cpu_loss_step_bench_and_cross_check_with_another_abi_library(capsys):
    """The CPU loss-step benchmark runs on the built library; when an ABI-compatible second library is present
    (the out-of-tree build of the reference writes one) the two must agree on every output of the step."""
    import json
    from pathlib import Path
    from cverl_b200 import bench_cpu_loss
    other = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "lib" / "libcverl_ref.so"
    args = ["--iters", "3", "--batch", "16", "--seq", "64"]
    if other.exists():
        args += ["--other", str(other)]
    assert bench_cpu_loss.main(args) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["ours_us_per_step"] > 0
    if other.exists():
        assert rep["max_abs_diff"] < 1e-5, rep["max_abs_diff_by_output"]
