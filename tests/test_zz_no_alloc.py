"""The allocation-free GRPO advantage entry point against the caller-scratch one.

Named to be collected last: it must pass both alone and after every other GPU test has used the
library (and the shared static scratch may hold anything by then)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 16384
ERR_LIMIT = -1001


def _entry():
    from cverl_b200 import _native as nv
    fn = nv.cuda().cvb_grpo_advantage_static       # the exported C symbol itself
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p, C.c_void_p, C.c_longlong,
                   C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return fn


def _case(rows, cols, seed, group):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mask = (torch.rand(rows, cols, device="cuda", generator=g) > 0.2).float()
    rew = torch.zeros(rows, cols, device="cuda")
    rew[:, -1] = (torch.rand(rows, device="cuda", generator=g) > 0.5).float() * 2 - 0.5
    gid = (torch.arange(rows, device="cuda") // group).to(torch.int64)
    return rew.contiguous(), mask.contiguous(), gid


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from cverl_b200 import _native as nv
    from cverl_b200.ops import rl
    fn = _entry()
    # two calls in a row with different shapes: the second must not depend on what the first left behind
    for rows, cols, seed, group, norm in [(1024, 257, 0, 8, 1), (96, 1024, 1, 4, 0)]:
        rew, mask, gid = _case(rows, cols, seed, group)
        adv = torch.full((rows, cols), float("nan"), device="cuda")
        ret = torch.full((rows, cols), float("nan"), device="cuda")
        rc = fn(rew.data_ptr(), mask.data_ptr(), gid.data_ptr(), 1e-6, norm, adv.data_ptr(), ret.data_ptr(), rows,
                cols, nv.stream())
        assert rc == 0
        ref_adv, ref_ret = rl.fused_grpo_advantage(rew, mask, gid, 1e-6, bool(norm))
        torch.cuda.synchronize()
        torch.testing.assert_close(adv, ref_adv, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(ret, ref_ret, rtol=1e-6, atol=1e-6)
        # and against the plain fp32 statement of the op
        t_adv, _ = rl.grpo_outcome_advantage(rew, mask, gid, 1e-6, bool(norm))
        torch.testing.assert_close(adv, t_adv.float(), rtol=1e-4, atol=1e-5)


def test_static_scratch_rejects_oversized_batch():
    from cverl_b200 import _native as nv
    fn = _entry()
    x = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1e-6, 1, x.data_ptr(), None, MAX_ROWS + 1, 1, nv.stream())
    assert rc == ERR_LIMIT                          # refused on the host: nothing was launched
    torch.cuda.synchronize()


def test_static_scratch_at_its_exact_limit():
    """``rows == 16384`` is the largest batch the fixed array holds: accepted, and correct to the last row."""
    from cverl_b200 import _native as nv
    from cverl_b200.ops import rl
    fn = _entry()
    rows, cols = MAX_ROWS, 8
    rew, mask, gid = _case(rows, cols, 5, 8)
    adv = torch.full((rows, cols), float("nan"), device="cuda")
    rc = fn(rew.data_ptr(), mask.data_ptr(), gid.data_ptr(), 1e-6, 1, adv.data_ptr(), None, rows, cols, nv.stream())
    assert rc == 0
    ref_adv, _ = rl.fused_grpo_advantage(rew, mask, gid, 1e-6, True)
    torch.cuda.synchronize()
    torch.testing.assert_close(adv, ref_adv, rtol=1e-6, atol=1e-6)
    assert torch.isfinite(adv[-8:]).all()
