"""Golden files for the RL math: write them, and replay them through the public C ABI.

``python -m cverl_b200.cli.golden dump out.bin [--seed 1234]``
``python -m cverl_b200.cli.golden compare out.bin``

File format ``CVERLGD1`` version 3, little endian, as read by the reference replay tool
(tools/compare_golden.cc:13-24) and written by its generator (tools/golden_dump.py:26-57): magic,
u32 version, u32 record count, then records ``u32 kind`` + payload.

* KL (1):   u32 penalty; f32 tensors logp, ref, out, d out / d logp
* GAE (2):  f32 gamma, lam; tensors rewards, values, mask, advantages, returns
* GRPO (3): f32 eps, u32 norm_by_std; i64 array group ids; tensors rewards, mask, advantages, returns
* PPO (4):  f32 clip, clip_low, clip_high, clip_c, u32 agg; tensors old_log_prob, log_prob, advantages, mask;
            f32 loss, clipfrac, ppo_kl, clipfrac_lower; tensor d loss / d log_prob

A tensor is ``u32 rows, u32 cols, rows*cols f32``; an i64 array is ``u32 n, n i64``.  ``dump`` takes the expected
values from Python verl when it is importable and otherwise from this package's PyTorch statements of the
same formulas (and says which in its output); ``compare`` checks every record through ``libcverl`` with
atol = rtol = 1e-5 and exits non-zero on a mismatch.
"""
from __future__ import annotations

import argparse
import random
import struct
import sys
from pathlib import Path
from typing import BinaryIO, List

import numpy as np
import torch

from ..ops import rl

MAGIC = b"CVERLGD1"
VERSION = 3
KIND_KL, KIND_GAE, KIND_GRPO, KIND_PPO = 1, 2, 3, 4
_KL_NAMES = ["k1", "abs", "k2", "k3"]
ATOL = RTOL = 1e-5


# ----------------------------------------------------------------------------- primitives
def _w_u32(f: BinaryIO, v: int) -> None:
    f.write(struct.pack("<I", v))


def _w_tensor(f: BinaryIO, t: torch.Tensor) -> None:
    a = t.detach().cpu().contiguous().numpy().astype(np.float32, copy=False)
    if a.ndim != 2:
        raise ValueError("golden tensors are 2-D")
    _w_u32(f, a.shape[0])
    _w_u32(f, a.shape[1])
    f.write(a.tobytes(order="C"))


def _w_i64(f: BinaryIO, v) -> None:
    a = np.asarray(v, dtype=np.int64).reshape(-1)
    _w_u32(f, a.size)
    f.write(a.tobytes(order="C"))


def _r_u32(f: BinaryIO) -> int:
    return struct.unpack("<I", f.read(4))[0]


def _r_f32(f: BinaryIO, n: int):
    return struct.unpack("<" + "f" * n, f.read(4 * n))


def _r_tensor(f: BinaryIO) -> torch.Tensor:
    rows, cols = _r_u32(f), _r_u32(f)
    a = np.frombuffer(f.read(4 * rows * cols), dtype="<f4").reshape(rows, cols)
    return torch.from_numpy(a.copy())


def _r_i64(f: BinaryIO) -> torch.Tensor:
    n = _r_u32(f)
    return torch.from_numpy(np.frombuffer(f.read(8 * n), dtype="<i8").copy())


# ----------------------------------------------------------------------------- dump
def _mask(rows: int, cols: int) -> torch.Tensor:
    m = torch.randint(0, 2, (rows, cols)).float()
    for r in range(rows):
        if m[r].sum() < 2:
            m[r, -2:] = 1.0
    return m


def _oracle():
    """(source name, kl, gae, grpo, ppo) callables returning the expected values."""
    try:
        from verl.trainer.ppo import core_algos as va  # type: ignore

        def ppo(old, lp, adv, mask, clip, c, agg):
            class Cfg(dict):
                pass
            cfg = Cfg(clip_ratio_c=c, global_batch_info={})
            cfg.clip_ratio, cfg.clip_ratio_low, cfg.clip_ratio_high, cfg.global_batch_info = clip, None, None, {}
            loss, met = va.compute_policy_loss_vanilla(old_log_prob=old, log_prob=lp, advantages=adv,
                                                       response_mask=mask, loss_agg_mode="token-mean", config=cfg,
                                                       rollout_is_weights=None)
            return loss, float(met["actor/pg_clipfrac"]), float(met["actor/ppo_kl"]), float(met["actor/pg_clipfrac_lower"])
        return ("verl", va.kl_penalty,
                lambda r, v, m, g, l: va.compute_gae_advantage_return(r, v, m, torch.tensor(g), torch.tensor(l)),
                lambda r, m, gid, norm: va.compute_grpo_outcome_advantage(r, m, gid, norm_adv_by_std_in_grpo=norm),
                ppo)
    except Exception:  # verl is not installed: this package's own PyTorch statements
        def ppo(old, lp, adv, mask, clip, c, agg):
            res = rl.ppo_clipped_loss(old, lp, adv, mask, clip, -1.0, -1.0, c, agg)
            return res.pg_loss, res.pg_clipfrac.item(), res.ppo_kl.item(), res.pg_clipfrac_lower.item()
        return ("cverl_b200 torch statements", rl.kl_penalty, rl.gae_advantage_return,
                lambda r, m, gid, norm: rl.grpo_outcome_advantage(r, m, torch.as_tensor(gid), 1e-6, norm), ppo)


def make_records(seed: int):
    source, kl, gae, grpo, ppo = _oracle()
    torch.manual_seed(seed)
    np.random.seed(seed)
    random.seed(seed)
    rows, cols = 8, 16
    recs: List[tuple] = []
    for pen in range(4):
        ref = torch.randn(rows, cols) * 0.5
        lp = (ref + torch.randn(rows, cols) * 0.3).requires_grad_(True)
        out = kl(lp, ref, _KL_NAMES[pen])
        out.sum().backward()
        recs.append((KIND_KL, pen, lp.detach(), ref, out.detach(), lp.grad.clone()))
    rew, val, m = torch.randn(rows, cols), torch.randn(rows, cols), _mask(rows, cols)
    adv, ret = gae(rew, val, m, 0.97, 0.91)
    recs.append((KIND_GAE, 0.97, 0.91, rew, val, m, adv, ret))
    rew, m = torch.randn(rows, cols) * _mask(rows, cols), _mask(rows, cols)
    gid = np.arange(rows, dtype=np.int64) // 2
    random.shuffle(gid)
    for norm in (False, True):
        adv, ret = grpo(rew, m, gid, norm)
        recs.append((KIND_GRPO, gid.copy(), 1.0e-6, int(norm), rew, m, adv, ret))
    old = torch.randn(rows, cols) * 0.5
    lp = (old + torch.randn(rows, cols) * 0.25).requires_grad_(True)
    adv, m = torch.randn(rows, cols), _mask(rows, cols)
    loss, clipfrac, ppo_kl, lower = ppo(old, lp, adv, m, 0.2, 3.0, rl.AGG_TOKEN_MEAN)
    loss.backward()
    recs.append((KIND_PPO, 0.2, -1.0, -1.0, 3.0, rl.AGG_TOKEN_MEAN, old, lp.detach(), adv, m, float(loss), clipfrac,
                 ppo_kl, lower, lp.grad.clone()))
    return source, recs


def write_records(path: Path, recs) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("wb") as f:
        f.write(MAGIC)
        _w_u32(f, VERSION)
        _w_u32(f, len(recs))
        for r in recs:
            _w_u32(f, r[0])
            if r[0] == KIND_KL:
                _w_u32(f, r[1])
                for t in r[2:6]:
                    _w_tensor(f, t)
            elif r[0] == KIND_GAE:
                f.write(struct.pack("<ff", r[1], r[2]))
                for t in r[3:8]:
                    _w_tensor(f, t)
            elif r[0] == KIND_GRPO:
                f.write(struct.pack("<fI", r[2], r[3]))
                _w_i64(f, r[1])
                for t in r[4:8]:
                    _w_tensor(f, t)
            else:
                f.write(struct.pack("<ffffI", *r[1:6]))
                for t in r[6:10]:
                    _w_tensor(f, t)
                f.write(struct.pack("<ffff", *r[10:14]))
                _w_tensor(f, r[14])


# ----------------------------------------------------------------------------- compare
def _close(name: str, got, want, fails: List[str]) -> None:
    got, want = torch.as_tensor(got, dtype=torch.float32), torch.as_tensor(want, dtype=torch.float32)
    if not torch.allclose(got, want, rtol=RTOL, atol=ATOL):
        fails.append(f"{name}: max abs diff {float((got - want).abs().max()):.3e}")


def compare_file(path: Path) -> List[str]:
    """Replays every record through the C ABI; returns the list of mismatches."""
    fails: List[str] = []
    abi = rl.c_abi
    with path.open("rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError("not a CVERLGD1 golden file")
        version, count = _r_u32(f), _r_u32(f)
        if not (1 <= version <= VERSION):
            raise ValueError(f"unsupported golden version {version}")
        for i in range(count):
            kind = _r_u32(f)
            tag = f"record {i}"
            if kind == KIND_KL:
                pen = _KL_NAMES[_r_u32(f)]
                lp, ref, out = _r_tensor(f), _r_tensor(f), _r_tensor(f)
                _close(f"{tag} kl[{pen}]", abi.kl_penalty(lp, ref, pen), out, fails)
                if version >= 2:
                    _close(f"{tag} kl[{pen}] backward", abi.kl_penalty(lp, ref, pen, backward=True), _r_tensor(f), fails)
            elif kind == KIND_GAE:
                gamma, lam = _r_f32(f, 2)
                rew, val, m, adv, ret = (_r_tensor(f) for _ in range(5))
                a, r = abi.gae(rew, val, m, gamma, lam)
                _close(f"{tag} gae advantages", a, adv, fails)
                _close(f"{tag} gae returns", r, ret, fails)
            elif kind == KIND_GRPO:
                eps, = _r_f32(f, 1)
                norm = _r_u32(f)
                gid = _r_i64(f)
                rew, m, adv, ret = (_r_tensor(f) for _ in range(4))
                a, r = abi.grpo(rew, m, gid, eps, bool(norm))
                _close(f"{tag} grpo advantages", a, adv, fails)
                _close(f"{tag} grpo returns", r, ret, fails)
            elif kind == KIND_PPO:
                clip, low, high, c = _r_f32(f, 4)
                agg = _r_u32(f)
                old, lp, adv, m = (_r_tensor(f) for _ in range(4))
                want = _r_f32(f, 4)
                got = abi.ppo_loss(old, lp, adv, m, clip, low, high, c, agg)
                for nme, g, w in zip(("loss", "clipfrac", "ppo_kl", "clipfrac_lower"), got, want):
                    _close(f"{tag} ppo {nme}", g, w, fails)
                if version >= 3:
                    _close(f"{tag} ppo backward", abi.ppo_loss_backward(old, lp, adv, m, clip, low, high, c, agg),
                           _r_tensor(f), fails)
            else:
                raise ValueError(f"unknown record kind {kind}")
    return fails


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("dump")
    d.add_argument("output", type=Path)
    d.add_argument("--seed", type=int, default=1234)
    c = sub.add_parser("compare")
    c.add_argument("input", type=Path)
    a = ap.parse_args(argv)
    if a.cmd == "dump":
        source, recs = make_records(a.seed)
        write_records(a.output, recs)
        print(f"wrote {len(recs)} golden records to {a.output} (expected values from: {source})")
        return 0
    fails = compare_file(a.input)
    for line in fails:
        print("MISMATCH", line)
    print(f"golden replay: {'FAILED' if fails else 'ok'} (atol = rtol = {ATOL})")
    return 1 if fails else 0


if __name__ == "__main__":
    sys.exit(main())
