"""Gated DeltaNet (gated delta rule) linear attention.

State recurrence per head (fp32), as in the reference's eager loop
(src/model/qwen3_5_text.cc:247-258):

    S *= exp(g_t);  kv = S^T k_t;  delta = (v_t - kv) * beta_t;
    S += k_t (x) delta;  o_t = S^T q_t

``gdn_recurrent_ref`` is that loop (the oracle).  ``gdn_chunked`` is the
chunk-parallel WY/UT form that the reference lacks: inside a chunk of C tokens
with cumulative log-decay ``c_t`` the pseudo-values solve the unit-lower-
triangular system ``(I + A) U = beta*(V - exp(c) K S0)`` with
``A[t,s] = beta_t exp(c_t - c_s) <k_t,k_s>`` (s < t), so a chunk costs a few
GEMMs and the sequential dependency is only chunk-to-chunk on the
``[dk, dv]`` state.  Both accept an initial state and return the final state,
which context parallelism carries from rank to rank.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_recurrent_ref(q, k, v, beta, g, initial_state=None):
    """q,k [B,H,T,dk], v [B,H,T,dv], beta,g [B,H,T] (fp32) -> (o [B,H,T,dv], S [B,H,dk,dv])."""
    B, H, T, dk = q.shape
    dv = v.shape[-1]
    S = initial_state.float().clone() if initial_state is not None else q.new_zeros(B, H, dk, dv, dtype=torch.float32)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, :, t]).unsqueeze(-1).unsqueeze(-1)
        kt = k[:, :, t].float()
        kv = (S * kt.unsqueeze(-1)).sum(-2)
        delta = (v[:, :, t].float() - kv) * beta[:, :, t].unsqueeze(-1)
        S = S + kt.unsqueeze(-1) * delta.unsqueeze(-2)
        outs.append((S * q[:, :, t].float().unsqueeze(-1)).sum(-2))
    o = torch.stack(outs, 2) if outs else q.new_zeros(B, H, 0, dv, dtype=torch.float32)
    return o, S


def gdn_chunked(q, k, v, beta, g, initial_state=None, chunk: int = 64):
    """Chunk-parallel evaluation of the same recurrence (differentiable, fp32)."""
    B, H, T, dk = q.shape
    dv = v.shape[-1]
    q, k, v, beta, g = q.float(), k.float(), v.float(), beta.float(), g.float()
    pad = (-T) % chunk
    if pad:
        q = F.pad(q, (0, 0, 0, pad))
        k = F.pad(k, (0, 0, 0, pad))
        v = F.pad(v, (0, 0, 0, pad))
        beta = F.pad(beta, (0, pad))
        g = F.pad(g, (0, pad))  # g = 0 and beta = 0 on padding: the state passes through unchanged
    Tp = T + pad
    n = Tp // chunk
    q, k, v = (x.reshape(B, H, n, chunk, -1) for x in (q, k, v))
    beta = beta.reshape(B, H, n, chunk)
    c = g.reshape(B, H, n, chunk).cumsum(-1)                       # cumulative log decay inside the chunk
    tri_strict = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril(-1)
    tri_incl = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril(0)
    # exp(c_t - c_s) for s <= t; the upper triangle (positive exponents that can overflow) is never used
    decay = torch.exp((c.unsqueeze(-1) - c.unsqueeze(-2)).masked_fill(~tri_incl, 0.0))
    kk = k @ k.transpose(-1, -2)
    A = (beta.unsqueeze(-1) * kk * decay).masked_fill(~tri_strict, 0.0)
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)   # (I + A)^-1
    Up = Tm @ (beta.unsqueeze(-1) * v)                              # T (beta V)
    W = Tm @ (beta.unsqueeze(-1) * torch.exp(c).unsqueeze(-1) * k)  # T (beta exp(c) K)
    qk = (q @ k.transpose(-1, -2) * decay).masked_fill(~tri_incl, 0.0)
    q_dec = q * torch.exp(c).unsqueeze(-1)
    c_last = c[..., -1]
    k_tail = k * torch.exp(c_last.unsqueeze(-1) - c).unsqueeze(-1)  # K exp(c_C - c_s)
    S = initial_state.float() if initial_state is not None else q.new_zeros(B, H, dk, dv)
    outs = []
    for i in range(n):
        v_new = Up[:, :, i] - W[:, :, i] @ S
        outs.append(q_dec[:, :, i] @ S + qk[:, :, i] @ v_new)
        S = S * torch.exp(c_last[:, :, i]).unsqueeze(-1).unsqueeze(-1) + k_tail[:, :, i].transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(B, H, Tp, dv)[:, :, :T]
    return o, S


def gated_delta_rule(q, k, v, beta, g, initial_state=None, *, chunk: int = 64, backend: str = "auto"):
    """Public entry: l2-normalised q (already scaled) and k are expected by the caller.

    ``backend``: ``recurrent`` (oracle loop), ``chunked`` (PyTorch chunk form) or
    ``auto`` (hand-written kernel when present, else ``chunked``).
    """
    if backend == "recurrent":
        return gdn_recurrent_ref(q, k, v, beta, g, initial_state)
    if backend == "auto" and q.is_cuda:
        from . import gdn_native
        if gdn_native.supported(q, v):
            return gdn_native.gated_delta_rule(q, k, v, beta, g, initial_state)
    return gdn_chunked(q, k, v, beta, g, initial_state, chunk)
