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


# ----------------------------------------------------------------------------
# Chunked form with a hand-derived backward.  The chunk-local algebra is batched
# over every chunk at once; only the two state scans walk the chunks in order,
# and on CUDA those run as tcgen05 kernels with the state held in TMEM
# (cuda/gdn_scan.cu).  Layout inside: [B, H, n_chunks, C, d].
# ----------------------------------------------------------------------------
def _chunk_local(q, k, v, beta, g, scale: float, eps: float = 1e-6):
    """Chunk-local quantities.  q,k [B,H,n,C,dk], v [B,H,n,C,dv], beta,g [B,H,n,C] (fp32)."""
    C = q.shape[-2]
    rq = torch.rsqrt((q * q).sum(-1, keepdim=True) + eps)
    rk = torch.rsqrt((k * k).sum(-1, keepdim=True) + eps)
    qn = q * rq * scale
    kn = k * rk
    c = g.cumsum(-1)
    tri_incl = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(0)
    tri_strict = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(-1)
    decay = torch.exp((c.unsqueeze(-1) - c.unsqueeze(-2)).masked_fill(~tri_incl, 0.0))
    G = kn @ kn.transpose(-1, -2)
    A = (beta.unsqueeze(-1) * decay * G).masked_fill(~tri_strict, 0.0)
    eye = torch.eye(C, device=q.device, dtype=q.dtype)
    T = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
    ec = torch.exp(c).unsqueeze(-1)
    Kb = beta.unsqueeze(-1) * ec * kn
    Vb = beta.unsqueeze(-1) * v
    W = T @ Kb
    U = T @ Vb
    P = ((qn @ kn.transpose(-1, -2)) * decay).masked_fill(~tri_incl, 0.0)
    gam = c[..., -1]
    Kdec = torch.exp(gam.unsqueeze(-1) - c).unsqueeze(-1) * kn
    Qd = ec * qn
    return dict(rq=rq, rk=rk, qn=qn, kn=kn, c=c, decay=decay, G=G, A=A, T=T, Kb=Kb, Vb=Vb, W=W, U=U, P=P,
                egam=torch.exp(gam), Kdec=Kdec, Qd=Qd, tri_incl=tri_incl, tri_strict=tri_strict)


def scan_fwd_ref(W, U, Kdec, egam, S0):
    """Vn_i = U_i - W_i S_i ; S_{i+1} = egam_i S_i + Kdec_i^T Vn_i.  Returns (Vn, S_chunks, S_final)."""
    n = W.shape[2]
    S = S0
    Vn, Ss = [], []
    for i in range(n):
        Ss.append(S)
        vn = U[:, :, i] - W[:, :, i] @ S
        Vn.append(vn)
        S = S * egam[:, :, i, None, None] + Kdec[:, :, i].transpose(-1, -2) @ vn
    return torch.stack(Vn, 2), torch.stack(Ss, 2), S


def scan_bwd_ref(dVloc, Kdec, Qd, W, dO, egam, dSf):
    """dVn_i = dVloc_i + Kdec_i dS ; dS <- egam_i dS + Qd_i^T dO_i - W_i^T dVn_i (i descending).
    Returns (dVn, dS_next per chunk, dS0)."""
    n = W.shape[2]
    dS = dSf
    dVn, dSn = [None] * n, [None] * n
    for i in range(n - 1, -1, -1):
        dSn[i] = dS
        dv = dVloc[:, :, i] + Kdec[:, :, i] @ dS
        dVn[i] = dv
        dS = dS * egam[:, :, i, None, None] + Qd[:, :, i].transpose(-1, -2) @ dO[:, :, i] \
            - W[:, :, i].transpose(-1, -2) @ dv
    return torch.stack(dVn, 2), torch.stack(dSn, 2), dS


def _scan_fwd(W, U, Kdec, egam, S0):
    if W.is_cuda:
        from . import gdn_native
        if gdn_native.scan_supported(W, U):
            return gdn_native.scan_fwd(W, U, Kdec, egam, S0)
    return scan_fwd_ref(W, U, Kdec, egam, S0)


def _scan_bwd(P, Kdec, Qd, W, dO, egam, dSf):
    if W.is_cuda:
        from . import gdn_native
        if gdn_native.scan_supported(W, dO):
            return gdn_native.scan_bwd(P, Kdec, Qd, W, dO, egam, dSf)
    return scan_bwd_ref(P.transpose(-1, -2) @ dO, Kdec, Qd, W, dO, egam, dSf)


class _tf32_matmul:
    """Chunk-local products are [64 x 64 x 128]-sized batched GEMMs on operands that were bf16 a
    moment ago; on CUDA they run on the tensor cores in TF32 instead of the SIMT fp32 path."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev
        return False


class _GdnChunked(torch.autograd.Function):
    """q,k [B,T,H,dk] (raw, un-normalised), v [B,T,H,dv], beta,g [B,T,H] fp32, S0 [B,H,dk,dv] or None.
    Returns (o [B,T,H,dv] in v's dtype, S_final fp32)."""

    @staticmethod
    def forward(ctx, q, k, v, beta, g, S0, scale, chunk):
        with _tf32_matmul():
            return _GdnChunked._forward(ctx, q, k, v, beta, g, S0, scale, chunk)

    @staticmethod
    def backward(ctx, do, dSf):
        with _tf32_matmul():
            return _GdnChunked._backward(ctx, do, dSf)

    @staticmethod
    def _forward(ctx, q, k, v, beta, g, S0, scale, chunk):
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        if q.is_cuda and chunk == 64:
            from . import gdn_native
            if gdn_native.chunk_supported(q, k, v):
                keep = gdn_native.chunk_bwd_enabled() and any(ctx.needs_input_grad[:6])
                o, Sf, Vn, SsT, pre = gdn_native.chunk_forward(q, k, v, beta, g, S0, scale, keep_prep=keep)
                ctx.cfg = (scale, chunk, 0, T // chunk, S0 is not None)
                ctx.native = True
                ctx.keep = keep
                ctx.states_kept = True
                if keep:   # the backward kernels reuse the chunk-local operands instead of recomputing them
                    ctx.states_kept = gdn_native.keep_states(B, H, T // chunk)
                    if ctx.states_kept:
                        a, b = Vn, SsT.transpose(-1, -2)
                    else:  # regenerated in the backward pass from U and the initial state
                        a, b = pre["U"], (S0 if S0 is not None else q.new_empty(0))
                    ctx.save_for_backward(q, k, v, beta, g, a, b, Sf, pre["W"], pre["Kd"],
                                          pre["Qd"], pre["P"], pre["egam"], pre["Tm"], pre["aux"])
                else:
                    ctx.save_for_backward(q, k, v, beta, g, Vn, SsT.transpose(-1, -2), Sf)
                return o, Sf
        if q.is_cuda:
            from ..utils import fallbacks
            fallbacks.note("gated_delta_rule", f"dtype {q.dtype}, shape {tuple(q.shape)}, chunk {chunk}: the chunk "
                                               f"kernels take bf16 [B, T, H, 128] with T % 64 == 0 read in place")
        ctx.native = False
        pad = (-T) % chunk
        n = (T + pad) // chunk

        def blk(x, last):
            x = x.float().transpose(1, 2)  # [B,H,T,*]
            if pad:
                x = F.pad(x, (0, 0, 0, pad)) if last else F.pad(x, (0, pad))
            return x.reshape(B, H, n, chunk, -1) if last else x.reshape(B, H, n, chunk)

        qb, kb, vb = blk(q, True), blk(k, True), blk(v, True)
        bb, gb = blk(beta, False), blk(g, False)
        loc = _chunk_local(qb, kb, vb, bb, gb, scale)
        S0f = S0.float() if S0 is not None else qb.new_zeros(B, H, dk, dv)
        Vn, Ss, Sf = _scan_fwd(loc["W"], loc["U"], loc["Kdec"], loc["egam"], S0f)
        O = loc["Qd"] @ Ss.float() + loc["P"] @ Vn.float()
        o = O.reshape(B, H, n * chunk, dv)[:, :, :T].transpose(1, 2).to(v.dtype)
        ctx.save_for_backward(q, k, v, beta, g, Vn, Ss)
        ctx.cfg = (scale, chunk, pad, n, S0 is not None)
        return o, Sf

    @staticmethod
    def _backward(ctx, do, dSf):
        scale, chunk, pad, n, has_s0 = ctx.cfg
        if ctx.native and ctx.keep:
            q, k, v, beta, g, Vn, Ss, Sf, W_, Kd_, Qd_, P_, eg_, Tm_, aux_ = ctx.saved_tensors
            from . import gdn_native
            pre = dict(W=W_, Kd=Kd_, Qd=Qd_, P=P_, egam=eg_, Tm=Tm_, aux=aux_)
            if ctx.states_kept:
                SsT = Ss.transpose(-1, -2)
            else:
                Vn, SsT = gdn_native.regenerate_states(W_, Vn, Kd_, eg_, Ss if has_s0 else None)
            dq, dk, dv, dbeta, dg, dS0 = gdn_native.chunk_backward(q, k, v, beta, scale, pre, Vn, SsT, Sf, do, dSf)
            return (dq, dk, dv, dbeta.to(beta.dtype), dg.to(g.dtype), (dS0 if has_s0 else None), None, None)
        if ctx.native:
            q, k, v, beta, g, Vn, Ss, Sf = ctx.saved_tensors
        else:
            q, k, v, beta, g, Vn, Ss = ctx.saved_tensors
        B, T, H, dk = q.shape
        dv = v.shape[-1]

        def blk(x, last):
            x = x.float().transpose(1, 2)
            if pad:
                x = F.pad(x, (0, 0, 0, pad)) if last else F.pad(x, (0, pad))
            return x.reshape(B, H, n, chunk, -1) if last else x.reshape(B, H, n, chunk)

        qb, kb, vb = blk(q, True), blk(k, True), blk(v, True)
        bb, gb = blk(beta, False), blk(g, False)
        L = _chunk_local(qb, kb, vb, bb, gb, scale)
        dO = blk(do, True)
        dSf = dSf.float() if dSf is not None else Ss.new_zeros(B, H, dk, dv)
        Vn, Ss = Vn.float(), Ss.float()
        kn, qn, c, decay, Tm = L["kn"], L["qn"], L["c"], L["decay"], L["T"]
        dVn, dSn, dS0 = _scan_bwd(L["P"], L["Kdec"], L["Qd"], L["W"], dO, L["egam"], dSf)
        dVn, dSn = dVn.float(), dSn.float()
        # ---- chunk-local gradients -------------------------------------------------
        dW = -(dVn @ Ss.transpose(-1, -2))
        dU = dVn
        dP = (dO @ Vn.transpose(-1, -2)).masked_fill(~L["tri_incl"], 0.0)
        dQd = dO @ Ss.transpose(-1, -2)
        ec = torch.exp(c).unsqueeze(-1)
        dPd = dP * decay
        dqn = ec * dQd + dPd @ kn
        dkn = dPd.transpose(-1, -2) @ qn
        dKdec = Vn @ dSn.transpose(-1, -2)
        edec = torch.exp(c[..., -1:].clone() - c).unsqueeze(-1)
        dkn = dkn + edec * dKdec
        dc = (dQd * L["Qd"]).sum(-1)
        MP = dP * L["P"]
        dc = dc + MP.sum(-1) - MP.sum(-2)
        s_t = (dKdec * L["Kdec"]).sum(-1)
        dc = dc - s_t
        dgam = s_t.sum(-1) + L["egam"] * (Ss * dSn).sum((-1, -2))
        dT = dW @ L["Kb"].transpose(-1, -2) + dU @ L["Vb"].transpose(-1, -2)
        dKb = Tm.transpose(-1, -2) @ dW
        dVb = Tm.transpose(-1, -2) @ dU
        dvb = bb.unsqueeze(-1) * dVb
        dbeta = (dVb * vb).sum(-1) + (dKb * ec * kn).sum(-1)
        dkn = dkn + bb.unsqueeze(-1) * ec * dKb
        dc = dc + (dKb * L["Kb"]).sum(-1)
        dA = -(Tm.transpose(-1, -2) @ dT @ Tm.transpose(-1, -2)).masked_fill(~L["tri_strict"], 0.0)
        MA = dA * L["A"]
        dbeta = dbeta + (dA * decay * L["G"]).sum(-1)
        dc = dc + MA.sum(-1) - MA.sum(-2)
        dG = dA * bb.unsqueeze(-1) * decay
        dkn = dkn + dG @ kn + dG.transpose(-1, -2) @ kn
        dc[..., -1] = dc[..., -1] + dgam
        dg = dc.flip(-1).cumsum(-1).flip(-1)
        # ---- l2norm backward -------------------------------------------------------
        khat = kn
        dk_raw = L["rk"] * (dkn - khat * (dkn * khat).sum(-1, keepdim=True))
        qhat = qn / scale
        dqh = dqn * scale
        dq_raw = L["rq"] * (dqh - qhat * (dqh * qhat).sum(-1, keepdim=True))

        def unblk(x, last, like):
            x = x.reshape(B, H, n * chunk, -1)[:, :, :T] if last else x.reshape(B, H, n * chunk)[:, :, :T]
            return x.transpose(1, 2).to(like.dtype)

        return (unblk(dq_raw, True, q), unblk(dk_raw, True, k), unblk(dvb, True, v), unblk(dbeta, False, beta),
                unblk(dg, False, g), (dS0 if has_s0 else None), None, None)


def gdn_gates_ref(b, a, A_log, dt_bias):
    """beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias), both fp32."""
    beta = torch.sigmoid(b.float())
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())
    return beta, g


class _GdnGates(torch.autograd.Function):
    """``gdn_gates_ref`` as one kernel each way on bf16 column groups ``b``, ``a`` [..., H] of the fused
    projection (read in place).  If they carry ``_grad_sink`` (set by ``conv1d_silu_split``) their gradients
    are written straight into the projection-gradient buffer."""

    @staticmethod
    def forward(ctx, b, a, A_log, dt_bias, sink_b, sink_a):
        from .. import _native as nv
        from .gemm import count_launch
        H = b.shape[-1]
        rows = b.numel() // H
        beta = torch.empty(b.shape, dtype=torch.float32, device=b.device)
        g = torch.empty(b.shape, dtype=torch.float32, device=b.device)
        nv.check(nv.cuda().cvb_gdn_gates_fwd(b.data_ptr(), a.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(),
                                             beta.data_ptr(), g.data_ptr(), rows, H, b.stride(-2), nv.stream()),
                 "cvb_gdn_gates_fwd")
        count_launch()
        ctx.save_for_backward(b, a, A_log, dt_bias)
        ctx.sinks = (sink_b, sink_a)
        return beta, g

    @staticmethod
    def backward(ctx, dbeta, dg):
        from .. import _native as nv
        from .gemm import count_launch
        from .norm import _wgrad_buffer
        b, a, A_log, dt_bias = ctx.saved_tensors
        H = b.shape[-1]
        rows = b.numel() // H
        dbeta = dbeta.float().contiguous()
        dg = dg.float().contiguous()
        db = da = None
        sb, sa = ctx.sinks
        if sb is not None and sa is not None and sb[0] is sa[0]:
            db, da = sb[0].view_for(sb[1], b.shape), sa[0].view_for(sa[1], a.shape)
        if db is None or da is None or db.stride(-2) != da.stride(-2):
            db = torch.empty(b.shape, dtype=b.dtype, device=b.device)
            da = torch.empty(a.shape, dtype=a.dtype, device=a.device)
        gA, mainA = _wgrad_buffer(A_log)
        gB, mainB = _wgrad_buffer(dt_bias)
        nv.check(nv.cuda().cvb_gdn_gates_bwd(dbeta.data_ptr(), dg.data_ptr(), b.data_ptr(), a.data_ptr(),
                                             A_log.data_ptr(), dt_bias.data_ptr(), db.data_ptr(), da.data_ptr(),
                                             gA.data_ptr(), gB.data_ptr(), rows, H, b.stride(-2), db.stride(-2),
                                             nv.stream()), "cvb_gdn_gates_bwd")
        count_launch()
        return (db, da, None if mainA else gA.to(A_log.dtype), None if mainB else gB.to(dt_bias.dtype), None, None)


def gdn_gates(b, a, A_log, dt_bias):
    """(beta, g) of the Gated-DeltaNet block, fp32, shaped like ``b``.  bf16 CUDA column groups with a common
    row stride run the fused kernels; anything else runs the torch statement."""
    H = b.shape[-1]

    def rows_view_ok(t):
        if t.dim() < 2 or t.stride(-1) != 1:
            return False
        s = t.stride(-2)
        for d in range(t.dim() - 2):        # leading dims must fold into the row index
            if t.stride(d) != t.stride(d + 1) * t.shape[d + 1]:
                return False
        return s >= H

    if (b.is_cuda and b.dtype == torch.bfloat16 and a.dtype == torch.bfloat16 and a.shape == b.shape
            and A_log.dtype == torch.bfloat16 and dt_bias.dtype == torch.bfloat16 and A_log.is_contiguous()
            and dt_bias.is_contiguous() and 0 < H <= 256 and (H & (H - 1)) == 0 and rows_view_ok(b) and rows_view_ok(a)
            and a.stride(-2) == b.stride(-2)):
        return _GdnGates.apply(b, a, A_log, dt_bias, getattr(b, "_grad_sink", None), getattr(a, "_grad_sink", None))
    return gdn_gates_ref(b, a, A_log, dt_bias)


class _GdnPacked(torch.autograd.Function):
    """The native chunk kernels on a packed activation ``[B,T,3*H*128]`` (column ranges q | k | v, as the
    convolution writes them).  The backward kernel stores dq, dk, dv straight into the column ranges of one
    gradient buffer, so no concatenation runs between it and the convolution's backward."""

    @staticmethod
    def _views(t, H):
        B, T, _ = t.shape
        return tuple(t[..., j * H * 128:(j + 1) * H * 128].view(B, T, H, 128) for j in range(3))

    @staticmethod
    def forward(ctx, mixed, beta, g, S0, scale, H):
        from . import gdn_native
        q, k, v = _GdnPacked._views(mixed, H)
        o, Sf, Vn, SsT, pre = gdn_native.chunk_forward(q, k, v, beta, g, S0, scale, keep_prep=True)
        B, T = mixed.shape[:2]
        kept = gdn_native.keep_states(B, H, T // 64)
        ctx.cfg = (scale, H, S0 is not None, kept)
        if kept:
            a, b = Vn, SsT
        else:   # the backward pass regenerates V' and the states from U and the initial state
            a, b = pre["U"], (S0 if S0 is not None else mixed.new_empty(0))
        ctx.save_for_backward(mixed, beta, g, a, b, Sf, pre["W"], pre["Kd"], pre["Qd"], pre["P"], pre["egam"],
                              pre["Tm"], pre["aux"])
        return o, Sf

    @staticmethod
    def backward(ctx, do, dSf):
        from . import gdn_native
        scale, H, has_s0, kept = ctx.cfg
        mixed, beta, g, Vn, SsT, Sf, W_, Kd_, Qd_, P_, eg_, Tm_, aux_ = ctx.saved_tensors
        if not kept:
            Vn, SsT = gdn_native.regenerate_states(W_, Vn, Kd_, eg_, SsT if has_s0 else None)
        q, k, v = _GdnPacked._views(mixed, H)
        d_mixed = torch.empty(mixed.shape, dtype=mixed.dtype, device=mixed.device)
        pre = dict(W=W_, Kd=Kd_, Qd=Qd_, P=P_, egam=eg_, Tm=Tm_, aux=aux_)
        _, _, _, dbeta, dg, dS0 = gdn_native.chunk_backward(q, k, v, beta, scale, pre, Vn, SsT, Sf, do, dSf,
                                                            out=_GdnPacked._views(d_mixed, H))
        return d_mixed, dbeta.to(beta.dtype), dg.to(g.dtype), (dS0 if has_s0 else None), None, None


def gated_delta_rule_packed(mixed, beta, g, initial_state=None, *, scale: float, heads: int):
    """``gated_delta_rule_fused`` on the packed ``[B,T,3*heads*d]`` tensor whose column ranges are q | k | v
    (equal numbers of key and value heads).  With the native chunk kernels the gradient of ``mixed`` is
    written in place by the backward kernel; otherwise this splits and calls the general entry."""
    B, T, Cm = mixed.shape
    d = Cm // (3 * heads)
    q, k, v = (part.reshape(B, T, heads, d) for part in mixed.split(heads * d, dim=-1))
    if mixed.is_cuda and d == 128 and Cm == 3 * heads * 128:
        from . import gdn_native
        if gdn_native.chunk_supported(q, k, v) and gdn_native.chunk_bwd_enabled():
            return _GdnPacked.apply(mixed, beta, g, initial_state, scale, heads)
    return gated_delta_rule_fused(q, k, v, beta, g, initial_state, scale=scale)


def gated_delta_rule_fused(q, k, v, beta, g, initial_state=None, *, scale: float, chunk: int = 64):
    """Gated delta rule on raw (un-normalised) q, k ``[B,T,H,d]``; l2norm and the ``scale`` on q are
    applied inside.  Returns ``(o [B,T,H,dv], final_state [B,H,dk,dv] fp32)``."""
    return _GdnChunked.apply(q, k, v, beta, g, initial_state, scale, chunk)
