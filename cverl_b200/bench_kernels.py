"""Per-kernel micro-benchmarks with roofline fractions.

``python -m cverl_b200.bench_kernels --kernel gemm_nt [--m 8192 --n 8192 --k 8192] [--iters 10]``

Each case times one hot kernel with CUDA events after warm-up, on operands larger than the 126 MB L2
(or with an L2 flush between iterations for the small ones), and prints one JSON line with the
achieved TFLOP/s or GB/s and its fraction of the measured peak (``MEASURED_PEAKS.json`` beside the
package when present, else the stated fallback).  ``--small`` shrinks the case to a few hundred MB
for profiler captures.  The same cases serve as the kernel rows of the performance tables.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def _peaks():
    p = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return dict(FALLBACK, source="fallback")


class _Flush:
    def __init__(self, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def _time(fn, iters, flush=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _bf(*shape, dev, scale=1.0):
    return (scale * torch.randn(*shape, device=dev)).to(torch.bfloat16)


def case_gemm(a, dev, kind):
    from . import ops
    M, N, K = a.m, a.n, a.k
    if kind == "gemm_nt":
        x, w = _bf(M, K, dev=dev), _bf(N, K, dev=dev)
        fn = lambda: ops.gemm_nt(x, w)
    elif kind == "gemm_nn":
        x, w = _bf(M, K, dev=dev), _bf(K, N, dev=dev)
        fn = lambda: ops.gemm_nn(x, w)
    else:
        x, w = _bf(K, M, dev=dev), _bf(K, N, dev=dev)
        acc = torch.zeros(M, N, device=dev)
        fn = lambda: ops.gemm_tn_acc(x, w, acc)
    return fn, 2.0 * M * N * K, None


def case_gemm_scatter(a, dev):
    """The reduce-scatter epilogue of the tensor-parallel row-parallel GEMM on ONE device: the row blocks of the
    partial product go to two different buffers (the "owners"), both in local memory here, exactly as they would
    go to this rank's and a peer's buffer over NVLink.  Serves profiler captures of that kernel, which must not
    run under a multi-rank command."""
    from . import _native as nv
    from .ops import gemm as G
    M, N, K = a.m, a.n, a.k
    if M % 256 or N % 64:
        raise SystemExit("gemm_scatter needs m % 256 == 0 and n % 64 == 0")
    x, w = _bf(M, K, dev=dev), _bf(N, K, dev=dev)
    rl = M // 2
    owners = [torch.empty(2, rl, N, device=dev, dtype=torch.bfloat16) for _ in range(2)]   # [slot][rows, N]
    me = 0
    bases = [owners[o].data_ptr() + (me * rl - o * rl) * N * 2 for o in range(2)]

    def fn():
        G.gemm_raw(x, w, None, M, N, K, a_mn=False, b_mn=False, epi=nv.EPI_STORE_BF16,
                   block_n=G._pick_block_n(M, N), scatter=(bases, rl), ldc=N)
    return fn, 2.0 * M * N * K, None


def case_peer_emulated(a, dev, which):
    """The self-communicating kernels with every "peer" buffer in this device's own memory: the same code and the
    same access pattern as across NVLink (profiler captures must not run under a multi-rank command, and two
    ranks' kernels that wait on each other must not share a GPU - these cases have no waits).

    rs_acc          ZeRO-2 bucket reduce-scatter: pull this rank's piece from ``world`` gradient buffers, accumulate
    adamw_allgather FlatAdamW on a shard whose bf16 result is stored into ``world`` parameter buffers
    bcast_store     weight push: one read, one store per destination
    sp_norm_fwd     sequence-parallel TP: sum of ``world`` GEMM partial slots + residual + RMSNorm on T / world rows,
                    normalised rows stored into ``world`` gathered buffers
    attn_merge      merge of one ring-attention hop's partial result into the fp32 accumulator
    """
    import ctypes as C
    from . import _native as nv
    world = 4
    st = lambda: nv.stream()   # noqa: E731
    if which in ("rs_acc", "adamw_allgather", "bcast_store"):
        n = a.numel // (world * 8) * (world * 8)
        shard = n // world
        if which == "rs_acc":
            bufs = [torch.full((n,), 1e-3 * (i + 1), dtype=torch.float32, device=dev) for i in range(world)]
            ptrs = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
            out = torch.zeros(shard, dtype=torch.float32, device=dev)
            fn = lambda: nv.check(nv.cuda().cvb_reduce_scatter_acc(ptrs, world, 1, shard, shard, 1.0 / world,
                                                                   out.data_ptr(), 0, 0, st()), "rs_acc")
            return fn, None, (world + 2) * shard * 4, bufs
        if which == "adamw_allgather":
            params = [torch.zeros(n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
            ptrs = (C.c_void_p * world)(*[b.data_ptr() for b in params])
            g, m, v = (torch.full((shard,), 1e-3, dtype=torch.float32, device=dev) for _ in range(3))
            fn = lambda: nv.check(nv.cuda().cvb_flat_adamw_allgather(g.data_ptr(), None, m.data_ptr(), v.data_ptr(),
                                                                     None, ptrs, world, 1, shard, shard, 1e-6, 0.9,
                                                                     0.95, 1e-8, 0.01, 1, st()), "adamw_allgather")
            return fn, None, shard * (4 * 5 + 2 + 2 * world), (params, g, m, v)
        src = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        dsts = [torch.empty(n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        ptrs = (C.c_void_p * world)(*[b.data_ptr() for b in dsts])
        fn = lambda: nv.check(nv.cuda().cvb_broadcast_store(src.data_ptr(), ptrs, world, n * 2, st()), "bcast_store")
        return fn, None, n * 2 * (1 + world), (src, dsts)
    if which == "sp_norm_fwd":
        T, H = 81920, 1024            # 64 sequences x 1280 tokens: the benchmark's micro-batch at TP=2
        rl = T // world
        parts = _bf(world, rl, H, dev=dev)
        resid, w = _bf(rl, H, dev=dev), _bf(H, dev=dev, scale=0.1)
        gathered = [torch.empty(T, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        dst = (C.c_void_p * world)(*[g.data_ptr() for g in gathered])
        resid_out = torch.empty(rl, H, dtype=torch.bfloat16, device=dev)
        rstd = torch.empty(rl, dtype=torch.float32, device=dev)
        fn = lambda: nv.check(nv.cuda().cvb_sp_add_rmsnorm_fwd(parts.data_ptr(), rl * H, world, resid.data_ptr(),
                                                               w.data_ptr(), dst, world, rl, resid_out.data_ptr(),
                                                               rstd.data_ptr(), rl, H, 1e-6, 1.0, st()), "sp_norm_fwd")
        return fn, None, rl * H * 2 * (world + 2 + world), (parts, gathered)
    if which == "attn_merge":
        B, T, Hq, D = 1, a.batch * 2048, 8, a.head_dim
        acc = torch.randn(B, T, Hq, D, device=dev)
        lse = torch.randn(B, Hq, T, device=dev)
        part, lp = _bf(B, T, Hq, D, dev=dev), torch.randn(B, Hq, T, device=dev)
        fn = lambda: nv.check(nv.cuda().cvb_attn_merge(acc.data_ptr(), lse.data_ptr(), part.data_ptr(), lp.data_ptr(),
                                                       B, T, T, Hq, D, 0, 0, st()), "attn_merge")
        return fn, None, B * T * Hq * D * (4 + 4 + 2), (acc, part)
    raise SystemExit(f"unknown kernel {which}")


def case_lmhead(a, dev, backward):
    from . import ops
    T, H, V = a.m, a.k, a.n
    h = _bf(T, H, dev=dev).requires_grad_(True)
    w = _bf(V, H, dev=dev, scale=0.02).requires_grad_(True)
    w.main_grad = torch.zeros(V, H, device=dev)
    tgt = torch.randint(0, V, (T,), device=dev)
    if not backward:
        def fn():
            with torch.no_grad():
                ops.lmhead_logprob(h, w, tgt, 0, None)
        return fn, 2.0 * T * V * H, None
    g = torch.randn(T, device=dev)

    def fn():
        lp = ops.lmhead_logprob(h, w, tgt, 0, None)
        lp.backward(g)
        h.grad = None
    return fn, 4 * 2.0 * T * V * H, None       # forward + recompute + dX + dW


def _gdn_inputs(a, dev):
    B, T, H = a.batch, a.seq, a.heads
    mixed = _bf(B, T, 3 * H * 128, dev=dev)
    q, k, v = (m.reshape(B, T, H, 128) for m in mixed.split(H * 128, dim=-1))
    beta = torch.sigmoid(torch.randn(B, T, H, device=dev))
    g = -0.3 * torch.rand(B, T, H, device=dev)
    return q, k, v, beta, g


def case_gdn(a, dev, which):
    from .ops import gdn_native as gn
    q, k, v, beta, g = _gdn_inputs(a, dev)
    B, T, H = a.batch, a.seq, a.heads
    scale = 128 ** -0.5
    o, Sf, Vn, SsT, pre = gn.chunk_forward(q, k, v, beta, g, None, scale, keep_prep=True)
    do = torch.randn_like(o)
    tile = B * T * H * 128 * 2            # bytes of one [B,T,H,128] bf16 operand
    state = B * H * (T // 64) * 128 * 128 * 2
    if which == "gdn_prep":
        return (lambda: gn.chunk_prep(q, k, v, beta, g, scale, want_aux=True)), None, 3 * tile + 4.5 * tile + 2 * tile
    if which == "gdn_fwd":
        return (lambda: gn.chunk_forward(q, k, v, beta, g, None, scale)), None, 3 * tile + 2 * (4.5 * tile) + 2 * state + 4 * tile
    if which == "gdn_bwd":
        return (lambda: gn.chunk_backward(q, k, v, beta, scale, pre, Vn, SsT, Sf, do, None)), None, \
            (5 + 4 + 3 + 5) * tile + 3 * state
    raise ValueError(which)


def case_conv(a, dev, backward):
    from . import ops
    B, S, C = a.batch, a.seq, a.channels
    x = _bf(B, S, C, dev=dev).requires_grad_(True)
    w = _bf(C, 4, dev=dev, scale=0.3).requires_grad_(True)
    w.main_grad = torch.zeros(C, 4, device=dev)
    nbytes = B * S * C * 2
    if not backward:
        def fn():
            with torch.no_grad():
                ops.conv1d_silu(x, w)
        return fn, None, 2 * nbytes
    y = ops.conv1d_silu(x, w)
    dy = torch.randn_like(y)

    def fn():
        y.backward(dy, retain_graph=True)
        x.grad = None
    return fn, None, 3 * nbytes


def case_rmsnorm(a, dev, backward):
    from . import ops
    T, H = a.m, a.k
    x, r = _bf(T, H, dev=dev).requires_grad_(True), _bf(T, H, dev=dev).requires_grad_(True)
    w = _bf(H, dev=dev).requires_grad_(True)
    w.main_grad = torch.zeros(H, device=dev)
    nbytes = T * H * 2
    if not backward:
        def fn():
            with torch.no_grad():
                ops.add_rmsnorm(x, r, w, 1e-6, 1.0)
        return fn, None, 4 * nbytes
    y, s = ops.add_rmsnorm(x, r, w, 1e-6, 1.0)
    dy = torch.randn_like(y)

    def fn():
        torch.autograd.backward([y, s], [dy, dy], retain_graph=True)
        x.grad = r.grad = None
    return fn, None, 4 * nbytes


def case_attention(a, dev, backward):
    """Causal GQA attention, Qwen3.5-0.8B shape by default (8 query heads, 2 kv heads, head dim 256)."""
    from .ops import attention
    B, S, Hq, Hkv, D = a.batch, a.seq, a.heads if a.heads != 16 else 8, 2, a.head_dim
    q = _bf(B * S, Hq, D, dev=dev).requires_grad_(True)
    k = _bf(B * S, Hkv, D, dev=dev).requires_grad_(True)
    v = _bf(B * S, Hkv, D, dev=dev).requires_grad_(True)
    flops = 4.0 * B * Hq * S * S * D / 2          # causal: half of the S x S score matrix
    if not backward:
        def fn():
            with torch.no_grad():
                attention.causal_attention(q, k, v, B, S)
        return fn, flops, None
    o = attention.causal_attention(q, k, v, B, S)
    do = torch.randn_like(o)

    def fn():
        o.backward(do, retain_graph=True)
        q.grad = k.grad = v.grad = None
    return fn, 2.5 * flops, None


def case_adamw(a, dev):
    from .ops import optim as oo
    n = a.numel
    g = torch.randn(n, device=dev)
    p = torch.randn(n, device=dev).bfloat16()
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    clip = torch.ones(1, device=dev)
    fn = lambda: oo.flat_adamw_step(g, None, p, m, v, clip=clip, grad_scale=1.0, lr=1e-6, beta1=0.9, beta2=0.95,
                                    eps=1e-8, weight_decay=0.01, step=3, zero_grad=True)
    return fn, None, n * (4 + 4 + 2 + 2 + 8 + 8)


def case_ppo(a, dev):
    from .ops import rl
    rows, cols = a.m, a.k
    old, lp, adv = (torch.randn(rows, cols, device=dev) * 0.1 for _ in range(3))
    mask = (torch.rand(rows, cols, device=dev) > 0.1).float()
    fn = lambda: rl.fused_ppo_loss(old, lp, adv, mask, None, clip_ratio=0.2)
    return fn, None, rows * cols * 4 * 5


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1280)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--channels", type=int, default=6144)
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true", help="a few hundred MB: for profiler captures")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    if a.small:
        a.m, a.n, a.k = min(a.m, 4096), min(a.n, 4096), min(a.k, 4096)
        a.batch, a.numel = min(a.batch, 8), min(a.numel, 1 << 26)
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    k = a.kernel
    if k in ("gemm_nt", "gemm_nn", "gemm_tn"):
        fn, flops, nbytes = case_gemm(a, dev, k)
    elif k == "gemm_scatter":
        fn, flops, nbytes = case_gemm_scatter(a, dev)
    elif k in ("lmhead_fwd", "lmhead_bwd"):
        fn, flops, nbytes = case_lmhead(a, dev, k.endswith("bwd"))
    elif k in ("gdn_prep", "gdn_fwd", "gdn_bwd"):
        fn, flops, nbytes = case_gdn(a, dev, k)
    elif k in ("conv_fwd", "conv_bwd"):
        fn, flops, nbytes = case_conv(a, dev, k.endswith("bwd"))
    elif k in ("rmsnorm_fwd", "rmsnorm_bwd"):
        fn, flops, nbytes = case_rmsnorm(a, dev, k.endswith("bwd"))
    elif k in ("attn_fwd", "attn_bwd"):
        fn, flops, nbytes = case_attention(a, dev, k.endswith("bwd"))
    elif k == "adamw":
        fn, flops, nbytes = case_adamw(a, dev)
    elif k == "ppo_loss":
        fn, flops, nbytes = case_ppo(a, dev)
    elif k in ("rs_acc", "adamw_allgather", "bcast_store", "sp_norm_fwd", "attn_merge"):
        fn, nbytes, keep = (lambda r: (r[0], r[2], r[3]))(case_peer_emulated(a, dev, k))
        flops = None
    else:
        raise SystemExit(f"unknown kernel {k}")
    flush = _Flush(dev) if (nbytes is not None and nbytes < (512 << 20)) or (flops is not None and a.small) else None
    ms = _time(fn, a.iters, flush)
    from . import _native as nv
    nv.check_status(dev)
    pk = _peaks()
    out = {"kernel": k, "ms": ms, "l2": "flushed between iterations" if flush else "operands exceed L2",
           "peaks": pk["source"]}
    if flops is not None:
        out["tflops"] = flops / ms / 1e9
        out["frac_of_bf16_peak"] = out["tflops"] / pk["bf16_tflops"]
    if nbytes is not None:
        out["algorithmic_gbs"] = nbytes / ms / 1e6
        out["frac_of_hbm_peak"] = out["algorithmic_gbs"] / pk["hbm_gbs"]
    out["shape"] = {kk: getattr(a, kk) for kk in ("m", "n", "k", "batch", "seq", "heads", "channels", "numel")}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
