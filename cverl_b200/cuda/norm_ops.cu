// Row-wise normalisation kernels (bf16 in/out, fp32 math), fused with what
// surrounds them in the Qwen3.5 / Qwen3-MoE blocks:
//   * residual add + RMSNorm  (h = x + r; y = h * rstd * (w0 + w))
//   * gated RMSNorm           (y = x * rstd * w * silu(z)), linear-attention output
//   * per-head q/k RMSNorm + partial rotary embedding in one pass
// and their backward passes, which accumulate weight gradients in fp32 with
// atomics into the flat main-grad buffer.
//
// One sub-warp per row: a row of D elements is covered by min(32, D/8) lanes,
// each holding 8-element (16-byte) vectors, so that D = 128 ... 8192 all run
// with coalesced 16-byte accesses and shuffle-only reductions.
//
// Reference behaviour: src/model/qwen3_5_text.cc:698-711 (RMSNorm, gated
// RMSNorm, fp32 compute), :724-757 and :1057-1066 (partial RoPE).
#include "ptx.cuh"
#include <initializer_list>

namespace cvb {

constexpr int NORM_THREADS = 256;

struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* p) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  Vec8 r;
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    r.v[2 * i] = f.x;
    r.v[2 * i + 1] = f.y;
  }
  return r;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Vec8& r) {
  uint4 u;
  u.x = pack_bf16x2(r.v[0], r.v[1]);
  u.y = pack_bf16x2(r.v[2], r.v[3]);
  u.z = pack_bf16x2(r.v[4], r.v[5]);
  u.w = pack_bf16x2(r.v[6], r.v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float seg_sum(float v, int lanes) {
  for (int o = lanes >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------------------
// forward: optional residual add, optional gate
// ---------------------------------------------------------------------------
// Element offset of gate row `row`.  block = 0: rows lie `stride` apart.  block > 0: the rows are (token, head)
// pairs of a column range of a wider [tokens, ...] tensor: `block` heads per token lie `stride` apart and the
// tokens `block_stride` apart.
__device__ __forceinline__ long long gate_off(long long row, long long stride, int block, long long block_stride) {
  if (block <= 0) return row * stride;
  const long long tok = row / block;
  return tok * block_stride + (row - tok * block) * stride;
}

template <int NVEC>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ resid_in,
                   const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ gate,
                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ resid_out,
                   float* __restrict__ rstd_out, long long rows, int D, long long x_stride,
                   long long gate_stride, float eps, float w_offset, int gate_block, long long gate_block_stride) {
  const int lanes = min(32, D / 8);
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes;
  const int sl = lane % lanes;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * NORM_THREADS + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * NORM_THREADS) >> 5;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += warps_total * rows_per_warp) {
    const long long row = r0 + sub;
    const bool ok = row < rows;
    float ss = 0.f;
    Vec8 h[NVEC];
    if (ok) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        Vec8 a = load8(x + row * x_stride + c);
        if (resid_in) {
          Vec8 b = load8(resid_in + row * D + c);
#pragma unroll
          for (int j = 0; j < 8; ++j) a.v[j] += b.v[j];
        }
        if (resid_out) {
          store8(resid_out + row * D + c, a);
          // the norm sees the bf16-rounded residual stream, as a consumer reading it back would
#pragma unroll
          for (int j = 0; j < 8; ++j) a.v[j] = __bfloat162float(__float2bfloat16_rn(a.v[j]));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += a.v[j] * a.v[j];
        h[i] = a;
      }
    }
    ss = seg_sum(ss, lanes);
    const float rstd = rsqrtf(ss / D + eps);
    if (ok) {
      if (rstd_out && sl == 0) rstd_out[row] = rstd;
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        const Vec8 a = h[i];
        Vec8 ww = load8(w + c);
        Vec8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = a.v[j] * rstd * (w_offset + ww.v[j]);
        if (gate) {
          Vec8 g = load8(gate + gate_off(row, gate_stride, gate_block, gate_block_stride) + c);
#pragma unroll
          for (int j = 0; j < 8; ++j) o.v[j] *= silu_f(g.v[j]);
        }
        store8(y + row * D + c, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// backward
//   dx = dres + rstd * (g - xhat * mean(g * xhat)),  g = dy * (w0 + w) [* silu(z)]
//   dw += sum_rows dy [* silu(z)] * xhat ;  dz = dy * xhat * (w0+w) * silu'(z)
// ---------------------------------------------------------------------------
template <int NVEC>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ dres,
                   __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dgate,
                   float* __restrict__ dw, long long rows, int D, long long x_stride,
                   long long gate_stride, long long dx_stride, float w_offset, int gate_block,
                   long long gate_block_stride, long long dgate_stride, long long dgate_block_stride) {
  extern __shared__ float s_dw[];  // [D]
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) s_dw[i] = 0.f;
  __syncthreads();
  const int lanes = min(32, D / 8);
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes;
  const int sl = lane % lanes;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * NORM_THREADS + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * NORM_THREADS) >> 5;
  float dw_acc[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += warps_total * rows_per_warp) {
    const long long row = r0 + sub;
    const bool ok = row < rows;
    const float rstd = ok ? rstd_in[row] : 0.f;
    float dot = 0.f;
    if (ok) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        Vec8 a = load8(x + row * x_stride + c);
        Vec8 g = load8(dy + row * D + c);
        Vec8 ww = load8(w + c);
        Vec8 z;
        if (gate) z = load8(gate + gate_off(row, gate_stride, gate_block, gate_block_stride) + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float gg = g.v[j] * (w_offset + ww.v[j]);
          if (gate) gg *= silu_f(z.v[j]);
          dot += gg * a.v[j] * rstd;
        }
      }
    }
    dot = seg_sum(dot, lanes) / D;
    if (ok) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        Vec8 a = load8(x + row * x_stride + c);
        Vec8 g = load8(dy + row * D + c);
        Vec8 ww = load8(w + c);
        Vec8 z, o, dz;
        if (gate) z = load8(gate + gate_off(row, gate_stride, gate_block, gate_block_stride) + c);
        Vec8 dr;
        if (dres) dr = load8(dres + row * D + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = a.v[j] * rstd;
          const float wj = w_offset + ww.v[j];
          float gy = g.v[j];
          if (gate) {
            const float sg = sigmoid_f(z.v[j]);
            const float sz = z.v[j] * sg;
            dz.v[j] = gy * xhat * wj * (sg * (1.f + z.v[j] * (1.f - sg)));
            gy *= sz;
          }
          const float gg = gy * wj;
          o.v[j] = rstd * (gg - xhat * dot) + (dres ? dr.v[j] : 0.f);
          dw_acc[i][j] += gy * xhat;
        }
        store8(dx + row * dx_stride + c, o);
        if (gate) store8(dgate + gate_off(row, dgate_stride, gate_block, dgate_block_stride) + c, dz);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * lanes + sl) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&s_dw[c + j], dw_acc[i][j]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) {
    const float v = s_dw[i];
    if (v != 0.f) atomicAdd(&dw[i], v);
  }
}

// ---------------------------------------------------------------------------
// q/k head RMSNorm + partial RoPE.  Rows are (token, head); D = head_dim.
// The first `rot` dims are rotated in "rotate_half" form:
//   out[i]       = n[i]*cos[i] - n[i+rot/2]*sin[i]        (i <  rot/2)
//   out[i+rot/2] = n[i+rot/2]*cos[i] + n[i]*sin[i]
// with cos/sin read from fp32 tables [max_pos, rot/2].  `inverse` applies the transposed
// rotation (backward).  pos = positions[token] or token % seq_len.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(NORM_THREADS)
headnorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         const int* __restrict__ positions, __nv_bfloat16* __restrict__ y,
                         float* __restrict__ rstd_out, long long tokens, int heads, int D,
                         long long x_tok_stride, long long x_head_stride, int rot,
                         const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                         int seq_len, float eps, float w_offset, int use_norm) {
  const int lanes = D / 8;  // D in {64,128,256}
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes;
  const int sl = lane % lanes;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * NORM_THREADS + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * NORM_THREADS) >> 5;
  const long long rows = tokens * heads;
  const int half = rot / 2;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += warps_total * rows_per_warp) {
    const long long row = r0 + sub;
    const bool ok = row < rows;
    const long long tok = ok ? row / heads : 0;
    const int head = ok ? static_cast<int>(row % heads) : 0;
    const int c = sl * 8;
    Vec8 a;
    float ss = 0.f;
    if (ok) {
      a = load8(x + tok * x_tok_stride + head * x_head_stride + c);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += a.v[j] * a.v[j];
    }
    ss = seg_sum(ss, lanes);
    float rstd = 1.f;
    if (use_norm) {
      rstd = rsqrtf(ss / D + eps);
      Vec8 ww;
      if (ok) ww = load8(w + c);
      if (ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) a.v[j] = a.v[j] * rstd * (w_offset + ww.v[j]);
      }
    }
    // rotation partner lives `half` elements away = half/8 lanes away
    const int pos = ok ? (positions ? positions[tok] : static_cast<int>(tok % seq_len)) : 0;
    Vec8 o = a;
    const int partner_lane_off = half / 8;
    const bool in_lo = c < half;
    const bool in_rot = c < rot;
    const int src_lane = (lane - sl) + (in_lo ? sl + partner_lane_off : sl - partner_lane_off);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float other = __shfl_sync(0xffffffffu, a.v[j], in_rot ? src_lane : lane);
      if (in_rot && ok) {
        const int i = (in_lo ? c : c - half) + j;
        const float cs = cos_tab[static_cast<long long>(pos) * half + i];
        const float sn = sin_tab[static_cast<long long>(pos) * half + i];
        o.v[j] = in_lo ? (a.v[j] * cs - other * sn) : (a.v[j] * cs + other * sn);
      }
    }
    if (ok) {
      store8(y + row * D + c, o);
      if (rstd_out && sl == 0) rstd_out[row] = rstd;
    }
  }
}

// backward: dn = R^T dy ; then RMSNorm backward on dn (if use_norm)
__global__ void __launch_bounds__(NORM_THREADS)
headnorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                         const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                         const int* __restrict__ positions, __nv_bfloat16* __restrict__ dx,
                         float* __restrict__ dw, long long tokens, int heads, int D,
                         long long x_tok_stride, long long x_head_stride, int rot,
                         const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                         int seq_len, float w_offset, int use_norm) {
  __shared__ float s_dw[256];
  for (int i = threadIdx.x; i < 256; i += NORM_THREADS) s_dw[i] = 0.f;
  __syncthreads();
  const int lanes = D / 8;
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes;
  const int sl = lane % lanes;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * NORM_THREADS + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * NORM_THREADS) >> 5;
  const long long rows = tokens * heads;
  const int half = rot / 2;
  float dw_acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) dw_acc[j] = 0.f;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += warps_total * rows_per_warp) {
    const long long row = r0 + sub;
    const bool ok = row < rows;
    const long long tok = ok ? row / heads : 0;
    const int head = ok ? static_cast<int>(row % heads) : 0;
    const int c = sl * 8;
    Vec8 g;
#pragma unroll
    for (int j = 0; j < 8; ++j) g.v[j] = 0.f;
    if (ok) g = load8(dy + row * D + c);
    const int pos = ok ? (positions ? positions[tok] : static_cast<int>(tok % seq_len)) : 0;
    const int partner_lane_off = half / 8;
    const bool in_lo = c < half;
    const bool in_rot = c < rot;
    const int src_lane = (lane - sl) + (in_lo ? sl + partner_lane_off : sl - partner_lane_off);
    Vec8 dn = g;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float other = __shfl_sync(0xffffffffu, g.v[j], in_rot ? src_lane : lane);
      if (in_rot && ok) {
        const int i = (in_lo ? c : c - half) + j;
        const float cs = cos_tab[static_cast<long long>(pos) * half + i];
        const float sn = sin_tab[static_cast<long long>(pos) * half + i];
        // transpose of the forward rotation
        dn.v[j] = in_lo ? (g.v[j] * cs + other * sn) : (g.v[j] * cs - other * sn);
      }
    }
    if (!use_norm) {
      if (ok) store8(dx + row * D + c, dn);
      continue;
    }
    Vec8 a, ww;
#pragma unroll
    for (int j = 0; j < 8; ++j) a.v[j] = 0.f, ww.v[j] = 0.f;
    if (ok) {
      a = load8(x + tok * x_tok_stride + head * x_head_stride + c);
      ww = load8(w + c);
    }
    const float rstd = ok ? rstd_in[row] : 0.f;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += dn.v[j] * (w_offset + ww.v[j]) * a.v[j] * rstd;
    dot = seg_sum(dot, lanes) / D;
    Vec8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xhat = a.v[j] * rstd;
      o.v[j] = rstd * (dn.v[j] * (w_offset + ww.v[j]) - xhat * dot);
      dw_acc[j] += dn.v[j] * xhat;
    }
    if (ok) store8(dx + row * D + c, o);
  }
  if (use_norm) {
    const int c = sl * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&s_dw[c + j], dw_acc[j]);
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += NORM_THREADS) {
      const float v = s_dw[i];
      if (v != 0.f) atomicAdd(&dw[i], v);
    }
  }
}

// vectors of 8 per lane for a row of D elements, or -1 when D is not supported

// ---------------------------------------------------------------------------
// Sequence-parallel residual add + RMSNorm (tensor parallelism with the residual stream sharded by token rows).
//
// forward:  x = sum_p parts[p] (+ resid_in) over this rank's rows; resid_out = x; y = rmsnorm(x) is stored at row
//           `dst_row0 + row` of EVERY buffer in `ydst` - the local copy and, through peer-mapped pointers over
//           NVLink, the copy on every other rank of the tensor-parallel group: the stores ARE the all-gather that
//           the following column-parallel GEMM needs.  `parts` are the `nparts` partial products that the
//           row-parallel GEMMs of all ranks scattered into this rank's buffer (their reduce-scatter), lying
//           `part_stride` elements apart.
// backward: dy = sum_p dy_parts[p] (the column-parallel input-gradient partials, scattered the same way);
//           dx = dres + rstd * (g - xhat * mean(g * xhat)), g = dy * (w0 + w); dx goes to `dx_local` and to row
//           `dst_row0 + row` of every buffer in `dxdst` (the all-gather of the row-parallel GEMM's output gradient).
// ---------------------------------------------------------------------------
struct SpDst {
  __nv_bfloat16* p[8];
};

template <int NVEC>
__global__ void __launch_bounds__(NORM_THREADS)
sp_add_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ parts, long long part_stride, int nparts,
                          const __nv_bfloat16* __restrict__ resid_in, const __nv_bfloat16* __restrict__ w,
                          SpDst ydst, int ndst, long long dst_row0, __nv_bfloat16* __restrict__ resid_out,
                          float* __restrict__ rstd_out, long long rows, int D, float eps, float w_offset) {
  const int lanes = min(32, D / 8);
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes;
  const int sl = lane % lanes;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * NORM_THREADS + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * NORM_THREADS) >> 5;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += warps_total * rows_per_warp) {
    const long long row = r0 + sub;
    const bool ok = row < rows;
    float ss = 0.f;
    Vec8 h[NVEC];
    if (ok) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        Vec8 a = load8(parts + row * D + c);
        for (int q = 1; q < nparts; ++q) {
          Vec8 b = load8(parts + q * part_stride + row * D + c);
#pragma unroll
          for (int j = 0; j < 8; ++j) a.v[j] += b.v[j];
        }
        if (resid_in) {
          Vec8 b = load8(resid_in + row * D + c);
#pragma unroll
          for (int j = 0; j < 8; ++j) a.v[j] += b.v[j];
        }
        store8(resid_out + row * D + c, a);
        // the norm sees the bf16-rounded residual stream, as a consumer reading it back would
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a.v[j] = __bfloat162float(__float2bfloat16_rn(a.v[j]));
          ss += a.v[j] * a.v[j];
        }
        h[i] = a;
      }
    }
    ss = seg_sum(ss, lanes);
    const float rstd = rsqrtf(ss / D + eps);
    if (ok) {
      if (sl == 0) rstd_out[row] = rstd;
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        const Vec8 a = h[i];
        Vec8 ww = load8(w + c);
        Vec8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = a.v[j] * rstd * (w_offset + ww.v[j]);
        for (int d = 0; d < ndst; ++d) store8(ydst.p[d] + (dst_row0 + row) * D + c, o);
      }
    }
  }
}

template <int NVEC>
__global__ void __launch_bounds__(NORM_THREADS)
sp_add_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy_parts, long long part_stride, int nparts,
                          const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                          const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                          __nv_bfloat16* __restrict__ dx_local, SpDst dxdst, int ndst, long long dst_row0,
                          float* __restrict__ dw, long long rows, int D, float w_offset) {
  extern __shared__ float s_dw[];  // [D]
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) s_dw[i] = 0.f;
  __syncthreads();
  const int lanes = min(32, D / 8);
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes;
  const int sl = lane % lanes;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * NORM_THREADS + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * NORM_THREADS) >> 5;
  float dw_acc[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += warps_total * rows_per_warp) {
    const long long row = r0 + sub;
    const bool ok = row < rows;
    const float rstd = ok ? rstd_in[row] : 0.f;
    float dot = 0.f;
    Vec8 gsum[NVEC];
    if (ok) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        Vec8 a = load8(x + row * D + c);
        Vec8 g = load8(dy_parts + row * D + c);
        for (int q = 1; q < nparts; ++q) {
          Vec8 b = load8(dy_parts + q * part_stride + row * D + c);
#pragma unroll
          for (int j = 0; j < 8; ++j) g.v[j] += b.v[j];
        }
        Vec8 ww = load8(w + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += g.v[j] * (w_offset + ww.v[j]) * a.v[j] * rstd;
        gsum[i] = g;
      }
    }
    dot = seg_sum(dot, lanes) / D;
    if (ok) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * lanes + sl) * 8;
        Vec8 a = load8(x + row * D + c);
        const Vec8 g = gsum[i];
        Vec8 ww = load8(w + c);
        Vec8 o, dr;
        if (dres) dr = load8(dres + row * D + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = a.v[j] * rstd;
          const float gg = g.v[j] * (w_offset + ww.v[j]);
          o.v[j] = rstd * (gg - xhat * dot) + (dres ? dr.v[j] : 0.f);
          dw_acc[i][j] += g.v[j] * xhat;
        }
        if (dx_local) store8(dx_local + row * D + c, o);
        for (int d = 0; d < ndst; ++d) store8(dxdst.p[d] + (dst_row0 + row) * D + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * lanes + sl) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&s_dw[c + j], dw_acc[i][j]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) {
    const float v = s_dw[i];
    if (v != 0.f) atomicAdd(&dw[i], v);
  }
}

static int norm_nvec(int D) {
  if (D % 8 != 0 || D <= 0) return -1;
  const int v = D / 8;
  if (v < 32) return (32 % v == 0) ? 1 : -1;
  if (v % 32 != 0) return -1;
  return v / 32;
}

static int norm_grid(long long rows, int rows_per_warp) {
  long long warps = (rows + rows_per_warp - 1) / rows_per_warp;
  long long blocks = (warps + (NORM_THREADS / 32) - 1) / (NORM_THREADS / 32);
  const long long cap = 148LL * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace cvb

using namespace cvb;
// every vector access in this file is 16 bytes wide: refuse misaligned tensors on the host
static inline bool cvb_misaligned(std::initializer_list<const void*> ptrs) {
  for (const void* q : ptrs)
    if (q != nullptr && (reinterpret_cast<uintptr_t>(q) & 15)) return true;
  return false;
}

extern "C" int cvb_rmsnorm_fwd(const void* x, const void* resid_in, const void* w, const void* gate, void* y,
                               void* resid_out, float* rstd, long long rows, int D, long long x_stride,
                               long long gate_stride, float eps, float w_offset, int gate_block,
                               long long gate_block_stride, void* stream) {
  const int nvec = norm_nvec(D);
  if (nvec < 0) return -1;
  if (cvb_misaligned({x, resid_in, w, gate, y, resid_out}) || x_stride % 8 || gate_stride % 8 ||
      gate_block_stride % 8 || gate_block < 0)
    return -2;
  if (rows <= 0) return 0;
  const int lanes = D / 8 < 32 ? D / 8 : 32;
#define CVB_FWD(NV)                                                                                          \
  case NV:                                                                                                   \
    rmsnorm_fwd_kernel<NV><<<norm_grid(rows, 32 / lanes), NORM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>( \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(resid_in),                   \
        static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(gate),                       \
        static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(resid_out), rstd, rows, D, x_stride,     \
        gate_stride, eps, w_offset, gate_block, gate_block_stride);                                          \
    break;
  switch (nvec) {
    CVB_FWD(1) CVB_FWD(2) CVB_FWD(3) CVB_FWD(4) CVB_FWD(5) CVB_FWD(6) CVB_FWD(7) CVB_FWD(8) CVB_FWD(12)
    CVB_FWD(14) CVB_FWD(16)
    default: return -1;
  }
#undef CVB_FWD
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* gate,
                               const void* dres, void* dx, void* dgate, float* dw, long long rows, int D,
                               long long x_stride, long long gate_stride, long long dx_stride, float w_offset,
                               int gate_block, long long gate_block_stride, long long dgate_stride,
                               long long dgate_block_stride, void* stream) {
  // gate rows: see gate_off(); dgate has the same row grouping with its own two strides
  const int nvec = norm_nvec(D);
  if (nvec < 0) return -1;
  if (cvb_misaligned({dy, x, w, gate, dres, dx, dgate}) || x_stride % 8 || gate_stride % 8 || dx_stride % 8 ||
      gate_block_stride % 8 || dgate_stride % 8 || dgate_block_stride % 8 || gate_block < 0)
    return -2;
  if (rows <= 0) return 0;
  const int lanes = D / 8 < 32 ? D / 8 : 32;
  int grid = norm_grid(rows, 32 / lanes);
  // One resident wave (fewer CTAs = fewer global atomics on dw): the 128-wide rows of the head norms need 80
  // registers, so three CTAs fit per SM; the wider instantiations fit two.
  static const int per_sm_env = [] { const char* e = getenv("CVERL_B200_NORM_BWD_CTAS_PER_SM"); return e ? atoi(e) : 0; }();
  const int per_sm = per_sm_env > 0 ? per_sm_env : (nvec <= 1 ? 3 : 2);
  if (grid > 148 * per_sm) grid = 148 * per_sm;
#define CVB_BWD(NV)                                                                                        \
  case NV:                                                                                                  \
    rmsnorm_bwd_kernel<NV><<<grid, NORM_THREADS, D * sizeof(float), static_cast<cudaStream_t>(stream)>>>(   \
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),                        \
        static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(gate),                \
        static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx),                           \
        static_cast<__nv_bfloat16*>(dgate), dw, rows, D, x_stride, gate_stride, dx_stride, w_offset,        \
        gate_block, gate_block_stride, dgate_stride, dgate_block_stride);                                   \
    break;
  switch (nvec) {
    CVB_BWD(1) CVB_BWD(2) CVB_BWD(3) CVB_BWD(4) CVB_BWD(5) CVB_BWD(6) CVB_BWD(7) CVB_BWD(8) CVB_BWD(12)
    CVB_BWD(14) CVB_BWD(16)
    default: return -1;
  }
#undef CVB_BWD
  return static_cast<int>(cudaGetLastError());
}


static bool sp_fill(SpDst* d, void* const* ptrs, int n) {
  if (n < 0 || n > 8) return false;
  for (int i = 0; i < 8; ++i) d->p[i] = nullptr;
  for (int i = 0; i < n; ++i) {
    if (!ptrs || !ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return false;
    d->p[i] = static_cast<__nv_bfloat16*>(ptrs[i]);
  }
  return true;
}

// `ydst`: `ndst` device pointers (host array), the copies of the gathered output on the ranks of the group; this
// rank's rows land at row `dst_row0` of each.  `parts`: `nparts` partial inputs `part_stride` elements apart.
extern "C" int cvb_sp_add_rmsnorm_fwd(const void* parts, long long part_stride, int nparts, const void* resid_in,
                                      const void* w, void* const* ydst, int ndst, long long dst_row0,
                                      void* resid_out, float* rstd, long long rows, int D, float eps,
                                      float w_offset, void* stream) {
  const int nvec = norm_nvec(D);
  SpDst dst;
  if (nvec < 0 || nparts < 1 || nparts > 8 || !sp_fill(&dst, ydst, ndst) || !resid_out || !rstd) return -1;
  if (cvb_misaligned({parts, resid_in, w, resid_out}) || part_stride % 8 || dst_row0 < 0) return -2;
  if (rows <= 0) return 0;
  const int lanes = D / 8 < 32 ? D / 8 : 32;
#define CVB_SPF(NV)                                                                                           \
  case NV:                                                                                                    \
    sp_add_rmsnorm_fwd_kernel<NV><<<norm_grid(rows, 32 / lanes), NORM_THREADS, 0,                             \
                                    static_cast<cudaStream_t>(stream)>>>(                                     \
        static_cast<const __nv_bfloat16*>(parts), part_stride, nparts,                                        \
        static_cast<const __nv_bfloat16*>(resid_in), static_cast<const __nv_bfloat16*>(w), dst, ndst,         \
        dst_row0, static_cast<__nv_bfloat16*>(resid_out), rstd, rows, D, eps, w_offset);                      \
    break;
  switch (nvec) {
    CVB_SPF(1) CVB_SPF(2) CVB_SPF(3) CVB_SPF(4) CVB_SPF(5) CVB_SPF(6) CVB_SPF(7) CVB_SPF(8) CVB_SPF(12)
    CVB_SPF(14) CVB_SPF(16)
    default: return -1;
  }
#undef CVB_SPF
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_sp_add_rmsnorm_bwd(const void* dy_parts, long long part_stride, int nparts, const void* x,
                                      const void* w, const float* rstd, const void* dres, void* dx_local,
                                      void* const* dxdst, int ndst, long long dst_row0, float* dw,
                                      long long rows, int D, float w_offset, void* stream) {
  const int nvec = norm_nvec(D);
  SpDst dst;
  if (nvec < 0 || nparts < 1 || nparts > 8 || !sp_fill(&dst, dxdst, ndst) || !dw || !rstd) return -1;
  if (cvb_misaligned({dy_parts, x, w, dres, dx_local}) || part_stride % 8 || dst_row0 < 0) return -2;
  if (rows <= 0) return 0;
  const int lanes = D / 8 < 32 ? D / 8 : 32;
  int grid = norm_grid(rows, 32 / lanes);
  if (grid > 148 * 2) grid = 148 * 2;
#define CVB_SPB(NV)                                                                                           \
  case NV:                                                                                                    \
    sp_add_rmsnorm_bwd_kernel<NV><<<grid, NORM_THREADS, D * sizeof(float), static_cast<cudaStream_t>(stream)>>>( \
        static_cast<const __nv_bfloat16*>(dy_parts), part_stride, nparts, static_cast<const __nv_bfloat16*>(x), \
        static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),                  \
        static_cast<__nv_bfloat16*>(dx_local), dst, ndst, dst_row0, dw, rows, D, w_offset);                   \
    break;
  switch (nvec) {
    CVB_SPB(1) CVB_SPB(2) CVB_SPB(3) CVB_SPB(4) CVB_SPB(5) CVB_SPB(6) CVB_SPB(7) CVB_SPB(8) CVB_SPB(12)
    CVB_SPB(14) CVB_SPB(16)
    default: return -1;
  }
#undef CVB_SPB
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_headnorm_rope_fwd(const void* x, const void* w, const int* positions, void* y, float* rstd,
                                     long long tokens, int heads, int D, long long x_tok_stride,
                                     long long x_head_stride, int rot, const float* cos_tab,
                                     const float* sin_tab, int seq_len, float eps, float w_offset,
                                     int use_norm, void* stream) {
  if (!(D == 64 || D == 128 || D == 256) || rot % 16 != 0 || rot > D) return -1;
  if (cvb_misaligned({x, w, y}) || x_tok_stride % 8 || x_head_stride % 8) return -2;
  if (tokens <= 0) return 0;
  headnorm_rope_fwd_kernel<<<norm_grid(tokens * heads, 32 / (D / 8)), NORM_THREADS, 0,
                             static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), positions,
      static_cast<__nv_bfloat16*>(y), rstd, tokens, heads, D, x_tok_stride, x_head_stride, rot, cos_tab,
      sin_tab, seq_len, eps, w_offset, use_norm);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_headnorm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                                     const int* positions, void* dx, float* dw, long long tokens, int heads,
                                     int D, long long x_tok_stride, long long x_head_stride, int rot,
                                     const float* cos_tab, const float* sin_tab, int seq_len,
                                     float w_offset, int use_norm, void* stream) {
  if (!(D == 64 || D == 128 || D == 256) || rot % 16 != 0 || rot > D) return -1;
  if (cvb_misaligned({dy, x, w, dx}) || x_tok_stride % 8 || x_head_stride % 8) return -2;
  if (tokens <= 0) return 0;
  int grid = norm_grid(tokens * heads, 32 / (D / 8));
  if (grid > 148 * 2) grid = 148 * 2;
  headnorm_rope_bwd_kernel<<<grid, NORM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, positions, static_cast<__nv_bfloat16*>(dx), dw, tokens,
      heads, D, x_tok_stride, x_head_stride, rot, cos_tab, sin_tab, seq_len, w_offset, use_norm);
  return static_cast<int>(cudaGetLastError());
}
