// Fused elementwise kernels of the Qwen3.5 / Qwen3-MoE blocks (bf16 storage,
// fp32 math, 16-byte vector accesses):
//   * SwiGLU        y = silu(g) * u        with [g | u] produced by one GEMM
//   * sigmoid gate  y = a * sigmoid(g)     (attention output gate)
//   * depthwise causal conv1d (k <= 4) + SiLU on channels-last activations
//   * embedding gather and its scatter-add backward into fp32 gradients
//   * fp32 -> bf16 casts, fills
// Reference behaviour: src/model/qwen3_5_text.cc:791-793 (SwiGLU), :1077-1079
// (output gate), :1241-1243 (conv1d + SiLU), :692 (embedding).
#include "ptx.cuh"
#include <initializer_list>

namespace cvb {

constexpr int EW_THREADS = 256;

struct V8 {
  float v[8];
};
__device__ __forceinline__ V8 unpack8v(const uint4& u) {
  V8 r;
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    r.v[2 * j] = f.x;
    r.v[2 * j + 1] = f.y;
  }
  return r;
}
__device__ __forceinline__ V8 ld8(const __nv_bfloat16* p) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  V8 r;
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    r.v[2 * i] = f.x;
    r.v[2 * i + 1] = f.y;
  }
  return r;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const V8& r) {
  uint4 u;
  u.x = pack_bf16x2(r.v[0], r.v[1]);
  u.y = pack_bf16x2(r.v[2], r.v[3]);
  u.z = pack_bf16x2(r.v[4], r.v[5]);
  u.w = pack_bf16x2(r.v[6], r.v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

static int ew_grid(long long n_vec) {
  long long b = (n_vec + EW_THREADS - 1) / EW_THREADS;
  const long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

// ------------------------------- SwiGLU ------------------------------------
// gu: [rows, 2*I] (gate | up), y: [rows, I]
__global__ void __launch_bounds__(EW_THREADS)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, long long rows, int I,
                  long long gu_stride) {
  const int vec_per_row = I / 8;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    V8 g = ld8(gu + r * gu_stride + c);
    V8 u = ld8(gu + r * gu_stride + I + c);
    V8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = g.v[j] * sigm(g.v[j]) * u.v[j];
    st8(y + r * I + c, o);
  }
}
__global__ void __launch_bounds__(EW_THREADS)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                  __nv_bfloat16* __restrict__ dgu, long long rows, int I, long long gu_stride) {
  const int vec_per_row = I / 8;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    V8 g = ld8(gu + r * gu_stride + c);
    V8 u = ld8(gu + r * gu_stride + I + c);
    V8 d = ld8(dy + r * I + c);
    V8 dg, du;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigm(g.v[j]);
      const float sl = g.v[j] * s;
      du.v[j] = d.v[j] * sl;
      dg.v[j] = d.v[j] * u.v[j] * s * (1.f + g.v[j] * (1.f - s));
    }
    st8(dgu + r * 2 * I + c, dg);
    st8(dgu + r * 2 * I + I + c, du);
  }
}

// ---------------------------- sigmoid gate ---------------------------------
// y[r, c] = a[r, c] * sigmoid(g[r, c]); a and g may be strided views.
__global__ void __launch_bounds__(EW_THREADS)
siggate_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ g,
                   __nv_bfloat16* __restrict__ y, long long rows, int C, long long a_stride,
                   long long g_stride, int g_block, int g_block_stride) {
  const int vec_per_row = C / 8;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    // the gate may be interleaved per head: column c of head h lives at h*g_block_stride + (c % g_block)
    const int gc = (c / g_block) * g_block_stride + (c % g_block);
    V8 av = ld8(a + r * a_stride + c);
    V8 gv = ld8(g + r * g_stride + gc);
    V8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = av.v[j] * sigm(gv.v[j]);
    st8(y + r * C + c, o);
  }
}
__global__ void __launch_bounds__(EW_THREADS)
siggate_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ a,
                   const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ da,
                   __nv_bfloat16* __restrict__ dg, long long rows, int C, long long a_stride,
                   long long g_stride, int g_block, int g_block_stride, long long da_stride,
                   long long dg_stride, int dg_block_stride) {
  const int vec_per_row = C / 8;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const int gc = (c / g_block) * g_block_stride + (c % g_block);
    V8 d = ld8(dy + r * C + c);
    V8 av = ld8(a + r * a_stride + c);
    V8 gv = ld8(g + r * g_stride + gc);
    V8 oa, og;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigm(gv.v[j]);
      oa.v[j] = d.v[j] * s;
      og.v[j] = d.v[j] * av.v[j] * s * (1.f - s);
    }
    st8(da + r * da_stride + c, oa);
    st8(dg + r * dg_stride + (c / g_block) * dg_block_stride + (c % g_block), og);
  }
}

// ------------------- depthwise causal conv1d (k=KW) + SiLU -----------------
// x: [B, S, C] channels-last (row stride x_stride), w: [C, KW] bf16.
//   pre[b,s,c] = sum_j w[c,j] * x[b, s-(KW-1)+j, c];  y = silu(pre)
// One thread owns 8 channels and walks `seg_len` consecutive positions with the previous KW-1 inputs in
// registers: one 16-byte load and one 16-byte store per output vector, weights read once per segment.
template <int KW>
__global__ void __launch_bounds__(EW_THREADS)
conv1d_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, long long B, int S, int C, long long x_stride, int seg_len) {
  const int vec_per_row = C / 8;
  const int segs = (S + seg_len - 1) / seg_len;
  const long long total = B * segs * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const long long bs = i / vec_per_row;
    const long long b = bs / segs;
    const int s_begin = static_cast<int>(bs % segs) * seg_len;
    const int s_end = min(S, s_begin + seg_len);
    float wv[8][KW];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int t = 0; t < KW; ++t) wv[j][t] = __bfloat162float(w[(c + j) * KW + t]);
    float win[KW][8];  // win[k] = x[s - (KW-1) + k]
#pragma unroll
    for (int k = 0; k < KW - 1; ++k) {
      const int sp = s_begin - (KW - 1) + k;
      if (sp >= 0) {
        const V8 xv = ld8(x + (b * S + sp) * x_stride + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) win[k + 1][j] = xv.v[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) win[k + 1][j] = 0.f;
      }
    }
    // software pipeline: four rows per group, the next group's loads in flight during the computation
    uint4 xn[4];
    auto fetch = [&](int s0) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        xn[u] = make_uint4(0u, 0u, 0u, 0u);
        if (s0 + u < s_end) xn[u] = *reinterpret_cast<const uint4*>(x + (b * S + s0 + u) * x_stride + c);
      }
    };
    fetch(s_begin);
    for (int s0 = s_begin; s0 < s_end; s0 += 4) {
      uint4 xr[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) xr[u] = xn[u];
      fetch(s0 + 4);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u >= s_end) break;
#pragma unroll
        for (int k = 0; k < KW - 1; ++k)
#pragma unroll
          for (int j = 0; j < 8; ++j) win[k][j] = win[k + 1][j];
        const V8 xv = unpack8v(xr[u]);
        V8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          win[KW - 1][j] = xv.v[j];
          float acc = 0.f;
#pragma unroll
          for (int t = 0; t < KW; ++t) acc += wv[j][t] * win[t][j];
          o.v[j] = acc * sigm(acc);
        }
        st8(y + (b * S + s0 + u) * C + c, o);
      }
    }
  }
}

// backward: recomputes pre; dx[s'] = sum_t w[t] * dpre[s' + (KW-1) - t]; dw[c,t] += sum dpre[s]*x[s-(KW-1)+t]
// One thread owns 4 channels and walks a segment of the sequence, so that dw is reduced in registers
// before the atomics.  Rows are taken four at a time with all eight loads issued up front: each thread
// keeps several memory requests in flight instead of one dependent load per row, and 4 channels per
// thread keep the register count low enough for two resident blocks per SM.
constexpr int CB = 4;  // channels per thread in the backward kernel
__device__ __forceinline__ void unpack4(const uint2& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
}
template <int KW>
__global__ void __launch_bounds__(EW_THREADS, 2)
conv1d_silu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw, long long B, int S, int C, long long x_stride, int seg_len,
                       long long dx_stride) {
  const int vec_per_row = C / CB;
  const int segs = (S + seg_len - 1) / seg_len;
  const long long total = B * segs * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const int c = static_cast<int>(i % vec_per_row) * CB;
    const long long bs = i / vec_per_row;
    const long long b = bs / segs;
    const int s_begin = static_cast<int>(bs % segs) * seg_len;
    const int s_end = min(S, s_begin + seg_len);
    float wv[CB][KW], dwa[CB][KW];
#pragma unroll
    for (int j = 0; j < CB; ++j)
#pragma unroll
      for (int t = 0; t < KW; ++t) wv[j][t] = __bfloat162float(w[(c + j) * KW + t]), dwa[j][t] = 0.f;
    // windows: dpre_win[k] = dpre[s - k], x_win[k] = x[s - k]
    float dpre_win[KW][CB], x_win[KW][CB];
#pragma unroll
    for (int k = 0; k < KW; ++k)
#pragma unroll
      for (int j = 0; j < CB; ++j) dpre_win[k][j] = 0.f, x_win[k][j] = 0.f;
#pragma unroll
    for (int k = 1; k < KW; ++k) {  // x history before s_begin (index k-1: shifted at the loop head)
      const int sp = s_begin - k;
      if (sp >= 0) unpack4(*reinterpret_cast<const uint2*>(x + (b * S + sp) * x_stride + c), x_win[k - 1]);
    }
    const int s_last = s_end + (KW - 1);
    // software pipeline: the loads of group g+1 are in flight while group g is computed
    uint2 xn[4], dn[4];
    auto fetch = [&](int s0) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int s = s0 + u;
        xn[u] = make_uint2(0u, 0u);
        dn[u] = xn[u];
        if (s < s_last && s < S) {
          xn[u] = *reinterpret_cast<const uint2*>(x + (b * S + s) * x_stride + c);
          dn[u] = *reinterpret_cast<const uint2*>(dy + (b * S + s) * C + c);
        }
      }
    };
    fetch(s_begin);
    for (int s0 = s_begin; s0 < s_last; s0 += 4) {
      uint2 xr[4], dr[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) xr[u] = xn[u], dr[u] = dn[u];
      fetch(s0 + 4);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int s = s0 + u;
        if (s >= s_last) break;
#pragma unroll
        for (int k = KW - 1; k > 0; --k)
#pragma unroll
          for (int j = 0; j < CB; ++j) {
            dpre_win[k][j] = dpre_win[k - 1][j];
            x_win[k][j] = x_win[k - 1][j];
          }
        if (s < S) {
          float d[CB];
          unpack4(xr[u], x_win[0]);
          unpack4(dr[u], d);
#pragma unroll
          for (int j = 0; j < CB; ++j) {
            float pre = 0.f;
#pragma unroll
            for (int t = 0; t < KW; ++t) pre += wv[j][t] * x_win[KW - 1 - t][j];
            const float sg = sigm(pre);
            dpre_win[0][j] = d[j] * sg * (1.f + pre * (1.f - sg));
          }
          if (s < s_end) {
#pragma unroll
            for (int j = 0; j < CB; ++j)
#pragma unroll
              for (int t = 0; t < KW; ++t) dwa[j][t] += dpre_win[0][j] * x_win[KW - 1 - t][j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < CB; ++j) dpre_win[0][j] = 0.f, x_win[0][j] = 0.f;
        }
        // dx for position p = s - (KW-1): sum_t w[t] * dpre[p + (KW-1) - t] = sum_t w[t] * dpre_win[t]
        const int p = s - (KW - 1);
        if (p >= s_begin && p < s_end) {
          float o[CB];
#pragma unroll
          for (int j = 0; j < CB; ++j) {
            float acc = 0.f;
#pragma unroll
            for (int t = 0; t < KW; ++t) acc += wv[j][t] * dpre_win[t][j];
            o[j] = acc;
          }
          *reinterpret_cast<uint2*>(dx + (b * S + p) * dx_stride + c) =
              make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < CB; ++j)
#pragma unroll
      for (int t = 0; t < KW; ++t) atomicAdd(dw + (c + j) * KW + t, dwa[j][t]);
  }
}

// ------------------------------- embedding ---------------------------------
__global__ void __launch_bounds__(EW_THREADS)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* __restrict__ out, long long tokens, int H, long long vocab_lo,
                     long long vocab_hi) {
  const int vec_per_row = H / 8;
  const long long total = tokens * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const long long t = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const long long id = ids[t];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= vocab_lo && id < vocab_hi) v = *reinterpret_cast<const uint4*>(table + (id - vocab_lo) * H + c);
    *reinterpret_cast<uint4*>(out + t * H + c) = v;
  }
}
__global__ void __launch_bounds__(EW_THREADS)
embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                     float* __restrict__ dtable, long long tokens, int H, long long vocab_lo,
                     long long vocab_hi) {
  const int vec_per_row = H / 8;
  const long long total = tokens * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    const long long t = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const long long id = ids[t];
    if (id < vocab_lo || id >= vocab_hi) continue;
    V8 d = ld8(dout + t * H + c);
    float* dst = dtable + (id - vocab_lo) * H + c;
    red_add_v4_f32(dst, d.v[0], d.v[1], d.v[2], d.v[3]);
    red_add_v4_f32(dst + 4, d.v[4], d.v[5], d.v[6], d.v[7]);
  }
}

// ------------------------------- casts -------------------------------------
__global__ void __launch_bounds__(EW_THREADS)
cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                        float scale) {
  const long long nv = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * EW_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * EW_THREADS) {
    float4 a = *reinterpret_cast<const float4*>(src + i * 8);
    float4 b = *reinterpret_cast<const float4*>(src + i * 8 + 4);
    uint4 u;
    u.x = pack_bf16x2(a.x * scale, a.y * scale);
    u.y = pack_bf16x2(a.z * scale, a.w * scale);
    u.z = pack_bf16x2(b.x * scale, b.y * scale);
    u.w = pack_bf16x2(b.z * scale, b.w * scale);
    *reinterpret_cast<uint4*>(dst + i * 8) = u;
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 8 + threadIdx.x; i < n; i += EW_THREADS) dst[i] = __float2bfloat16_rn(src[i] * scale);
  }
}

}  // namespace cvb

using namespace cvb;
// every vector access in this file is 16 bytes wide: refuse misaligned tensors on the host
static inline bool cvb_misaligned(std::initializer_list<const void*> ptrs) {
  for (const void* q : ptrs)
    if (q != nullptr && (reinterpret_cast<uintptr_t>(q) & 15)) return true;
  return false;
}
#define BF(p) static_cast<const __nv_bfloat16*>(p)
#define BFM(p) static_cast<__nv_bfloat16*>(p)
#define ST(s) static_cast<cudaStream_t>(s)

extern "C" int cvb_swiglu_fwd(const void* gu, void* y, long long rows, int I, long long gu_stride, void* stream) {
  if (I % 8 || gu_stride % 8 || cvb_misaligned({gu, y})) return -1;
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(rows * (I / 8)), EW_THREADS, 0, ST(stream)>>>(BF(gu), BFM(y), rows, I, gu_stride);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long rows, int I,
                              long long gu_stride, void* stream) {
  if (I % 8 || gu_stride % 8 || cvb_misaligned({dy, gu, dgu})) return -1;
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(rows * (I / 8)), EW_THREADS, 0, ST(stream)>>>(BF(dy), BF(gu), BFM(dgu), rows, I,
                                                                          gu_stride);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_siggate_fwd(const void* a, const void* g, void* y, long long rows, int C, long long a_stride,
                               long long g_stride, int g_block, int g_block_stride, void* stream) {
  if (C % 8 || a_stride % 8 || g_stride % 8 || g_block % 8 || g_block_stride % 8 || cvb_misaligned({a, g, y}))
    return -1;
  if (rows <= 0) return 0;
  siggate_fwd_kernel<<<ew_grid(rows * (C / 8)), EW_THREADS, 0, ST(stream)>>>(BF(a), BF(g), BFM(y), rows, C,
                                                                           a_stride, g_stride, g_block,
                                                                           g_block_stride);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_siggate_bwd(const void* dy, const void* a, const void* g, void* da, void* dg, long long rows,
                               int C, long long a_stride, long long g_stride, int g_block, int g_block_stride,
                               long long da_stride, long long dg_stride, int dg_block_stride, void* stream) {
  if (C % 8 || a_stride % 8 || g_stride % 8 || g_block % 8 || g_block_stride % 8 || da_stride % 8 ||
      dg_stride % 8 || dg_block_stride % 8 || cvb_misaligned({dy, a, g, da, dg}))
    return -1;
  if (rows <= 0) return 0;
  siggate_bwd_kernel<<<ew_grid(rows * (C / 8)), EW_THREADS, 0, ST(stream)>>>(
      BF(dy), BF(a), BF(g), BFM(da), BFM(dg), rows, C, a_stride, g_stride, g_block, g_block_stride, da_stride,
      dg_stride, dg_block_stride);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_conv1d_silu_fwd(const void* x, const void* w, void* y, long long B, int S, int C, int KW,
                                   long long x_stride, void* stream) {
  if (C % 8 || x_stride % 8 || cvb_misaligned({x, y})) return -1;
  if (B <= 0) return 0;
  const int seg_len = 32;
  const int segs = (S + seg_len - 1) / seg_len;
  const int grid = ew_grid(B * segs * (C / 8));
  if (KW == 4)
    conv1d_silu_fwd_kernel<4><<<grid, EW_THREADS, 0, ST(stream)>>>(BF(x), BF(w), BFM(y), B, S, C, x_stride, seg_len);
  else if (KW == 3)
    conv1d_silu_fwd_kernel<3><<<grid, EW_THREADS, 0, ST(stream)>>>(BF(x), BF(w), BFM(y), B, S, C, x_stride, seg_len);
  else if (KW == 2)
    conv1d_silu_fwd_kernel<2><<<grid, EW_THREADS, 0, ST(stream)>>>(BF(x), BF(w), BFM(y), B, S, C, x_stride, seg_len);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_conv1d_silu_bwd(const void* dy, const void* x, const void* w, void* dx, float* dw, long long B,
                                   int S, int C, int KW, long long x_stride, long long dx_stride, void* stream) {
  if (C % 8 || x_stride % 8 || dx_stride % 8 || cvb_misaligned({dy, x, dx})) return -1;
  if (B <= 0) return 0;
  // enough segments to fill the machine, long enough to amortise the atomics
  int seg_len = 64;
  const int segs = (S + seg_len - 1) / seg_len;
  const int grid = ew_grid(B * segs * (C / CB));
  if (KW == 4)
    conv1d_silu_bwd_kernel<4><<<grid, EW_THREADS, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), BFM(dx), dw, B, S, C,
                                                                  x_stride, seg_len, dx_stride);
  else if (KW == 3)
    conv1d_silu_bwd_kernel<3><<<grid, EW_THREADS, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), BFM(dx), dw, B, S, C,
                                                                  x_stride, seg_len, dx_stride);
  else if (KW == 2)
    conv1d_silu_bwd_kernel<2><<<grid, EW_THREADS, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), BFM(dx), dw, B, S, C,
                                                                  x_stride, seg_len, dx_stride);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int H,
                                 long long vocab_lo, long long vocab_hi, void* stream) {
  if (H % 8 || cvb_misaligned({table, out})) return -1;
  if (tokens <= 0) return 0;
  embedding_fwd_kernel<<<ew_grid(tokens * (H / 8)), EW_THREADS, 0, ST(stream)>>>(ids, BF(table), BFM(out), tokens,
                                                                               H, vocab_lo, vocab_hi);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_embedding_bwd(const long long* ids, const void* dout, float* dtable, long long tokens, int H,
                                 long long vocab_lo, long long vocab_hi, void* stream) {
  if (H % 8 || cvb_misaligned({dout, dtable})) return -1;
  if (tokens <= 0) return 0;
  embedding_bwd_kernel<<<ew_grid(tokens * (H / 8)), EW_THREADS, 0, ST(stream)>>>(ids, BF(dout), dtable, tokens, H,
                                                                               vocab_lo, vocab_hi);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<ew_grid(n / 8 + 1), EW_THREADS, 0, ST(stream)>>>(src, BFM(dst), n, scale);
  return static_cast<int>(cudaGetLastError());
}
