// One-token decode kernels for cached generation (rollout): attention of the new token over the K / V cache, and
// the single-step Gated-DeltaNet state update.  Both read the current sequence length / nothing shape-dependent
// from DEVICE memory, so one captured CUDA graph serves every decode step.
//
// The reference has no cached decode at all: its rollout worker re-runs the whole forward over prompt + prefix
// for every new token (src/rollout/policy_worker.cc:99-102); the math of one step is the reference's attention
// (src/model/qwen3_5_text.cc:1036-1082) and scan step (:247-258) applied to the last position.
#include "ptx.cuh"

namespace cvb {

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;

// ---------------------------------------------------------------------------------------------------
// decode attention: grid = (B, Hkv); the CTA appends k_new / v_new of (b, kvh) to the cache at position len-1 and
// attends the G = Hq / Hkv query heads of this group to keys 0 .. len-1.  Warp w handles keys w, w + 8, ...;
// lane l holds D / 32 consecutive dims; online softmax per warp and head, merged across warps at the end.
//   q      [B, Hq, D]  bf16 (row stride q_stride between tokens, heads D apart within the row: head h at h * q_hs)
//   kcache [B, Lmax, Hkv, D], vcache same (bf16, contiguous)
//   out    [B, Hq, D]  bf16 contiguous
// ---------------------------------------------------------------------------------------------------
template <int D, int G>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, long long q_hs,
                        const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                        long long kv_stride, __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                        __nv_bfloat16* __restrict__ out, const int* __restrict__ len_ptr, int Lmax, int Hq, int Hkv,
                        float scale, int* status) {
  constexpr int E = D / 32;  // dims per lane (4 or 8)
  const int b = blockIdx.x, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int len = *len_ptr;
  if (len < 1 || len > Lmax) {  // a length outside the cache: report it and attend to what exists
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, ERR_BAD_ARG);
    len = len < 1 ? 1 : Lmax;
  }
  const long long cache_row = static_cast<long long>(Hkv) * D;
  __nv_bfloat16* kc = kcache + (static_cast<long long>(b) * Lmax) * cache_row + static_cast<long long>(kvh) * D;
  __nv_bfloat16* vc = vcache + (static_cast<long long>(b) * Lmax) * cache_row + static_cast<long long>(kvh) * D;
  // append the new token's key / value (one warp does it; everyone waits)
  if (warp == 0) {
    const __nv_bfloat16* kn = k_new + static_cast<long long>(b) * kv_stride + static_cast<long long>(kvh) * D;
    const __nv_bfloat16* vn = v_new + static_cast<long long>(b) * kv_stride + static_cast<long long>(kvh) * D;
    for (int e = 0; e < E; ++e) {
      kc[static_cast<long long>(len - 1) * cache_row + lane * E + e] = kn[lane * E + e];
      vc[static_cast<long long>(len - 1) * cache_row + lane * E + e] = vn[lane * E + e];
    }
  }
  __syncthreads();

  float qv[G][E];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + static_cast<long long>(b) * q_stride + static_cast<long long>(kvh * G + g) * q_hs;
#pragma unroll
    for (int e = 0; e < E; ++e) qv[g][e] = __bfloat162float(qp[lane * E + e]) * scale;
  }
  float m[G], l[G], acc[G][E];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
  }
  for (int j = warp; j < len; j += DEC_WARPS) {
    float kk[E], vv[E];
    const __nv_bfloat16* kp = kc + static_cast<long long>(j) * cache_row + lane * E;
    const __nv_bfloat16* vp = vc + static_cast<long long>(j) * cache_row + lane * E;
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kp + e));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vp + e));
      kk[e] = a.x;
      kk[e + 1] = a.y;
      vv[e] = c.x;
      vv[e + 1] = c.y;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) s += qv[g][e] * kk[e];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m[g], s);
      const float corr = __expf(m[g] - mn);
      const float p = __expf(s - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[g][e] = acc[g][e] * corr + p * vv[e];
      m[g] = mn;
    }
  }
  // merge the warps: shared memory holds (m, l) per warp and head, then the rescaled accumulators
  __shared__ float sm_m[DEC_WARPS][G], sm_l[DEC_WARPS][G];
  __shared__ float sm_acc[DEC_WARPS][G][D];
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      sm_m[warp][g] = m[g];
      sm_l[warp][g] = l[g];
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < E; ++e) sm_acc[warp][g][lane * E + e] = acc[g][e];
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += DEC_THREADS) {
    const int g = idx / D, d = idx - g * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, sm_m[w][g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mx);
      num += sm_acc[w][g][d] * c;
      den += sm_l[w][g] * c;
    }
    out[(static_cast<long long>(b) * Hq + kvh * G + g) * D + d] = __float2bfloat16_rn(num / den);
  }
}

// ---------------------------------------------------------------------------------------------------
// Gated-DeltaNet single step, with the depthwise causal convolution in front of it: grid = (B, Hv), 128
// threads; thread j owns channel j of this head's q, k and v and column j (value dim) of the state
// S [dk = 128, dv = 128] fp32 of (b, head), kept in registers for one read and one write:
//   x   = silu(sum_t w[c, t] * window[t, c])      window = the last KW - 1 raw rows (ring cache) + the new row
//   q^  = l2norm(q) / sqrt(dk), k^ = l2norm(k), beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias)
//   S *= e^g;  kv = S^T k^;  delta = (v - kv) beta;  S += k^ (x) delta;  o = S^T q^
// `proj` rows are [q heads | k heads | v heads | ...] of one token (raw, before the convolution).  The ring cache
// conv_ring [B, KW, C] holds raw rows; the row of token t lives in slot t % KW, so a step only WRITES slot
// (len - 1) % KW - which nobody reads during this step (everyone takes the new row from `proj`) - and reads the
// other KW - 1 slots.  q / k channels are shared by the Hv / Hk value heads of a key head: the first of them
// writes their slot.  len = sequence length including the new token, read from device memory.
// ---------------------------------------------------------------------------------------------------
template <int KW>
__global__ void __launch_bounds__(128)
gdn_decode_step_kernel(const __nv_bfloat16* __restrict__ proj, long long proj_stride, int Hk, int Hv,
                       const __nv_bfloat16* __restrict__ conv_w, __nv_bfloat16* __restrict__ conv_ring,
                       const int* __restrict__ len_ptr, const __nv_bfloat16* __restrict__ bgate,
                       const __nv_bfloat16* __restrict__ agate, long long gate_stride,
                       const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias,
                       float* __restrict__ state, __nv_bfloat16* __restrict__ out) {
  constexpr int DK = 128, DV = 128;
  const int b = blockIdx.x, hv = blockIdx.y, j = threadIdx.x;
  const int rep = Hv / Hk;
  const int hk = hv / rep;
  const int C = 2 * Hk * DK + Hv * DV;
  const int t = *len_ptr - 1;                      // index of the new token
  const __nv_bfloat16* row = proj + static_cast<long long>(b) * proj_stride;
  __nv_bfloat16* ring = conv_ring + static_cast<long long>(b) * KW * C;
  const int ch[3] = {hk * DK + j, Hk * DK + hk * DK + j, 2 * Hk * DK + hv * DV + j};
  float x[3];
#pragma unroll
  for (int s = 0; s < 3; ++s) {
    const int c = ch[s];
    const __nv_bfloat16 fresh = row[c];
    float acc = __bfloat162float(conv_w[static_cast<long long>(c) * KW + (KW - 1)]) * __bfloat162float(fresh);
#pragma unroll
    for (int d = 1; d < KW; ++d) {                // token t - d, weight tap KW - 1 - d (tokens before 0 are zero)
      if (t - d >= 0)
        acc += __bfloat162float(conv_w[static_cast<long long>(c) * KW + (KW - 1 - d)]) *
               __bfloat162float(ring[static_cast<long long>(((t - d) % KW)) * C + c]);
    }
    x[s] = acc / (1.f + __expf(-acc));
    if (s == 2 || hv % rep == 0) ring[static_cast<long long>(t % KW) * C + c] = fresh;
  }
  __shared__ float sq[DK], sk[DK], red[8];
  const float qr = __bfloat162float(__float2bfloat16_rn(x[0]));   // the training path rounds the conv output to bf16
  const float kr = __bfloat162float(__float2bfloat16_rn(x[1]));
  const float vr = __bfloat162float(__float2bfloat16_rn(x[2]));
  // two block-wide sums of squares (q and k) through warp shuffles and shared memory
  float s1 = qr * qr, s2 = kr * kr;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if ((j & 31) == 0) {
    red[j >> 5] = s1;
    red[4 + (j >> 5)] = s2;
  }
  __syncthreads();
  const float qn = red[0] + red[1] + red[2] + red[3], kn = red[4] + red[5] + red[6] + red[7];
  sq[j] = qr * rsqrtf(qn + 1e-6f) * 0.08838834764831845f;  // 1 / sqrt(128)
  sk[j] = kr * rsqrtf(kn + 1e-6f);
  __syncthreads();
  const float beta = 1.f / (1.f + __expf(-__bfloat162float(bgate[static_cast<long long>(b) * gate_stride + hv])));
  const float ax = __bfloat162float(agate[static_cast<long long>(b) * gate_stride + hv]) + __bfloat162float(dt_bias[hv]);
  const float softplus = ax > 20.f ? ax : log1pf(__expf(ax));
  const float decay = __expf(-__expf(__bfloat162float(A_log[hv])) * softplus);
  float* S = state + ((static_cast<long long>(b) * Hv + hv) * DK) * DV + j;
  float col[DK];
  float kv = 0.f;
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    col[i] = S[static_cast<long long>(i) * DV] * decay;
    kv += col[i] * sk[i];
  }
  const float delta = (vr - kv) * beta;
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const float sn = col[i] + sk[i] * delta;
    S[static_cast<long long>(i) * DV] = sn;
    o += sn * sq[i];
  }
  out[(static_cast<long long>(b) * Hv + hv) * DV + j] = __float2bfloat16_rn(o);
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_decode_attention(const void* q, long long q_stride, long long q_head_stride, const void* k_new,
                                    const void* v_new, long long kv_stride, void* kcache, void* vcache, void* out,
                                    const int* len_ptr, int B, int Lmax, int Hq, int Hkv, int D, float scale,
                                    int* status, void* stream) {
  if (!q || !k_new || !v_new || !kcache || !vcache || !out || !len_ptr || B <= 0 || Hkv <= 0 || Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  dim3 grid(B, Hkv);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define CVB_DEC(D_, G_)                                                                                          \
  if (D == D_ && G == G_) {                                                                                      \
    decode_attention_kernel<D_, G_><<<grid, DEC_THREADS, 0, st>>>(                                               \
        static_cast<const __nv_bfloat16*>(q), q_stride, q_head_stride, static_cast<const __nv_bfloat16*>(k_new), \
        static_cast<const __nv_bfloat16*>(v_new), kv_stride, static_cast<__nv_bfloat16*>(kcache),                \
        static_cast<__nv_bfloat16*>(vcache), static_cast<__nv_bfloat16*>(out), len_ptr, Lmax, Hq, Hkv, scale,    \
        status);                                                                                                 \
    return static_cast<int>(cudaGetLastError());                                                                 \
  }
  CVB_DEC(256, 4) CVB_DEC(256, 2) CVB_DEC(256, 1) CVB_DEC(128, 8) CVB_DEC(128, 4) CVB_DEC(128, 2) CVB_DEC(128, 1)
#undef CVB_DEC
  return -2;  // head dim / group size without an instantiation
}

// proj: [B, >= 2*Hk*128 + Hv*128] raw projection rows; conv_w [C, KW] bf16; conv_ring [B, KW, C] bf16 (slot of token
// t is t % KW); bgate / agate: per-head gate inputs with row stride gate_stride; state [B, Hv, 128, 128] fp32.
extern "C" int cvb_gdn_decode_step(const void* proj, long long proj_stride, int Hk, int Hv, const void* conv_w,
                                   void* conv_ring, int KW, const int* len_ptr, const void* bgate, const void* agate,
                                   long long gate_stride, const void* A_log, const void* dt_bias, float* state,
                                   void* out, int B, void* stream) {
  if (!proj || !conv_w || !conv_ring || !len_ptr || !bgate || !agate || !A_log || !dt_bias || !state || !out ||
      B <= 0 || Hk <= 0 || Hv % Hk)
    return -1;
  dim3 grid(B, Hv);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define CVB_GDS(KW_)                                                                                             \
  if (KW == KW_) {                                                                                               \
    gdn_decode_step_kernel<KW_><<<grid, 128, 0, st>>>(                                                           \
        static_cast<const __nv_bfloat16*>(proj), proj_stride, Hk, Hv, static_cast<const __nv_bfloat16*>(conv_w), \
        static_cast<__nv_bfloat16*>(conv_ring), len_ptr, static_cast<const __nv_bfloat16*>(bgate),               \
        static_cast<const __nv_bfloat16*>(agate), gate_stride, static_cast<const __nv_bfloat16*>(A_log),         \
        static_cast<const __nv_bfloat16*>(dt_bias), state, static_cast<__nv_bfloat16*>(out));                    \
    return static_cast<int>(cudaGetLastError());                                                                 \
  }
  CVB_GDS(4) CVB_GDS(3) CVB_GDS(2)
#undef CVB_GDS
  return -2;
}
