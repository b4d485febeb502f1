// Fused MoE router: top-k selection + softmax over the router logits, forward and backward.
//
// One warp per token.  Forward reads the token's E logits (fp32, produced by the tcgen05 GEMM with the
// fp32 epilogue), picks the k largest by k rounds of warp arg-max, and writes the expert ids and the
// routing weights: softmax over the selected logits (norm_topk_prob) or the selected entries of the
// softmax over all experts.  Backward turns d(weights) into d(logits) with the softmax Jacobian in the
// same one-warp-per-token layout; the dense [T, E] gradient then feeds the router's two small GEMMs.
//
// The reference composes matmul / topk / softmax / gather ATen ops (src/model/qwen3_5_text.cc:713-760).
#include "ptx.cuh"

namespace cvb {

constexpr int RT_THREADS = 256;
constexpr int RT_MAX_PER_LANE = 8;  // E <= 256

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) v = ov, i = oi;
  }
}

// logits [T, E] fp32 -> idx [T, k] int64, w [T, k] fp32
__global__ void __launch_bounds__(RT_THREADS)
router_topk_fwd_kernel(const float* __restrict__ logits, long long T, int E, int k, int norm_topk,
                       long long* __restrict__ idx, float* __restrict__ w) {
  const long long tok = (static_cast<long long>(blockIdx.x) * RT_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  const int per = (E + 31) / 32;
  float v[RT_MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    v[j] = (j < per && e < E) ? logits[tok * E + e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float denom_all = 0.f;
  if (!norm_topk) {
#pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) denom_all += (v[j] > -INFINITY) ? __expf(v[j] - mx) : 0.f;
    denom_all = warp_sum(denom_all);
  }
  float sel_val = 0.f;   // lane r keeps the r-th selected logit
  int sel_idx = 0;
  float denom_k = 0.f;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j)
      if (v[j] > bv) bv = v[j], bi = j * 32 + lane;
    warp_argmax(bv, bi);
    if ((bi & 31) == lane) {   // remove the winner from its owner's candidates
#pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j)
        if (j == (bi >> 5)) v[j] = -INFINITY;
    }
    if (lane == r) sel_val = bv, sel_idx = bi;
    denom_k += __expf(bv - mx);                       // first winner is the global max: exponents <= 0
  }
  if (lane < k) {
    const float p = __expf(sel_val - mx) / (norm_topk ? denom_k : denom_all);
    idx[tok * k + lane] = sel_idx;
    w[tok * k + lane] = p;
  }
}

// dlogits [T, E] fp32 from dw [T, k]
__global__ void __launch_bounds__(RT_THREADS)
router_topk_bwd_kernel(const float* __restrict__ logits, const long long* __restrict__ idx,
                       const float* __restrict__ w, const float* __restrict__ dw, long long T, int E, int k,
                       int norm_topk, float* __restrict__ dlogits) {
  const long long tok = (static_cast<long long>(blockIdx.x) * RT_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  const float wi = lane < k ? w[tok * k + lane] : 0.f;
  const float di = lane < k ? dw[tok * k + lane] : 0.f;
  const int ei = lane < k ? static_cast<int>(idx[tok * k + lane]) : -1;
  const float dot = warp_sum(wi * di);   // sum_i w_i dw_i
  float mx = -INFINITY, denom = 1.f;
  const int per = (E + 31) / 32;
  if (!norm_topk) {
    for (int j = 0; j < per; ++j) {
      const int e = j * 32 + lane;
      if (e < E) mx = fmaxf(mx, logits[tok * E + e]);
    }
    mx = warp_max(mx);
    float s = 0.f;
    for (int j = 0; j < per; ++j) {
      const int e = j * 32 + lane;
      if (e < E) s += __expf(logits[tok * E + e] - mx);
    }
    denom = warp_sum(s);
  }
  for (int j = 0; j < per; ++j) {
    const int e = j * 32 + lane;
    if (e >= E) continue;
    float g = norm_topk ? 0.f : -(__expf(logits[tok * E + e] - mx) / denom) * dot;
    dlogits[tok * E + e] = g;
  }
  __syncwarp();
  if (lane < k) {   // selected experts: w_i (dw_i - dot) replaces / adds to the dense term
    const float g = wi * (di - dot);
    if (norm_topk) dlogits[tok * E + ei] = g;
    else dlogits[tok * E + ei] = wi * di - wi * dot;
  }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_router_topk_fwd(const float* logits, long long T, int E, int k, int norm_topk, long long* idx,
                                   float* w, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 32 * RT_MAX_PER_LANE || k <= 0 || k > 32 || k > E) return -1;
  const long long blocks = (T * 32 + RT_THREADS - 1) / RT_THREADS;
  router_topk_fwd_kernel<<<static_cast<unsigned>(blocks), RT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, T, E, k, norm_topk, idx, w);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_router_topk_bwd(const float* logits, const long long* idx, const float* w, const float* dw,
                                   long long T, int E, int k, int norm_topk, float* dlogits, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 32 * RT_MAX_PER_LANE || k <= 0 || k > 32 || k > E) return -1;
  const long long blocks = (T * 32 + RT_THREADS - 1) / RT_THREADS;
  router_topk_bwd_kernel<<<static_cast<unsigned>(blocks), RT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, idx, w, dw, T, E, k, norm_topk, dlogits);
  return static_cast<int>(cudaGetLastError());
}
