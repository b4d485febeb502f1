// Merge of partial attention results across the hops of context-parallel (ring) attention.
//
// Every hop yields, for a block of query rows, an output normalised over the keys of that hop and the log-sum-exp
// of its scores.  Two such pairs combine exactly:
//     lse' = log(exp(lse) + exp(lse_p)),   acc' = acc * exp(lse - lse') + part * exp(lse_p - lse')
// One warp owns one (batch, row, head): it reads the two scalars once and streams the head dimension in 16-byte
// pieces, so a hop's merge is one pass over the fp32 accumulator instead of the seven element-wise passes of the
// same arithmetic written with tensor ops.  The reference merges hops with tensor ops
// (src/distributed/context_parallel.cc:143-260).
#include "ptx.cuh"

namespace cvb {

// acc [B, T, H, D] fp32 and lse [B, H, T] fp32 are the running result; part [B, Tp, H, D] bf16 and
// lse_p [B, H, Tp] fp32 cover rows [row0, row0 + Tp).  first != 0: the rows take the partial result as it is.
__global__ void __launch_bounds__(256)
attn_merge_kernel(float* __restrict__ acc, float* __restrict__ lse, const __nv_bfloat16* __restrict__ part,
                  const float* __restrict__ lse_p, int T, int Tp, int H, int D, int row0, int first, long long items) {
  const long long w = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= items) return;
  const int h = static_cast<int>(w % H);
  const long long bt = w / H;
  const int t = static_cast<int>(bt % Tp);
  const long long b = bt / Tp;
  const long long li = (b * H + h) * T + row0 + t;
  const float lp = lse_p[(b * H + h) * Tp + t];
  float w0 = 0.f, w1 = 1.f, ln = lp;
  if (!first) {
    const float lo = lse[li];
    const float m = fmaxf(lo, lp);
    if (m == -INFINITY) {            // neither side saw a key: keep zeros
      w0 = 0.f; w1 = 0.f; ln = -INFINITY;
    } else {
      const float e0 = __expf(lo - m), e1 = __expf(lp - m);
      ln = m + __logf(e0 + e1);
      w0 = e0 / (e0 + e1);
      w1 = e1 / (e0 + e1);
    }
  }
  if (lane == 0) lse[li] = ln;
  float* a = acc + ((b * T + row0 + t) * H + h) * static_cast<long long>(D);
  const __nv_bfloat16* p = part + ((b * Tp + t) * H + h) * static_cast<long long>(D);
  for (int d = lane * 4; d < D; d += 128) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p + d);
    const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!first) o = *reinterpret_cast<const float4*>(a + d);
    o.x = o.x * w0 + p0.x * w1;
    o.y = o.y * w0 + p0.y * w1;
    o.z = o.z * w0 + p1.x * w1;
    o.w = o.w * w0 + p1.y * w1;
    *reinterpret_cast<float4*>(a + d) = o;
  }
}

}  // namespace cvb

extern "C" int cvb_attn_merge(float* acc, float* lse, const void* part, const float* lse_p, long long B, int T, int Tp,
                              int H, int D, int row0, int first, void* stream) {
  if (B <= 0 || Tp <= 0) return 0;
  if (D % 4 || row0 < 0 || row0 + Tp > T ||
      ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(part)) & 15))
    return -1;
  const long long items = B * Tp * H;
  const long long blocks = (items * 32 + 255) / 256;
  if (blocks >= (1ll << 31)) return -1;
  cvb::attn_merge_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      acc, lse, static_cast<const __nv_bfloat16*>(part), lse_p, T, Tp, H, D, row0, first, items);
  return static_cast<int>(cudaGetLastError());
}
