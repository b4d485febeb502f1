// Flat-shard optimizer kernels: squared-norm reduction, clip-scale, and the
// single-pass FlatAdamW update (grad scale + clip, fp32 moments, decoupled
// weight decay, optional fp32 master copy, bf16 model write, grad zeroing).
//
// Update rule (reference: src/torch/fp32_master_adamw.cc:284-308):
//   m = b1*m + (1-b1)*g ;  v = b2*v + (1-b2)*g*g
//   p = p*(1 - lr*wd) - (lr/(1-b1^t)) * m / (sqrt(v/(1-b2^t)) + eps)
// Clip rule (src/distributed/optimizer_sharding.cc:701-709):
//   scale = max_norm/(norm+1e-6) when norm is finite and > max_norm, else 1.
#include "ptx.cuh"

namespace cvb {

constexpr int OPT_THREADS = 256;

static int opt_grid(long long n_vec) {
  long long b = (n_vec + OPT_THREADS - 1) / OPT_THREADS;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

// out_sq[0] += sum(g^2)  (fp32 accumulate per thread, fp64 across blocks is
// avoided: one float atomic per block keeps the result a plain fp32 tensor
// that NCCL can all-reduce; per-thread partial sums are short)
__global__ void __launch_bounds__(OPT_THREADS)
sumsq_f32_kernel(const float* __restrict__ g, long long n, float scale, float* __restrict__ out_sq) {
  __shared__ float sh[OPT_THREADS / 32];
  float acc = 0.f;
  const long long nv = n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * OPT_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * OPT_THREADS) {
    const float4 v = *reinterpret_cast<const float4*>(g + i * 4);
    acc += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
  }
  if (blockIdx.x == 0)
    for (long long i = nv * 4 + threadIdx.x; i < n; i += OPT_THREADS) acc += g[i] * g[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < OPT_THREADS / 32 ? sh[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) atomicAdd(out_sq, r * scale * scale);
  }
}

// clip[0] = scale, clip[1] = global norm
__global__ void clip_scale_kernel(const float* __restrict__ global_sq, float max_norm, float* __restrict__ clip) {
  if (threadIdx.x == 0) {
    const float norm = sqrtf(global_sq[0]);
    float s = 1.f;
    if (max_norm > 0.f && isfinite(norm) && norm > max_norm) s = max_norm / (norm + 1.0e-6f);
    clip[0] = s;
    clip[1] = norm;
  }
}

struct AdamArgs {
  float* grad;               // fp32 gradient shard (read, optionally zeroed)
  float* master;             // fp32 master shard or nullptr
  __nv_bfloat16* model;      // bf16 model shard (read when no master; always written when non-null)
  float* model_f32;          // fp32 model shard (used instead of `model` for fp32 training)
  float* m;
  float* v;
  const float* clip;         // device scalar multiplied into the gradient (or nullptr)
  long long n;
  float grad_scale;          // static factor (e.g. 1/dp for mean reduction)
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int zero_grad;
};

__global__ void __launch_bounds__(OPT_THREADS)
flat_adamw_kernel(const AdamArgs a) {
  const float cs = (a.clip ? a.clip[0] : 1.f) * a.grad_scale;
  const float step_size = a.lr / a.bc1;
  const float decay = 1.f - a.lr * a.weight_decay;
  const float inv_bc2 = 1.f / a.bc2;
  const long long nv = a.n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * OPT_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * OPT_THREADS) {
    float4 g = *reinterpret_cast<const float4*>(a.grad + i * 4);
    float4 m = *reinterpret_cast<const float4*>(a.m + i * 4);
    float4 v = *reinterpret_cast<const float4*>(a.v + i * 4);
    float p[4];
    if (a.master) {
      const float4 pm = *reinterpret_cast<const float4*>(a.master + i * 4);
      p[0] = pm.x, p[1] = pm.y, p[2] = pm.z, p[3] = pm.w;
    } else if (a.model_f32) {
      const float4 pm = *reinterpret_cast<const float4*>(a.model_f32 + i * 4);
      p[0] = pm.x, p[1] = pm.y, p[2] = pm.z, p[3] = pm.w;
    } else {
      const uint2 pb = *reinterpret_cast<const uint2*>(a.model + i * 4);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pb);
      const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
      p[0] = f0.x, p[1] = f0.y, p[2] = f1.x, p[3] = f1.y;
    }
    float gg[4] = {g.x * cs, g.y * cs, g.z * cs, g.w * cs};
    float mm[4] = {m.x, m.y, m.z, m.w};
    float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gg[j];
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gg[j] * gg[j];
      p[j] = p[j] * decay;
      p[j] -= step_size * mm[j] / (sqrtf(vv[j] * inv_bc2) + a.eps);
    }
    *reinterpret_cast<float4*>(a.m + i * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(a.v + i * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (a.master) *reinterpret_cast<float4*>(a.master + i * 4) = make_float4(p[0], p[1], p[2], p[3]);
    if (a.model_f32) *reinterpret_cast<float4*>(a.model_f32 + i * 4) = make_float4(p[0], p[1], p[2], p[3]);
    if (a.model) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      *reinterpret_cast<uint2*>(a.model + i * 4) = o;
    }
    if (a.zero_grad) *reinterpret_cast<float4*>(a.grad + i * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < a.n; i += OPT_THREADS) {
      const float g = a.grad[i] * cs;
      float p = a.master ? a.master[i] : (a.model_f32 ? a.model_f32[i] : __bfloat162float(a.model[i]));
      const float m = a.beta1 * a.m[i] + (1.f - a.beta1) * g;
      const float v = a.beta2 * a.v[i] + (1.f - a.beta2) * g * g;
      p = p * decay - step_size * m / (sqrtf(v * inv_bc2) + a.eps);
      a.m[i] = m;
      a.v[i] = v;
      if (a.master) a.master[i] = p;
      if (a.model_f32) a.model_f32[i] = p;
      if (a.model) a.model[i] = __float2bfloat16_rn(p);
      if (a.zero_grad) a.grad[i] = 0.f;
    }
  }
}

}  // namespace cvb

using namespace cvb;
#define ST(s) static_cast<cudaStream_t>(s)

extern "C" int cvb_sumsq_f32(const float* g, long long n, float scale, float* out_sq, void* stream) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) & 15) return -1;
  sumsq_f32_kernel<<<opt_grid(n / 4 + 1), OPT_THREADS, 0, ST(stream)>>>(g, n, scale, out_sq);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_clip_scale(const float* global_sq, float max_norm, float* clip, void* stream) {
  clip_scale_kernel<<<1, 32, 0, ST(stream)>>>(global_sq, max_norm, clip);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_flat_adamw(float* grad, float* master, void* model_bf16, float* model_f32, float* m, float* v,
                              const float* clip, long long n, float grad_scale, float lr, float beta1, float beta2,
                              float eps, float weight_decay, long long step, int zero_grad, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15)
    return -1;
  if ((master && (reinterpret_cast<uintptr_t>(master) & 15)) || (model_bf16 && (reinterpret_cast<uintptr_t>(model_bf16) & 7)) ||
      (model_f32 && (reinterpret_cast<uintptr_t>(model_f32) & 15)))
    return -1;
  AdamArgs a;
  a.grad = grad; a.master = master; a.model = static_cast<__nv_bfloat16*>(model_bf16); a.model_f32 = model_f32;
  a.m = m; a.v = v; a.clip = clip; a.n = n; a.grad_scale = grad_scale; a.lr = lr; a.beta1 = beta1; a.beta2 = beta2;
  a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = static_cast<float>(1.0 - pow(static_cast<double>(beta1), static_cast<double>(step)));
  a.bc2 = static_cast<float>(1.0 - pow(static_cast<double>(beta2), static_cast<double>(step)));
  a.zero_grad = zero_grad;
  flat_adamw_kernel<<<opt_grid(n / 4 + 1), OPT_THREADS, 0, ST(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}
