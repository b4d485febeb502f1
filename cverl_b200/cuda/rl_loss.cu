// RL loss / advantage kernels on device fp32 tensors [rows, cols]:
// masked sum / mean / whiten, KL penalties (k1, abs, k2, k3) with backward,
// GAE, GRPO outcome advantage, and the PPO clipped (dual-clip) policy loss
// fused with its gradient w.r.t. log_prob and an optional KL term.
//
// Semantics follow the public RL-math contract of the reference
// (src/torch/core_algos_torch.cc:9-193): eps 1e-8 in masked_mean, unbiased
// variance in whiten, ratio = exp(clamp(lp - old, +-20)), dual clip applied
// only where the advantage is negative, three loss aggregation modes.
//
// Reductions accumulate in fp64 scratch words that the caller provides
// (`ws`, zeroed by the launcher with a memset node on the same stream).
#include "ptx.cuh"

namespace cvb {

constexpr int RL_THREADS = 256;
constexpr double kEps = 1.0e-8;

__device__ __forceinline__ double block_sum_d(double v, double* sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  double r = 0.0;
  if (threadIdx.x < (blockDim.x >> 5)) r = sh[threadIdx.x];
  if (w == 0) {
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;  // valid in thread 0
}

static int rl_grid(long long n) {
  long long b = (n + RL_THREADS - 1) / RL_THREADS;
  if (b > 148 * 4) b = 148 * 4;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

// ws[0] += sum(v*m), ws[1] += sum(m)
__global__ void __launch_bounds__(RL_THREADS)
masked_sums_kernel(const float* __restrict__ v, const float* __restrict__ m, long long n, double* ws) {
  __shared__ double sh[RL_THREADS / 32];
  double a = 0.0, b = 0.0;
  for (long long i = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * RL_THREADS) {
    a += static_cast<double>(v[i]) * m[i];
    b += m[i];
  }
  a = block_sum_d(a, sh);
  b = block_sum_d(b, sh);
  if (threadIdx.x == 0) {
    atomicAdd(&ws[0], a);
    atomicAdd(&ws[1], b);
  }
}
// ws[2] += sum((v-mean)^2 * m) with mean = ws[0]/(ws[1]+eps)
__global__ void __launch_bounds__(RL_THREADS)
masked_var_kernel(const float* __restrict__ v, const float* __restrict__ m, long long n, double* ws) {
  __shared__ double sh[RL_THREADS / 32];
  const float mean = static_cast<float>(ws[0] / (ws[1] + kEps));
  double a = 0.0;
  for (long long i = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * RL_THREADS) {
    const float c = v[i] - mean;
    a += static_cast<double>(c * c) * m[i];
  }
  a = block_sum_d(a, sh);
  if (threadIdx.x == 0) atomicAdd(&ws[2], a);
}
__global__ void __launch_bounds__(RL_THREADS)
whiten_apply_kernel(const float* __restrict__ v, float* __restrict__ out, long long n, const double* ws,
                    int shift_mean) {
  const double msum = ws[1];
  const float mean = static_cast<float>(ws[0] / (msum + kEps));
  float var = static_cast<float>(ws[2] / (msum + kEps));
  var = var * static_cast<float>(msum) / (static_cast<float>(msum) - 1.0f);
  const float rs = rsqrtf(var + static_cast<float>(kEps));
  for (long long i = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * RL_THREADS) {
    float w = (v[i] - mean) * rs;
    if (!shift_mean) w += mean;
    out[i] = w;
  }
}
__global__ void finalize_sum_mean_kernel(const double* ws, float* out, int mean) {
  if (threadIdx.x == 0) out[0] = static_cast<float>(mean ? ws[0] / (ws[1] + kEps) : ws[0]);
}

// ----------------------------- KL penalty ----------------------------------
__device__ __forceinline__ float kl_value(float lp, float ref, int kind) {
  const float d = lp - ref;
  if (kind == 0) return d;
  if (kind == 1) return fabsf(d);
  if (kind == 2) return 0.5f * d * d;
  const float k = fminf(fmaxf(ref - lp, -20.f), 20.f);
  return fminf(fmaxf(expf(k) - k - 1.f, -10.f), 10.f);
}
__device__ __forceinline__ float kl_grad(float lp, float ref, int kind) {
  const float d = lp - ref;
  if (kind == 0) return 1.f;
  if (kind == 1) return d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
  if (kind == 2) return d;
  const float kraw = ref - lp;
  if (kraw < -20.f || kraw > 20.f) return 0.f;
  const float e = expf(kraw);
  const float val = e - kraw - 1.f;
  if (val < -10.f || val > 10.f) return 0.f;
  return -(e - 1.f);
}
__global__ void __launch_bounds__(RL_THREADS)
kl_kernel(const float* __restrict__ lp, const float* __restrict__ ref, float* __restrict__ out, long long n,
          int kind, int backward) {
  for (long long i = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * RL_THREADS)
    out[i] = backward ? kl_grad(lp[i], ref[i], kind) : kl_value(lp[i], ref[i], kind);
}

// -------------------------------- GAE --------------------------------------
// one thread per row walks the columns backwards (masked carries)
__global__ void __launch_bounds__(RL_THREADS)
gae_kernel(const float* __restrict__ rew, const float* __restrict__ val, const float* __restrict__ mask,
           float* __restrict__ adv, float* __restrict__ ret, long long rows, int cols, float gamma, float lam) {
  const long long r = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x;
  if (r >= rows) return;
  float next_value = 0.f, last = 0.f;
  for (int c = cols - 1; c >= 0; --c) {
    const long long i = r * cols + c;
    const float v = val[i], m = mask[i];
    const float delta = rew[i] + gamma * next_value - v;
    const float cand = delta + gamma * lam * last;
    next_value = v * m + (1.f - m) * next_value;
    last = cand * m + (1.f - m) * last;
    adv[i] = last;
    if (ret) ret[i] = last + v;
  }
}

// -------------------------------- GRPO -------------------------------------
// scores[r] = sum_c rewards[r,c]
__global__ void __launch_bounds__(RL_THREADS)
row_sum_kernel(const float* __restrict__ x, float* __restrict__ out, long long rows, int cols) {
  const long long warp = (static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  float s = 0.f;
  for (int c = lane; c < cols; c += 32) s += x[warp * cols + c];
  s = warp_sum(s);
  if (lane == 0) out[warp] = s;
}
// one warp per row compares its group id against every row (B is ~1e3)
__global__ void __launch_bounds__(RL_THREADS)
grpo_scalar_kernel(const float* __restrict__ scores, const long long* __restrict__ gid, float* __restrict__ scal,
                   long long rows, float eps, int norm_by_std) {
  const long long warp = (static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const long long g = gid[warp];
  float sum = 0.f, cnt = 0.f;
  for (long long j = lane; j < rows; j += 32)
    if (gid[j] == g) sum += scores[j], cnt += 1.f;
  sum = warp_sum(sum);
  cnt = warp_sum(cnt);
  const float mean = cnt > 1.f ? sum / fmaxf(cnt, 1.f) : 0.f;
  float s = scores[warp] - mean;
  if (norm_by_std) {
    float sq = 0.f;
    for (long long j = lane; j < rows; j += 32)
      if (gid[j] == g) {
        const float d = scores[j] - mean;
        sq += d * d;
      }
    sq = warp_sum(sq);
    const float sd = cnt > 1.f ? sqrtf(sq / fmaxf(cnt - 1.f, 1.f)) : 1.f;
    s = s / (sd + eps);
  }
  if (lane == 0) scal[warp] = s;
}
__global__ void __launch_bounds__(RL_THREADS)
grpo_broadcast_kernel(const float* __restrict__ scal, const float* __restrict__ mask, float* __restrict__ adv,
                      float* __restrict__ ret, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * RL_THREADS) {
    const float a = scal[i / cols] * mask[i];
    adv[i] = a;
    if (ret) ret[i] = a;
  }
}

// ------------------------------- PPO loss ----------------------------------
// Pass 1: per-row token count, total token count and number of non-empty rows.
//   ws[3] += sum(mask); ws[4] += #rows with count > 0; rowcnt[r] = count
__global__ void __launch_bounds__(RL_THREADS)
ppo_mask_stats_kernel(const float* __restrict__ mask, float* __restrict__ rowcnt, long long rows, int cols,
                      double* ws) {
  const long long warp = (static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  float s = 0.f;
  for (int c = lane; c < cols; c += 32) s += mask[warp * cols + c];
  s = warp_sum(s);
  if (lane == 0) {
    rowcnt[warp] = s;
    atomicAdd(&ws[3], static_cast<double>(s));
    if (s > 0.f) atomicAdd(&ws[4], 1.0);
  }
}

struct PpoArgs {
  const float* old_lp;
  const float* lp;
  const float* adv;
  const float* mask;
  const float* ref_lp;  // optional
  const float* rowcnt;
  float* grad;  // optional: d(total loss)/d lp
  long long rows;
  int cols;
  float clip_low, clip_high, clip_c;
  int agg_mode;
  float kl_coef;
  int kl_kind;
  float loss_scale;  // multiplies the gradient and nothing else
  double* ws;        // ws[3]=sum mask, ws[4]=seq count, ws[5..9] metric sums
};

// Pass 2: token losses, gradient and metric sums.
//   ws[5] += pg loss (aggregated), ws[6] += clipfrac num, ws[7] += -delta*mask, ws[8] += lower clip num,
//   ws[9] += kl*mask
__global__ void __launch_bounds__(RL_THREADS)
ppo_loss_kernel(const PpoArgs a) {
  __shared__ double sh[RL_THREADS / 32];
  const double msum = a.ws[3];
  const double nseq = a.ws[4];
  const long long n = a.rows * a.cols;
  double s_loss = 0, s_clip = 0, s_kl = 0, s_low = 0, s_ref = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * RL_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * RL_THREADS) {
    const float m = a.mask[i];
    const float A = a.adv[i];
    const float draw = a.lp[i] - a.old_lp[i];
    const float d = fminf(fmaxf(draw, -20.f), 20.f);
    const float dpass = (draw >= -20.f && draw <= 20.f) ? 1.f : 0.f;
    const float ratio = expf(d);
    const float lo = 1.f - a.clip_low, hi = 1.f + a.clip_high;
    const float rc = fminf(fmaxf(ratio, lo), hi);
    const float cpass = (ratio >= lo && ratio <= hi) ? 1.f : 0.f;
    const float l1 = -A * ratio, l2 = -A * rc, l3 = -A * a.clip_c;
    const float g1 = -A * ratio * dpass, g2 = -A * ratio * dpass * cpass;
    float mx, gmx;
    if (l1 > l2) mx = l1, gmx = g1;
    else if (l2 > l1) mx = l2, gmx = g2;
    else mx = l1, gmx = 0.5f * (g1 + g2);
    float loss = mx, g = gmx;
    if (A < 0.f) {
      if (l3 < mx) loss = l3, g = 0.f;
      else if (l3 == mx) g = 0.5f * gmx;
    }
    // aggregation weight of this token
    float wgt;
    if (a.agg_mode == 0) {
      wgt = m / static_cast<float>(msum + kEps);
    } else {
      const float cnt = a.rowcnt[i / a.cols];
      const float seqm = cnt > 0.f ? 1.f : 0.f;
      wgt = m * seqm / static_cast<float>(nseq + kEps);
      if (a.agg_mode == 2) wgt /= (cnt + static_cast<float>(kEps));
    }
    s_loss += static_cast<double>(loss) * wgt;
    s_clip += (l2 > l1 ? 1.0 : 0.0) * m;
    s_kl += static_cast<double>(-d) * m;
    s_low += ((mx > l3 && A < 0.f) ? 1.0 : 0.0) * m;
    float gtot = g * wgt;
    if (a.ref_lp) {
      const float kv = kl_value(a.lp[i], a.ref_lp[i], a.kl_kind);
      s_ref += static_cast<double>(kv) * m;
      // KL term is aggregated as a token mean with the same denominator
      gtot += a.kl_coef * kl_grad(a.lp[i], a.ref_lp[i], a.kl_kind) * m / static_cast<float>(msum + kEps);
    }
    if (a.grad) a.grad[i] = gtot * a.loss_scale;
  }
  s_loss = block_sum_d(s_loss, sh);
  s_clip = block_sum_d(s_clip, sh);
  s_kl = block_sum_d(s_kl, sh);
  s_low = block_sum_d(s_low, sh);
  s_ref = block_sum_d(s_ref, sh);
  if (threadIdx.x == 0) {
    atomicAdd(&a.ws[5], s_loss);
    atomicAdd(&a.ws[6], s_clip);
    atomicAdd(&a.ws[7], s_kl);
    atomicAdd(&a.ws[8], s_low);
    atomicAdd(&a.ws[9], s_ref);
  }
}
// out[0..4] = pg_loss, clipfrac, ppo_kl, clipfrac_lower, kl_mean ; out[5] = token count
__global__ void ppo_finalize_kernel(const double* ws, float* out) {
  if (threadIdx.x == 0) {
    const double den = ws[3] + kEps;
    out[0] = static_cast<float>(ws[5]);
    out[1] = static_cast<float>(ws[6] / den);
    out[2] = static_cast<float>(ws[7] / den);
    out[3] = static_cast<float>(ws[8] / den);
    out[4] = static_cast<float>(ws[9] / den);
    out[5] = static_cast<float>(ws[3]);
  }
}

}  // namespace cvb

using namespace cvb;
#define ST(s) static_cast<cudaStream_t>(s)

// Scratch: `ws` points at >= 16 doubles of device memory owned by the caller.
extern "C" int cvb_rl_workspace_doubles() { return 16; }

extern "C" int cvb_masked_sum_mean(const float* v, const float* m, long long n, int mean, float* out, double* ws,
                                   void* stream) {
  cudaMemsetAsync(ws, 0, 16 * sizeof(double), ST(stream));
  masked_sums_kernel<<<rl_grid(n), RL_THREADS, 0, ST(stream)>>>(v, m, n, ws);
  finalize_sum_mean_kernel<<<1, 32, 0, ST(stream)>>>(ws, out, mean);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_masked_whiten(const float* v, const float* m, long long n, int shift_mean, float* out,
                                 double* ws, void* stream) {
  cudaMemsetAsync(ws, 0, 16 * sizeof(double), ST(stream));
  masked_sums_kernel<<<rl_grid(n), RL_THREADS, 0, ST(stream)>>>(v, m, n, ws);
  masked_var_kernel<<<rl_grid(n), RL_THREADS, 0, ST(stream)>>>(v, m, n, ws);
  whiten_apply_kernel<<<rl_grid(n), RL_THREADS, 0, ST(stream)>>>(v, out, n, ws, shift_mean);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_kl_penalty(const float* lp, const float* ref, float* out, long long n, int kind, int backward,
                              void* stream) {
  kl_kernel<<<rl_grid(n), RL_THREADS, 0, ST(stream)>>>(lp, ref, out, n, kind, backward);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_gae(const float* rew, const float* val, const float* mask, float* adv_raw, float* adv_out,
                       float* ret, long long rows, int cols, float gamma, float lam, double* ws, void* stream) {
  gae_kernel<<<static_cast<int>((rows + RL_THREADS - 1) / RL_THREADS), RL_THREADS, 0, ST(stream)>>>(
      rew, val, mask, adv_raw, ret, rows, cols, gamma, lam);
  return cvb_masked_whiten(adv_raw, mask, rows * cols, 1, adv_out, ws, stream);
}
extern "C" int cvb_grpo_advantage(const float* rewards, const float* mask, const long long* gid, float eps,
                                  int norm_by_std, float* adv, float* ret, float* row_scratch, long long rows,
                                  int cols, void* stream) {
  // row_scratch: 2*rows floats
  const int warps_grid = static_cast<int>((rows * 32 + RL_THREADS - 1) / RL_THREADS);
  row_sum_kernel<<<warps_grid, RL_THREADS, 0, ST(stream)>>>(rewards, row_scratch, rows, cols);
  grpo_scalar_kernel<<<warps_grid, RL_THREADS, 0, ST(stream)>>>(row_scratch, gid, row_scratch + rows, rows, eps,
                                                               norm_by_std);
  grpo_broadcast_kernel<<<rl_grid(rows * cols), RL_THREADS, 0, ST(stream)>>>(row_scratch + rows, mask, adv, ret,
                                                                            rows, cols);
  return static_cast<int>(cudaGetLastError());
}
// metrics_out: 6 floats.  grad may be null.  ref_lp may be null.  rowcnt: rows floats of scratch.
extern "C" int cvb_ppo_loss(const float* old_lp, const float* lp, const float* adv, const float* mask,
                            const float* ref_lp, float* grad, float* metrics_out, float* rowcnt, long long rows,
                            int cols, float clip, float clip_low, float clip_high, float clip_c, int agg_mode,
                            float kl_coef, int kl_kind, float loss_scale, double* ws, void* stream) {
  if (!(clip_c > 1.0f)) return -1;
  if (clip_low < 0.f) clip_low = clip;
  if (clip_high < 0.f) clip_high = clip;
  cudaMemsetAsync(ws, 0, 16 * sizeof(double), ST(stream));
  const int warps_grid = static_cast<int>((rows * 32 + RL_THREADS - 1) / RL_THREADS);
  ppo_mask_stats_kernel<<<warps_grid, RL_THREADS, 0, ST(stream)>>>(mask, rowcnt, rows, cols, ws);
  PpoArgs a;
  a.old_lp = old_lp; a.lp = lp; a.adv = adv; a.mask = mask; a.ref_lp = ref_lp; a.rowcnt = rowcnt; a.grad = grad;
  a.rows = rows; a.cols = cols; a.clip_low = clip_low; a.clip_high = clip_high; a.clip_c = clip_c;
  a.agg_mode = agg_mode; a.kl_coef = kl_coef; a.kl_kind = kl_kind; a.loss_scale = loss_scale; a.ws = ws;
  ppo_loss_kernel<<<rl_grid(rows * cols), RL_THREADS, 0, ST(stream)>>>(a);
  ppo_finalize_kernel<<<1, 32, 0, ST(stream)>>>(ws, metrics_out);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------- GRPO advantage without allocation -------------------
// Same three kernels as cvb_grpo_advantage; the 2*rows floats of per-row scratch (row scores,
// then per-row scalars) come from a fixed array in this library's device image, so neither the
// caller nor this function allocates.  See rl_no_alloc.h for who needs that and for the rules.
#include <cstdio>
#include <mutex>

#include "rl_no_alloc.h"

namespace cvb {
// 2 * CVB_GRPO_STATIC_MAX_ROWS floats = 128 KB, one instance per device that loads this module.
static __device__ __align__(256) float g_grpo_static_scratch[2 * CVB_GRPO_STATIC_MAX_ROWS];

constexpr int kMaxDevices = 64;
static float* g_grpo_scratch_addr[kMaxDevices] = {};  // per-device address of the array, looked up once
static std::mutex g_grpo_scratch_mutex;

// Device address of the scratch array on the CURRENT device.  The look-up runs once per device,
// under that device's context (the symbol has a different address on every device).
static int grpo_static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    std::fprintf(stderr, "cvb_grpo_advantage_static: no usable current device (%s)\n", cudaGetErrorString(e));
    return CVB_ERR_STATIC_SCRATCH_SETUP;
  }
  std::lock_guard<std::mutex> lock(g_grpo_scratch_mutex);
  if (!g_grpo_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_grpo_static_scratch);
    if (e != cudaSuccess || !p) {
      std::fprintf(stderr, "cvb_grpo_advantage_static: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                   cudaGetErrorString(e));
      return CVB_ERR_STATIC_SCRATCH_SETUP;
    }
    g_grpo_scratch_addr[dev] = p;
  }
  *out = g_grpo_scratch_addr[dev];
  return 0;
}
}  // namespace cvb

extern "C" int cvb_grpo_advantage_static(const float* rewards, const float* mask, const long long* gid, float eps,
                                         int norm_by_std, float* adv, float* ret, long long rows, int cols,
                                         void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (rows > CVB_GRPO_STATIC_MAX_ROWS) {
    std::fprintf(stderr,
                 "cvb_grpo_advantage_static: %lld rows exceed the fixed scratch of %d rows; use cvb_grpo_advantage "
                 "with a caller-owned scratch buffer\n",
                 rows, CVB_GRPO_STATIC_MAX_ROWS);
    return CVB_ERR_STATIC_SCRATCH_LIMIT;
  }
  float* scratch = nullptr;
  if (const int rc = grpo_static_scratch(&scratch)) return rc;
  // scratch[0, rows): row scores; scratch[rows, 2*rows): per-row scalars.  Both ranges are fully
  // written by the first two kernels before the next one reads them: no zeroing between calls.
  const int warps_grid = static_cast<int>((rows * 32 + RL_THREADS - 1) / RL_THREADS);
  row_sum_kernel<<<warps_grid, RL_THREADS, 0, ST(stream)>>>(rewards, scratch, rows, cols);
  grpo_scalar_kernel<<<warps_grid, RL_THREADS, 0, ST(stream)>>>(scratch, gid, scratch + rows, rows, eps, norm_by_std);
  grpo_broadcast_kernel<<<rl_grid(rows * cols), RL_THREADS, 0, ST(stream)>>>(scratch + rows, mask, adv, ret, rows,
                                                                            cols);
  return static_cast<int>(cudaGetLastError());
}
