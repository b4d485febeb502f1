// Gate math of the Gated-DeltaNet block in one kernel each way:
//     beta = sigmoid(b)            g = -exp(A_log) * softplus(a + dt_bias)
// b, a: bf16 [rows, H] column groups of the fused input projection (row stride `in_stride`), A_log, dt_bias: [H]
// parameters, beta, g: fp32 [rows, H].  The backward writes db, da as bf16 with their own row stride (so they can
// land in the projection-gradient buffer) and accumulates dA_log, ddt_bias (fp32) with one atomic per block and head.
// Reference math: src/model/qwen3_5_text.cc:1246-1252 (beta / g of the linear-attention block); the reference runs
// it as separate tensor ops.
#include "ptx.cuh"

namespace cvb {

constexpr int GG_THREADS = 256;
constexpr int GG_MAX_H = 256;

__device__ __forceinline__ float gg_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float gg_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(GG_THREADS)
gdn_gates_fwd_kernel(const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ a,
                     const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias,
                     float* __restrict__ beta, float* __restrict__ g, long long rows, int H, long long in_stride) {
  const long long total = rows * H;
  for (long long i = static_cast<long long>(blockIdx.x) * GG_THREADS + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * GG_THREADS) {
    const long long r = i / H;
    const int h = static_cast<int>(i - r * H);
    const float bv = __bfloat162float(b[r * in_stride + h]);
    const float av = __bfloat162float(a[r * in_stride + h]);
    beta[i] = gg_sigmoid(bv);
    g[i] = -__expf(__bfloat162float(A_log[h])) * gg_softplus(av + __bfloat162float(dt_bias[h]));
  }
}

// One block owns a contiguous range of rows; thread (tid % H) accumulates its head over the rows tid / H,
// tid / H + GG_THREADS / H, ...  Requires GG_THREADS % H == 0 (H a power of two up to 256).
__global__ void __launch_bounds__(GG_THREADS)
gdn_gates_bwd_kernel(const float* __restrict__ dbeta, const float* __restrict__ dg,
                     const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ a,
                     const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias,
                     __nv_bfloat16* __restrict__ db, __nv_bfloat16* __restrict__ da, float* __restrict__ dA_log,
                     float* __restrict__ ddt_bias, long long rows, int H, long long in_stride, long long d_stride,
                     long long rows_per_block) {
  __shared__ float s_dA[GG_THREADS], s_dB[GG_THREADS];
  const int h = threadIdx.x % H;
  const int lane_row = threadIdx.x / H;
  const int rows_per_pass = GG_THREADS / H;
  const long long r_begin = static_cast<long long>(blockIdx.x) * rows_per_block;
  const long long r_end = r_begin + rows_per_block < rows ? r_begin + rows_per_block : rows;
  const float neg_ea = -__expf(__bfloat162float(A_log[h]));
  const float bias = __bfloat162float(dt_bias[h]);
  float acc_dA = 0.f, acc_dB = 0.f;
  for (long long r = r_begin + lane_row; r < r_end; r += rows_per_pass) {
    const float bv = __bfloat162float(b[r * in_stride + h]);
    const float x = __bfloat162float(a[r * in_stride + h]) + bias;
    const float sb = gg_sigmoid(bv);
    const float dgv = dg[r * H + h];
    const float dsp = x > 20.f ? 1.f : gg_sigmoid(x);   // d softplus / dx
    const float dx = dgv * neg_ea * dsp;
    db[r * d_stride + h] = __float2bfloat16_rn(dbeta[r * H + h] * sb * (1.f - sb));
    da[r * d_stride + h] = __float2bfloat16_rn(dx);
    acc_dB += dx;
    acc_dA += dgv * neg_ea * gg_softplus(x);             // dg * g
  }
  s_dA[threadIdx.x] = acc_dA;
  s_dB[threadIdx.x] = acc_dB;
  __syncthreads();
  if (threadIdx.x < H) {
    float sa = 0.f, sbv = 0.f;
    for (int k = threadIdx.x; k < GG_THREADS; k += H) sa += s_dA[k], sbv += s_dB[k];
    atomicAdd(dA_log + threadIdx.x, sa);
    atomicAdd(ddt_bias + threadIdx.x, sbv);
  }
}

}  // namespace cvb

using namespace cvb;

static bool gg_head_count_ok(int H) { return H > 0 && H <= GG_MAX_H && (H & (H - 1)) == 0; }

extern "C" int cvb_gdn_gates_fwd(const void* b, const void* a, const void* A_log, const void* dt_bias, float* beta,
                                 float* g, long long rows, int H, long long in_stride, void* stream) {
  if (rows <= 0) return 0;
  if (!gg_head_count_ok(H)) return -2;
  const long long total = rows * H;
  long long blocks = (total + GG_THREADS - 1) / GG_THREADS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  gdn_gates_fwd_kernel<<<static_cast<unsigned>(blocks), GG_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(b), static_cast<const __nv_bfloat16*>(a),
      static_cast<const __nv_bfloat16*>(A_log), static_cast<const __nv_bfloat16*>(dt_bias), beta, g, rows, H,
      in_stride);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_gdn_gates_bwd(const float* dbeta, const float* dg, const void* b, const void* a, const void* A_log,
                                 const void* dt_bias, void* db, void* da, float* dA_log, float* ddt_bias,
                                 long long rows, int H, long long in_stride, long long d_stride, void* stream) {
  if (rows <= 0) return 0;
  if (!gg_head_count_ok(H)) return -2;
  long long blocks = 148 * 4;
  long long rows_per_block = (rows + blocks - 1) / blocks;
  const int rows_per_pass = GG_THREADS / H;
  rows_per_block = (rows_per_block + rows_per_pass - 1) / rows_per_pass * rows_per_pass;
  blocks = (rows + rows_per_block - 1) / rows_per_block;
  gdn_gates_bwd_kernel<<<static_cast<unsigned>(blocks), GG_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      dbeta, dg, static_cast<const __nv_bfloat16*>(b), static_cast<const __nv_bfloat16*>(a),
      static_cast<const __nv_bfloat16*>(A_log), static_cast<const __nv_bfloat16*>(dt_bias),
      static_cast<__nv_bfloat16*>(db), static_cast<__nv_bfloat16*>(da), dA_log, ddt_bias, rows, H, in_stride,
      d_stride, rows_per_block);
  return static_cast<int>(cudaGetLastError());
}
