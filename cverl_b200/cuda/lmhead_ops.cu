// Tied LM-head log-prob without materialising [rows, vocab] logits.
//
// The GEMM (gemm_tcgen05.cu, EPI_LSE_PARTIAL) leaves, per row and per N tile,
// a running max and a sum of exponentials, plus the logit of the target
// token.  This kernel merges the partials into the row log-sum-exp and the
// target log-probability.  The backward pass re-runs the GEMM with
// EPI_SOFTMAX_GRAD, which writes g*(onehot - softmax) in bf16.
// Reference behaviour (full logits + log_softmax + gather):
// src/model/qwen3_5_text.cc:1590-1602; vocab-parallel form :1614-1629.
#include "ptx.cuh"

namespace cvb {

// vocab-parallel: `ext_*` hold another rank's (max, sum, target) triple to be merged first
__global__ void __launch_bounds__(256)
lse_combine_kernel(const float* __restrict__ part_max, const float* __restrict__ part_sum,
                   const float* __restrict__ tgt_logit, float* __restrict__ lse, float* __restrict__ logprob,
                   float* __restrict__ row_max_out, float* __restrict__ row_sum_out, long long M, int n_tiles) {
  const long long r = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (r >= M) return;
  float mx = -INFINITY;
  for (int t = 0; t < n_tiles; ++t) mx = fmaxf(mx, part_max[static_cast<long long>(t) * M + r]);
  float s = 0.f;
  for (int t = 0; t < n_tiles; ++t)
    s += part_sum[static_cast<long long>(t) * M + r] * __expf(part_max[static_cast<long long>(t) * M + r] - mx);
  if (row_max_out) row_max_out[r] = mx;
  if (row_sum_out) row_sum_out[r] = s;
  const float l = mx + logf(s);
  if (lse) lse[r] = l;
  if (logprob) logprob[r] = tgt_logit[r] - l;
}

// merge per-rank (max, sum) pairs gathered as [ranks, M] into lse; logprob = sum_r tgt[r] - lse
__global__ void __launch_bounds__(256)
lse_merge_ranks_kernel(const float* __restrict__ maxs, const float* __restrict__ sums,
                       const float* __restrict__ tgts, float* __restrict__ lse, float* __restrict__ logprob,
                       long long M, int ranks) {
  const long long r = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (r >= M) return;
  float mx = -INFINITY;
  for (int k = 0; k < ranks; ++k) mx = fmaxf(mx, maxs[static_cast<long long>(k) * M + r]);
  float s = 0.f, t = 0.f;
  for (int k = 0; k < ranks; ++k) {
    s += sums[static_cast<long long>(k) * M + r] * __expf(maxs[static_cast<long long>(k) * M + r] - mx);
    t += tgts[static_cast<long long>(k) * M + r];
  }
  const float l = mx + logf(s);
  lse[r] = l;
  logprob[r] = t - l;
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_lse_combine(const float* part_max, const float* part_sum, const float* tgt_logit, float* lse,
                               float* logprob, float* row_max_out, float* row_sum_out, long long M, int n_tiles,
                               void* stream) {
  if (M <= 0) return 0;
  lse_combine_kernel<<<static_cast<int>((M + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      part_max, part_sum, tgt_logit, lse, logprob, row_max_out, row_sum_out, M, n_tiles);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cvb_lse_merge_ranks(const float* maxs, const float* sums, const float* tgts, float* lse,
                                   float* logprob, long long M, int ranks, void* stream) {
  if (M <= 0) return 0;
  lse_merge_ranks_kernel<<<static_cast<int>((M + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      maxs, sums, tgts, lse, logprob, M, ranks);
  return static_cast<int>(cudaGetLastError());
}
