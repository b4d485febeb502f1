// CUDA siblings of the public RL-math C ABI (csrc/include/cverl/core_algos.h): the same operations on
// fp32 device tensors, exported by libcverl_b200_cuda.so.  All pointers are device pointers on the current
// device; `stream` is a cudaStream_t; every function returns 0 or a CUDA / argument error code and only
// enqueues work.  Matrices are row-major [rows, cols] without padding; `n` counts elements.
// Scratch is owned by the caller: `ws` = cvb_rl_workspace_doubles() doubles, zeroed by the callee.
//
// Enumerations follow the CPU ABI: KL kind 0 = k1, 1 = abs, 2 = k2, 3 = k3; loss aggregation
// 0 = token-mean, 1 = seq-mean-token-sum, 2 = seq-mean-token-mean.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int cvb_rl_workspace_doubles();

// out[0] = sum(values * mask)  (mean != 0: divided by sum(mask) + 1e-8)
int cvb_masked_sum_mean(const float* values, const float* mask, long long n, int mean, float* out, double* ws,
                        void* stream);
// out = (values - mean) / sqrt(var + 1e-8) (+ mean when shift_mean == 0), masked mean and unbiased variance
int cvb_masked_whiten(const float* values, const float* mask, long long n, int shift_mean, float* out, double* ws,
                      void* stream);
// out = penalty(logprob, ref) or, with backward != 0, d penalty / d logprob
int cvb_kl_penalty(const float* logprob, const float* ref, float* out, long long n, int kind, int backward,
                   void* stream);
// GAE: adv_raw (un-whitened) and ret written per token, adv_out = whiten(adv_raw, mask)
int cvb_gae(const float* rewards, const float* values, const float* mask, float* adv_raw, float* adv_out, float* ret,
            long long rows, int cols, float gamma, float lam, double* ws, void* stream);
// GRPO outcome advantage; group ids int64 [rows]; row_scratch: 2 * rows floats; ret may be null
int cvb_grpo_advantage(const float* rewards, const float* mask, const long long* group_ids, float eps, int norm_by_std,
                       float* adv, float* ret, float* row_scratch, long long rows, int cols, void* stream);
// Dual-clip PPO loss fused with its gradient w.r.t. log_prob (grad may be null) and an optional KL term
// (ref_lp may be null).  metrics_out: pg_loss, pg_clipfrac, ppo_kl, pg_clipfrac_lower, kl_loss, token count.
// rowcnt: rows floats of scratch.  The gradient is scaled by loss_scale.
int cvb_ppo_loss(const float* old_lp, const float* lp, const float* adv, const float* mask, const float* ref_lp,
                 float* grad, float* metrics_out, float* rowcnt, long long rows, int cols, float clip, float clip_low,
                 float clip_high, float clip_c, int agg_mode, float kl_coef, int kl_kind, float loss_scale, double* ws,
                 void* stream);

#ifdef __cplusplus
}
#endif
