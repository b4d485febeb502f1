/* Public C ABI of the RL math: masked reductions, KL penalties, GAE, GRPO
 * outcome advantages and the PPO clipped policy loss, on fp32 [rows, cols]
 * views.  Symbol names, argument order and enum values follow the reference
 * (include/cverl/core_algos.h:12-100).  The `_f32_cpu` entry points are served
 * by a dependency-free C++ implementation; the device versions are the `cvb_*`
 * launchers declared in cverl_b200/cuda/core_algos_cuda.h (fused sm_100a kernels
 * on device pointers, exported from libcverl_b200_cuda.so).
 *
 * Every function validates its views (non-null data, F32, expected device,
 * non-negative and matching shapes) and returns CVERL_ERR_INVALID_ARGUMENT
 * instead of throwing. */
#ifndef CVERL_CORE_ALGOS_H_
#define CVERL_CORE_ALGOS_H_

#include <stdint.h>

#include "cverl/status.h"
#include "cverl/tensor.h"

#ifdef __cplusplus
extern "C" {
#endif

/* How per-token losses collapse into one scalar. */
typedef enum cverl_loss_agg_mode_e {
  CVERL_LOSS_AGG_TOKEN_MEAN = 0,         /* sum(l*m) / (sum(m) + 1e-8) */
  CVERL_LOSS_AGG_SEQ_MEAN_TOKEN_SUM = 1, /* mean over non-empty rows of the row sums */
  CVERL_LOSS_AGG_SEQ_MEAN_TOKEN_MEAN = 2 /* mean over non-empty rows of the row means */
} cverl_loss_agg_mode_t;

/* KL estimators between the policy and a reference policy. */
typedef enum cverl_kl_penalty_e {
  CVERL_KL_K1 = 0,  /* lp - ref */
  CVERL_KL_ABS = 1, /* |lp - ref| */
  CVERL_KL_K2 = 2,  /* 0.5 (lp - ref)^2 */
  CVERL_KL_K3 = 3   /* clamp(exp(k) - k - 1, +-10), k = clamp(ref - lp, +-20) */
} cverl_kl_penalty_t;

typedef struct cverl_ppo_loss_result_s {
  float pg_loss;           /* aggregated clipped policy-gradient loss */
  float pg_clipfrac;       /* masked fraction where the clipped branch is active */
  float ppo_kl;            /* masked mean of -(clamped log-ratio) */
  float pg_clipfrac_lower; /* masked fraction cut by the dual-clip bound (adv < 0) */
} cverl_ppo_loss_result_t;

/* sum(values * mask) */
cverl_status_t cverl_masked_sum_f32_cpu(cverl_const_tensor2d_t values, cverl_const_tensor2d_t mask,
                                        float* out_sum);
/* sum(values * mask) / (sum(mask) + 1e-8) */
cverl_status_t cverl_masked_mean_f32_cpu(cverl_const_tensor2d_t values, cverl_const_tensor2d_t mask,
                                         float* out_mean);
/* (values - mean) * rsqrt(unbiased var + 1e-8); the mean is added back when shift_mean == 0 */
cverl_status_t cverl_masked_whiten_f32_cpu(cverl_const_tensor2d_t values, cverl_const_tensor2d_t mask,
                                           int shift_mean, cverl_tensor2d_t out);

cverl_status_t cverl_kl_penalty_f32_cpu(cverl_const_tensor2d_t logprob, cverl_const_tensor2d_t ref_logprob,
                                        cverl_kl_penalty_t penalty, cverl_tensor2d_t out);
/* d sum(kl) / d logprob */
cverl_status_t cverl_kl_penalty_backward_f32_cpu(cverl_const_tensor2d_t logprob,
                                                 cverl_const_tensor2d_t ref_logprob,
                                                 cverl_kl_penalty_t penalty, cverl_tensor2d_t grad_logprob);

/* Generalised advantage estimation over the response columns (reverse scan with
 * masked carries).  `returns` = raw advantages + values; `advantages` = whitened. */
cverl_status_t cverl_gae_advantage_return_f32_cpu(cverl_const_tensor2d_t token_level_rewards,
                                                  cverl_const_tensor2d_t values,
                                                  cverl_const_tensor2d_t response_mask, float gamma, float lam,
                                                  cverl_tensor2d_t advantages, cverl_tensor2d_t returns);

/* GRPO outcome advantage: row score = sum of token rewards, normalised within
 * its group (mean 0 for singleton groups, unbiased std, std 1 for singletons),
 * broadcast over the response mask.  `group_ids` has `rows` entries. */
cverl_status_t cverl_grpo_outcome_advantage_f32_cpu(cverl_const_tensor2d_t token_level_rewards,
                                                    cverl_const_tensor2d_t response_mask,
                                                    const int64_t* group_ids, float epsilon,
                                                    int norm_adv_by_std, cverl_tensor2d_t advantages,
                                                    cverl_tensor2d_t returns);

/* PPO clipped objective with dual clip (clip_ratio_c > 1 required).  Negative
 * clip_ratio_low / clip_ratio_high mean "use clip_ratio". */
cverl_status_t cverl_ppo_clipped_loss_f32_cpu(cverl_const_tensor2d_t old_log_prob,
                                              cverl_const_tensor2d_t log_prob,
                                              cverl_const_tensor2d_t advantages,
                                              cverl_const_tensor2d_t response_mask, float clip_ratio,
                                              float clip_ratio_low, float clip_ratio_high, float clip_ratio_c,
                                              cverl_loss_agg_mode_t agg_mode, cverl_ppo_loss_result_t* out);
/* d pg_loss / d log_prob */
cverl_status_t cverl_ppo_clipped_loss_backward_f32_cpu(cverl_const_tensor2d_t old_log_prob,
                                                       cverl_const_tensor2d_t log_prob,
                                                       cverl_const_tensor2d_t advantages,
                                                       cverl_const_tensor2d_t response_mask, float clip_ratio,
                                                       float clip_ratio_low, float clip_ratio_high,
                                                       float clip_ratio_c, cverl_loss_agg_mode_t agg_mode,
                                                       cverl_tensor2d_t grad_log_prob);

#ifdef __cplusplus
}
#endif
#endif /* CVERL_CORE_ALGOS_H_ */
