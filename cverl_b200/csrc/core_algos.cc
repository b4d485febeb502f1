// Plain C++ fp32 implementation of the public RL-math C ABI (no tensor
// library behind it).  Sums accumulate in double and round once, so results
// sit within 1e-6 of an fp32 pairwise-summed evaluation of the same formulas.
//
// Formulas follow the reference's LibTorch implementation
// (src/torch/core_algos_torch.cc:9-193); argument validation follows its C
// shim (src/core_algos_c_api.cc:11-41): null data, a dtype other than F32, a
// device other than CPU, negative extents or mismatched shapes are rejected
// with CVERL_ERR_INVALID_ARGUMENT, and nothing throws across the boundary.
#include "cverl/core_algos.h"

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <map>
#include <vector>

namespace {

constexpr double kEps = 1.0e-8;

template <class View>
bool view_ok(const View& t) {
  return t.data != nullptr && t.dtype == CVERL_DTYPE_F32 && t.device == CVERL_DEVICE_CPU && t.rows >= 0 &&
         t.cols >= 0;
}
template <class A, class B>
bool same_shape(const A& a, const B& b) {
  return a.rows == b.rows && a.cols == b.cols;
}
inline const float* cptr(const cverl_const_tensor2d_t& t) { return static_cast<const float*>(t.data); }
inline float* mptr(const cverl_tensor2d_t& t) { return static_cast<float*>(t.data); }
inline int64_t numel(const cverl_const_tensor2d_t& t) { return t.rows * t.cols; }

struct MaskedStats {
  double vsum = 0.0;  // sum(v*m)
  double msum = 0.0;  // sum(m)
};
MaskedStats masked_stats(const float* v, const float* m, int64_t n) {
  MaskedStats s;
  for (int64_t i = 0; i < n; ++i) {
    s.vsum += static_cast<double>(v[i]) * m[i];
    s.msum += m[i];
  }
  return s;
}

void whiten(const float* v, const float* m, int64_t n, bool shift_mean, float* out) {
  const MaskedStats s = masked_stats(v, m, n);
  const float mean = static_cast<float>(s.vsum / (s.msum + kEps));
  double sq = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    const float c = v[i] - mean;
    sq += static_cast<double>(c * c) * m[i];
  }
  float var = static_cast<float>(sq / (s.msum + kEps));
  const float msum = static_cast<float>(s.msum);
  var = var * msum / (msum - 1.0f);  // unbiased estimate
  const float rs = 1.0f / std::sqrt(var + static_cast<float>(kEps));
  for (int64_t i = 0; i < n; ++i) {
    float w = (v[i] - mean) * rs;
    if (!shift_mean) w += mean;
    out[i] = w;
  }
}

inline float clampf(float x, float lo, float hi) { return std::min(std::max(x, lo), hi); }

float kl_value(float lp, float ref, cverl_kl_penalty_t kind) {
  const float d = lp - ref;
  switch (kind) {
    case CVERL_KL_K1: return d;
    case CVERL_KL_ABS: return std::fabs(d);
    case CVERL_KL_K2: return 0.5f * d * d;
    case CVERL_KL_K3: {
      const float k = clampf(ref - lp, -20.f, 20.f);
      return clampf(std::exp(k) - k - 1.f, -10.f, 10.f);
    }
  }
  return 0.f;
}
float kl_grad(float lp, float ref, cverl_kl_penalty_t kind) {
  const float d = lp - ref;
  switch (kind) {
    case CVERL_KL_K1: return 1.f;
    case CVERL_KL_ABS: return d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
    case CVERL_KL_K2: return d;
    case CVERL_KL_K3: {
      const float kraw = ref - lp;
      if (kraw < -20.f || kraw > 20.f) return 0.f;  // clamp blocks the gradient outside its range
      const float e = std::exp(kraw);
      const float val = e - kraw - 1.f;
      if (val < -10.f || val > 10.f) return 0.f;
      return -(e - 1.f);
    }
  }
  return 0.f;
}
bool kl_kind_ok(cverl_kl_penalty_t k) { return k >= CVERL_KL_K1 && k <= CVERL_KL_K3; }

// Token loss, its derivative w.r.t. log_prob, and the metric indicator terms.
struct PpoToken {
  float loss, dloss, clipped, lower, neg_delta;
};
PpoToken ppo_token(float old_lp, float lp, float A, float lo, float hi, float c) {
  const float draw = lp - old_lp;
  const float d = clampf(draw, -20.f, 20.f);
  const float dpass = (draw >= -20.f && draw <= 20.f) ? 1.f : 0.f;
  const float ratio = std::exp(d);
  const float rc = clampf(ratio, lo, hi);
  const float cpass = (ratio >= lo && ratio <= hi) ? 1.f : 0.f;
  const float l1 = -A * ratio, l2 = -A * rc, l3 = -A * c;
  const float g1 = -A * ratio * dpass, g2 = g1 * cpass;
  float mx, gmx;
  if (l1 > l2) {
    mx = l1, gmx = g1;
  } else if (l2 > l1) {
    mx = l2, gmx = g2;
  } else {  // tie: the sub-gradient splits evenly, as an autograd maximum does
    mx = l1, gmx = 0.5f * (g1 + g2);
  }
  PpoToken t;
  t.loss = mx;
  t.dloss = gmx;
  if (A < 0.f) {
    if (l3 < mx) {
      t.loss = l3, t.dloss = 0.f;
    } else if (l3 == mx) {
      t.dloss = 0.5f * gmx;
    }
  }
  t.clipped = l2 > l1 ? 1.f : 0.f;
  t.lower = (mx > l3 && A < 0.f) ? 1.f : 0.f;
  t.neg_delta = -d;
  return t;
}

struct PpoInputs {
  const float *old_lp, *lp, *adv, *mask;
  int64_t rows, cols;
  float lo, hi, c;
  cverl_loss_agg_mode_t mode;
};

// Per-token aggregation weights: loss = sum_i weight[i] * token_loss[i].
std::vector<float> agg_weights(const PpoInputs& in) {
  const int64_t n = in.rows * in.cols;
  std::vector<float> w(static_cast<size_t>(n));
  if (in.mode == CVERL_LOSS_AGG_TOKEN_MEAN) {
    double msum = 0.0;
    for (int64_t i = 0; i < n; ++i) msum += in.mask[i];
    const float den = static_cast<float>(msum + kEps);
    for (int64_t i = 0; i < n; ++i) w[i] = in.mask[i] / den;
    return w;
  }
  std::vector<float> cnt(static_cast<size_t>(in.rows));
  double nseq = 0.0;
  for (int64_t r = 0; r < in.rows; ++r) {
    double c = 0.0;
    for (int64_t j = 0; j < in.cols; ++j) c += in.mask[r * in.cols + j];
    cnt[r] = static_cast<float>(c);
    if (c > 0.0) nseq += 1.0;
  }
  const float den = static_cast<float>(nseq + kEps);
  for (int64_t r = 0; r < in.rows; ++r) {
    const float seqm = cnt[r] > 0.f ? 1.f : 0.f;
    float scale = seqm / den;
    if (in.mode == CVERL_LOSS_AGG_SEQ_MEAN_TOKEN_MEAN) scale /= (cnt[r] + static_cast<float>(kEps));
    for (int64_t j = 0; j < in.cols; ++j) w[r * in.cols + j] = in.mask[r * in.cols + j] * scale;
  }
  return w;
}

bool ppo_args_ok(cverl_const_tensor2d_t a, cverl_const_tensor2d_t b, cverl_const_tensor2d_t c,
                 cverl_const_tensor2d_t d, float clip_c, cverl_loss_agg_mode_t mode) {
  if (!view_ok(a) || !view_ok(b) || !view_ok(c) || !view_ok(d)) return false;
  if (!same_shape(a, b) || !same_shape(a, c) || !same_shape(a, d)) return false;
  if (!(clip_c > 1.0f)) return false;
  return mode >= CVERL_LOSS_AGG_TOKEN_MEAN && mode <= CVERL_LOSS_AGG_SEQ_MEAN_TOKEN_MEAN;
}

}  // namespace

extern "C" {

const char* cverl_status_string(cverl_status_t status) {
  switch (status) {
    case CVERL_OK: return "ok";
    case CVERL_ERR_INVALID_ARGUMENT: return "invalid argument";
    case CVERL_ERR_UNSUPPORTED: return "unsupported";
  }
  return "unknown status";
}

cverl_status_t cverl_masked_sum_f32_cpu(cverl_const_tensor2d_t values, cverl_const_tensor2d_t mask,
                                        float* out_sum) {
  if (!out_sum || !view_ok(values) || !view_ok(mask) || !same_shape(values, mask))
    return CVERL_ERR_INVALID_ARGUMENT;
  *out_sum = static_cast<float>(masked_stats(cptr(values), cptr(mask), numel(values)).vsum);
  return CVERL_OK;
}

cverl_status_t cverl_masked_mean_f32_cpu(cverl_const_tensor2d_t values, cverl_const_tensor2d_t mask,
                                         float* out_mean) {
  if (!out_mean || !view_ok(values) || !view_ok(mask) || !same_shape(values, mask))
    return CVERL_ERR_INVALID_ARGUMENT;
  const MaskedStats s = masked_stats(cptr(values), cptr(mask), numel(values));
  *out_mean = static_cast<float>(s.vsum / (s.msum + kEps));
  return CVERL_OK;
}

cverl_status_t cverl_masked_whiten_f32_cpu(cverl_const_tensor2d_t values, cverl_const_tensor2d_t mask,
                                           int shift_mean, cverl_tensor2d_t out) {
  if (!view_ok(values) || !view_ok(mask) || !same_shape(values, mask) || !view_ok(out) ||
      !same_shape(values, out))
    return CVERL_ERR_INVALID_ARGUMENT;
  whiten(cptr(values), cptr(mask), numel(values), shift_mean != 0, mptr(out));
  return CVERL_OK;
}

cverl_status_t cverl_kl_penalty_f32_cpu(cverl_const_tensor2d_t logprob, cverl_const_tensor2d_t ref_logprob,
                                        cverl_kl_penalty_t penalty, cverl_tensor2d_t out) {
  if (!view_ok(logprob) || !view_ok(ref_logprob) || !same_shape(logprob, ref_logprob) || !view_ok(out) ||
      !same_shape(logprob, out) || !kl_kind_ok(penalty))
    return CVERL_ERR_INVALID_ARGUMENT;
  const int64_t n = numel(logprob);
  for (int64_t i = 0; i < n; ++i) mptr(out)[i] = kl_value(cptr(logprob)[i], cptr(ref_logprob)[i], penalty);
  return CVERL_OK;
}

cverl_status_t cverl_kl_penalty_backward_f32_cpu(cverl_const_tensor2d_t logprob,
                                                 cverl_const_tensor2d_t ref_logprob,
                                                 cverl_kl_penalty_t penalty, cverl_tensor2d_t grad_logprob) {
  if (!view_ok(logprob) || !view_ok(ref_logprob) || !same_shape(logprob, ref_logprob) ||
      !view_ok(grad_logprob) || !same_shape(logprob, grad_logprob) || !kl_kind_ok(penalty))
    return CVERL_ERR_INVALID_ARGUMENT;
  const int64_t n = numel(logprob);
  for (int64_t i = 0; i < n; ++i)
    mptr(grad_logprob)[i] = kl_grad(cptr(logprob)[i], cptr(ref_logprob)[i], penalty);
  return CVERL_OK;
}

cverl_status_t cverl_gae_advantage_return_f32_cpu(cverl_const_tensor2d_t token_level_rewards,
                                                  cverl_const_tensor2d_t values,
                                                  cverl_const_tensor2d_t response_mask, float gamma, float lam,
                                                  cverl_tensor2d_t advantages, cverl_tensor2d_t returns) {
  if (!view_ok(token_level_rewards) || !view_ok(values) || !view_ok(response_mask) ||
      !same_shape(token_level_rewards, values) || !same_shape(token_level_rewards, response_mask) ||
      !view_ok(advantages) || !same_shape(token_level_rewards, advantages) || !view_ok(returns) ||
      !same_shape(token_level_rewards, returns))
    return CVERL_ERR_INVALID_ARGUMENT;
  const int64_t rows = token_level_rewards.rows, cols = token_level_rewards.cols;
  const float *rew = cptr(token_level_rewards), *val = cptr(values), *msk = cptr(response_mask);
  std::vector<float> raw(static_cast<size_t>(rows * cols));
  for (int64_t r = 0; r < rows; ++r) {
    float next_value = 0.f, last = 0.f;
    for (int64_t c = cols - 1; c >= 0; --c) {
      const int64_t i = r * cols + c;
      const float delta = rew[i] + gamma * next_value - val[i];
      const float cand = delta + gamma * lam * last;
      next_value = val[i] * msk[i] + (1.f - msk[i]) * next_value;
      last = cand * msk[i] + (1.f - msk[i]) * last;
      raw[i] = last;
    }
  }
  for (int64_t i = 0; i < rows * cols; ++i) mptr(returns)[i] = raw[i] + val[i];
  whiten(raw.data(), msk, rows * cols, /*shift_mean=*/true, mptr(advantages));
  return CVERL_OK;
}

cverl_status_t cverl_grpo_outcome_advantage_f32_cpu(cverl_const_tensor2d_t token_level_rewards,
                                                    cverl_const_tensor2d_t response_mask,
                                                    const int64_t* group_ids, float epsilon,
                                                    int norm_adv_by_std, cverl_tensor2d_t advantages,
                                                    cverl_tensor2d_t returns) {
  if (!group_ids || !view_ok(token_level_rewards) || !view_ok(response_mask) ||
      !same_shape(token_level_rewards, response_mask) || !view_ok(advantages) ||
      !same_shape(token_level_rewards, advantages) || !view_ok(returns) ||
      !same_shape(token_level_rewards, returns))
    return CVERL_ERR_INVALID_ARGUMENT;
  const int64_t rows = token_level_rewards.rows, cols = token_level_rewards.cols;
  const float *rew = cptr(token_level_rewards), *msk = cptr(response_mask);
  std::vector<float> score(static_cast<size_t>(rows));
  struct Group {
    double sum = 0.0, sq = 0.0;
    int64_t count = 0;
    float mean = 0.f, std = 1.f;
  };
  std::map<int64_t, Group> groups;
  for (int64_t r = 0; r < rows; ++r) {
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += rew[r * cols + c];
    score[r] = static_cast<float>(s);
    Group& g = groups[group_ids[r]];
    g.sum += score[r];
    g.count += 1;
  }
  for (auto& kv : groups) {
    Group& g = kv.second;
    g.mean = g.count > 1 ? static_cast<float>(g.sum / static_cast<double>(g.count)) : 0.f;
  }
  if (norm_adv_by_std) {
    for (int64_t r = 0; r < rows; ++r) {
      Group& g = groups[group_ids[r]];
      const float d = score[r] - g.mean;
      g.sq += static_cast<double>(d) * d;
    }
    for (auto& kv : groups) {
      Group& g = kv.second;
      g.std = g.count > 1 ? static_cast<float>(std::sqrt(g.sq / static_cast<double>(g.count - 1))) : 1.f;
    }
  }
  for (int64_t r = 0; r < rows; ++r) {
    const Group& g = groups[group_ids[r]];
    float s = score[r] - g.mean;
    if (norm_adv_by_std) s = s / (g.std + epsilon);
    for (int64_t c = 0; c < cols; ++c) {
      const float a = s * msk[r * cols + c];
      mptr(advantages)[r * cols + c] = a;
      mptr(returns)[r * cols + c] = a;
    }
  }
  return CVERL_OK;
}

cverl_status_t cverl_ppo_clipped_loss_f32_cpu(cverl_const_tensor2d_t old_log_prob,
                                              cverl_const_tensor2d_t log_prob,
                                              cverl_const_tensor2d_t advantages,
                                              cverl_const_tensor2d_t response_mask, float clip_ratio,
                                              float clip_ratio_low, float clip_ratio_high, float clip_ratio_c,
                                              cverl_loss_agg_mode_t agg_mode, cverl_ppo_loss_result_t* out) {
  if (!out || !ppo_args_ok(old_log_prob, log_prob, advantages, response_mask, clip_ratio_c, agg_mode))
    return CVERL_ERR_INVALID_ARGUMENT;
  if (clip_ratio_low < 0.f) clip_ratio_low = clip_ratio;
  if (clip_ratio_high < 0.f) clip_ratio_high = clip_ratio;
  PpoInputs in{cptr(old_log_prob), cptr(log_prob), cptr(advantages), cptr(response_mask), log_prob.rows,
               log_prob.cols, 1.f - clip_ratio_low, 1.f + clip_ratio_high, clip_ratio_c, agg_mode};
  const std::vector<float> w = agg_weights(in);
  const int64_t n = in.rows * in.cols;
  double loss = 0.0, clip = 0.0, low = 0.0, kl = 0.0, msum = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    const PpoToken t = ppo_token(in.old_lp[i], in.lp[i], in.adv[i], in.lo, in.hi, in.c);
    const float m = in.mask[i];
    loss += static_cast<double>(t.loss) * w[i];
    clip += static_cast<double>(t.clipped) * m;
    low += static_cast<double>(t.lower) * m;
    kl += static_cast<double>(t.neg_delta) * m;
    msum += m;
  }
  out->pg_loss = static_cast<float>(loss);
  out->pg_clipfrac = static_cast<float>(clip / (msum + kEps));
  out->ppo_kl = static_cast<float>(kl / (msum + kEps));
  out->pg_clipfrac_lower = static_cast<float>(low / (msum + kEps));
  return CVERL_OK;
}

cverl_status_t cverl_ppo_clipped_loss_backward_f32_cpu(cverl_const_tensor2d_t old_log_prob,
                                                       cverl_const_tensor2d_t log_prob,
                                                       cverl_const_tensor2d_t advantages,
                                                       cverl_const_tensor2d_t response_mask, float clip_ratio,
                                                       float clip_ratio_low, float clip_ratio_high,
                                                       float clip_ratio_c, cverl_loss_agg_mode_t agg_mode,
                                                       cverl_tensor2d_t grad_log_prob) {
  if (!ppo_args_ok(old_log_prob, log_prob, advantages, response_mask, clip_ratio_c, agg_mode) ||
      !view_ok(grad_log_prob) || !same_shape(log_prob, grad_log_prob))
    return CVERL_ERR_INVALID_ARGUMENT;
  if (clip_ratio_low < 0.f) clip_ratio_low = clip_ratio;
  if (clip_ratio_high < 0.f) clip_ratio_high = clip_ratio;
  PpoInputs in{cptr(old_log_prob), cptr(log_prob), cptr(advantages), cptr(response_mask), log_prob.rows,
               log_prob.cols, 1.f - clip_ratio_low, 1.f + clip_ratio_high, clip_ratio_c, agg_mode};
  const std::vector<float> w = agg_weights(in);
  const int64_t n = in.rows * in.cols;
  for (int64_t i = 0; i < n; ++i) {
    const PpoToken t = ppo_token(in.old_lp[i], in.lp[i], in.adv[i], in.lo, in.hi, in.c);
    mptr(grad_log_prob)[i] = t.dloss * w[i];
  }
  return CVERL_OK;
}

}  // extern "C"
