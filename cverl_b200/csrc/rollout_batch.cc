// Builds the tensors of a GRPO step from prompts, sampled responses and gold answers, on several threads.
//
// Same rules as the reference's builder (src/rollout/rollout_batch.cc:42-136): a prompt is tokenised once per prompt
// index with the limit max_prompt_len (the FIRST max_prompt_len tokens of an over-long prompt are kept, an
// optional BOS in front) and LEFT-padded; a response that comes as text is tokenised with the limit
// max_response_len and gets an EOS where the limit leaves room (add_eos, the reference's default), a response that
// comes with token ids keeps its first max_response_len ids; responses are RIGHT-padded; response_mask marks
// real response tokens; group_ids is the prompt index; the scalar GSM8K rule reward sits on the last real
// response token.  The reference walks the samples in one thread; here the distinct prompts and then
// the samples are spread over worker threads (tokenisation and the reward rule are the whole cost), and every
// worker writes only its own rows of the caller's buffers.
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <string>
#include <thread>
#include <vector>

extern "C" {
int64_t cverl_bpe_encode(void* h, const char* text, int64_t len, int64_t* out, int64_t capacity);
int64_t cverl_byte_encode(const char* text, int64_t len, int add_bos, int add_eos, int64_t max_tokens, int64_t* out,
                          int64_t capacity);
double cverl_gsm8k_reward(const char* solution, const char* ground_truth, int flexible, int64_t clip_chars,
                          double correct_score, double format_score, double no_answer_score);
}

namespace {

enum { TOK_BYTE = 0, TOK_BPE = 1 };

// text -> ids with the reference's option rules: BOS in front when asked for (and the vocabulary has one), EOS at
// the end only if the limit leaves room, at most max_tokens ids (the head is kept)
std::vector<int64_t> encode(int kind, void* handle, const char* text, int64_t len, bool add_bos, bool add_eos,
                            int64_t bos_id, int64_t eos_id, int64_t max_tokens) {
  std::vector<int64_t> ids(static_cast<size_t>(len) + 8);   // a token covers at least one byte
  const int64_t cap = static_cast<int64_t>(ids.size());
  const int64_t n = kind == TOK_BPE ? cverl_bpe_encode(handle, text, len, ids.data(), cap)
                                    : cverl_byte_encode(text, len, 0, 0, 0, ids.data(), cap);
  ids.resize(static_cast<size_t>(std::max<int64_t>(0, std::min(n, cap))));
  if (add_bos && bos_id >= 0) ids.insert(ids.begin(), bos_id);
  if (max_tokens > 0 && static_cast<int64_t>(ids.size()) > max_tokens) ids.resize(static_cast<size_t>(max_tokens));
  if (add_eos && eos_id >= 0 && (max_tokens <= 0 || static_cast<int64_t>(ids.size()) < max_tokens)) ids.push_back(eos_id);
  return ids;
}

template <class F>
void parallel_for(int64_t n, int threads, F&& body) {
  std::atomic<int64_t> next{0};
  auto work = [&]() {
    for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) body(i);
  };
  const int64_t nt = std::max<int64_t>(1, std::min<int64_t>(threads, n));
  if (nt == 1) {
    work();
    return;
  }
  std::vector<std::thread> pool;
  for (int64_t t = 0; t < nt; ++t) pool.emplace_back(work);
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// tokenizer_kind 0: byte tokenizer (handle unused); 1: BPE handle of cverl_bpe_open.
// given_ids / given_offsets / has_given (all three or none): token ids that came with a response; sample i uses
// given_ids[given_offsets[i] .. given_offsets[i+1]) when has_given[i], else its text is tokenised.
// Outputs, caller-allocated: prompt_ids [B, P], response_ids [B, R] (int64), response_mask, token_rewards [B, R]
// (float), rewards [B] (float), group_ids [B] (int64).  Returns 0, or 1 for a bad argument (nothing is written
// beyond the rows already filled).
int cverl_build_gsm8k_rollout_batch(int tokenizer_kind, void* tokenizer, int64_t pad_id,
                                    const char* const* prompts, const int64_t* prompt_lens, const char* const* answers,
                                    int64_t n_prompts, const int64_t* sample_prompt, const char* const* responses,
                                    const int64_t* response_lens, const int64_t* given_ids,
                                    const int64_t* given_offsets, const uint8_t* has_given, int64_t n_samples,
                                    int64_t max_prompt_len, int64_t max_response_len, int add_bos, int add_eos,
                                    int64_t bos_id, int64_t eos_id, int flexible, int64_t clip_chars,
                                    double correct_score, double format_score, double no_answer_score, int threads,
                                    int64_t* prompt_ids, int64_t* response_ids, float* response_mask,
                                    float* token_rewards, float* rewards, int64_t* group_ids) {
  if (!prompts || !prompt_lens || !answers || !sample_prompt || !responses || !response_lens || !prompt_ids ||
      !response_ids || !response_mask || !token_rewards || !rewards || !group_ids)
    return 1;
  if (n_prompts < 0 || n_samples <= 0 || max_prompt_len <= 0 || max_response_len <= 0) return 1;
  if ((tokenizer_kind != TOK_BYTE && tokenizer_kind != TOK_BPE) || (tokenizer_kind == TOK_BPE && !tokenizer)) return 1;
  const bool given = given_ids && given_offsets && has_given;
  std::vector<uint8_t> used(static_cast<size_t>(n_prompts), 0);
  for (int64_t b = 0; b < n_samples; ++b) {
    if (sample_prompt[b] < 0 || sample_prompt[b] >= n_prompts) return 1;
    used[static_cast<size_t>(sample_prompt[b])] = 1;
    if (given && has_given[b] && given_offsets[b + 1] < given_offsets[b]) return 1;
  }
  std::vector<int64_t> distinct;
  for (int64_t p = 0; p < n_prompts; ++p)
    if (used[static_cast<size_t>(p)]) distinct.push_back(p);
  std::vector<std::vector<int64_t>> prompt_tokens(static_cast<size_t>(n_prompts));
  parallel_for(static_cast<int64_t>(distinct.size()), threads, [&](int64_t k) {
    const int64_t p = distinct[static_cast<size_t>(k)];
    prompt_tokens[static_cast<size_t>(p)] = encode(tokenizer_kind, tokenizer, prompts[p], prompt_lens[p], add_bos != 0,
                                                   false, bos_id, eos_id, max_prompt_len);
  });
  const int64_t P = max_prompt_len, R = max_response_len;
  parallel_for(n_samples, threads, [&](int64_t b) {
    const int64_t p = sample_prompt[b];
    int64_t* prow = prompt_ids + b * P;
    int64_t* rrow = response_ids + b * R;
    float* mrow = response_mask + b * R;
    float* trow = token_rewards + b * R;
    std::fill(prow, prow + P, pad_id);
    std::fill(rrow, rrow + R, pad_id);
    std::fill(mrow, mrow + R, 0.0f);
    std::fill(trow, trow + R, 0.0f);
    const auto& pt = prompt_tokens[static_cast<size_t>(p)];
    const int64_t keep = std::min<int64_t>(P, static_cast<int64_t>(pt.size()));          // already cut to P ids
    std::copy(pt.end() - keep, pt.end(), prow + (P - keep));
    int64_t n = 0;
    if (given && has_given[b]) {
      n = std::min<int64_t>(R, given_offsets[b + 1] - given_offsets[b]);
      std::copy(given_ids + given_offsets[b], given_ids + given_offsets[b] + n, rrow);
    } else {
      const auto rt = encode(tokenizer_kind, tokenizer, responses[b], response_lens[b], false, add_eos != 0, bos_id,
                             eos_id, R);
      n = std::min<int64_t>(R, static_cast<int64_t>(rt.size()));                         // the head of the response
      std::copy(rt.begin(), rt.begin() + n, rrow);
    }
    std::fill(mrow, mrow + n, 1.0f);
    const std::string text(responses[b], static_cast<size_t>(response_lens[b]));         // the rule reads a C string
    const double rew = cverl_gsm8k_reward(text.c_str(), answers[p], flexible, clip_chars, correct_score, format_score,
                                          no_answer_score);
    rewards[b] = static_cast<float>(rew);
    if (n > 0) trow[n - 1] = static_cast<float>(rew);
    group_ids[b] = p;
  });
  return 0;
}

}  // extern "C"
