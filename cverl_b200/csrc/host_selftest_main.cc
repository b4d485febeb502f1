// Stand-alone exercise of the host runtime's C ABI, meant to be built with -fsanitize=address,undefined or
// -fsanitize=thread (python -m cverl_b200._build --sanitize address|thread) and run on a CPU box:
//   * the RL math entry points on ragged masks, from several threads at once (they share no state);
//   * argument validation paths (null data, shape mismatch) that must return an error, not touch memory;
//   * the topology planner, 1F1B schedule and greedy owner assignment;
//   * the safetensors writer / reader round trip, the byte tokenizer, the GSM8K answer extraction and the JSONL reader;
//   * the shared-memory request / response transport with a server thread and a client thread;
//   * with a tokenizer.json as the first argument, the BPE tokenizer from two threads on one handle;
//   * with a plugin .so as the second argument, the rollout-worker plugin loader.
// Exit code 0 and a silent sanitizer are the pass criterion.  The reference ships no sanitizer target.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <unistd.h>

#include "cverl/core_algos.h"
#include "cverl/rollout_plugin.h"
#include "cverl/topology.h"

extern "C" {
void* cverl_shm_transport_open(const char* name, int64_t payload_capacity, int create);
void cverl_shm_transport_close(void* h);
int64_t cverl_shm_client_call(void* h, const void* request, int64_t request_size, void* response,
                              int64_t response_capacity, int64_t timeout_ms);
int64_t cverl_shm_server_wait(void* h, void* request, int64_t capacity, int64_t timeout_ms);
int cverl_shm_server_reply(void* h, const void* response, int64_t size, int status);
void* cverl_st_open(const char* path, char* err, int err_len);
void cverl_st_close(void* h);
int64_t cverl_st_count(void* h);
const char* cverl_st_name(void* h, int64_t i);
int cverl_st_info(void* h, const char* name, int* dtype, int* ndim, int64_t* shape8, int64_t* nbytes);
int cverl_st_read(void* h, const char* name, void* dst, int64_t nbytes);
int cverl_st_read_range(void* h, const char* name, int64_t offset, int64_t nbytes, void* dst, int threads);
int cverl_st_write(const char* path, int64_t n, const char* const* names, const int* dtypes, const int* ndims,
                   const int64_t* shapes, const void* const* data);
int64_t cverl_byte_encode(const char* text, int64_t len, int add_bos, int add_eos, int64_t max_tokens, int64_t* out,
                          int64_t capacity);
int64_t cverl_byte_decode(const int64_t* ids, int64_t n, int skip_special, char* out, int64_t capacity);
int cverl_gsm8k_extract(const char* solution, int flexible, int64_t clip_chars, char* out, int64_t capacity);
double cverl_gsm8k_reward(const char* solution, const char* ground_truth, int flexible, int64_t clip_chars,
                          double correct_score, double format_score, double no_answer_score);
void* cverl_jsonl_open(const char* path, const char* field_a, const char* field_b, int64_t max_rows);
const char* cverl_jsonl_error(void* h);
int64_t cverl_jsonl_rows(void* h);
const char* cverl_jsonl_get(void* h, int64_t row, int which);
void cverl_jsonl_close(void* h);
void* cverl_bpe_open(const char* tokenizer_json, char* err, int err_len);
void cverl_bpe_close(void* h);
int64_t cverl_bpe_vocab_size(void* h);
int64_t cverl_bpe_encode(void* h, const char* text, int64_t len, int64_t* out, int64_t capacity);
int64_t cverl_bpe_decode(void* h, const int64_t* ids, int64_t n, int skip_special, char* out, int64_t capacity);
int cverl_build_gsm8k_rollout_batch(int tokenizer_kind, void* tokenizer, int64_t pad_id, const char* const* prompts,
                                    const int64_t* prompt_lens, const char* const* answers, int64_t n_prompts,
                                    const int64_t* sample_prompt, const char* const* responses,
                                    const int64_t* response_lens, const int64_t* given_ids,
                                    const int64_t* given_offsets, const uint8_t* has_given, int64_t n_samples,
                                    int64_t max_prompt_len, int64_t max_response_len, int add_bos, int add_eos,
                                    int64_t bos_id, int64_t eos_id, int flexible, int64_t clip_chars,
                                    double correct_score, double format_score, double no_answer_score, int threads,
                                    int64_t* prompt_ids, int64_t* response_ids, float* response_mask,
                                    float* token_rewards, float* rewards, int64_t* group_ids);
int64_t cverl_bpe_encode_batch(void* h, const char* const* texts, const int64_t* lens, int64_t n, int threads,
                               int64_t* out, int64_t capacity, int64_t* offsets);
}

namespace {

int g_failures = 0;
#define EXPECT(cond)                                                   \
  do {                                                                 \
    if (!(cond)) {                                                     \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      __atomic_add_fetch(&g_failures, 1, __ATOMIC_SEQ_CST);            \
    }                                                                  \
  } while (0)

cverl_const_tensor2d_t cview(const std::vector<float>& v, int64_t r, int64_t c) {
  return {v.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, r, c};
}
cverl_tensor2d_t view(std::vector<float>& v, int64_t r, int64_t c) {
  return {v.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, r, c};
}

void rl_math(unsigned seed) {
  const int64_t R = 16, C = 37;
  std::vector<float> lp(R * C), old(R * C), ref(R * C), mask(R * C), rew(R * C, 0.f), val(R * C);
  std::vector<int64_t> groups(R);
  uint32_t s = seed * 2654435761u + 1u;
  auto rnd = [&]() { s = s * 1664525u + 1013904223u; return (s >> 8) * (1.0f / 16777216.0f); };
  for (int64_t r = 0; r < R; ++r) {
    const int64_t len = 1 + static_cast<int64_t>(rnd() * (C - 1));
    groups[r] = r / 4;
    for (int64_t c = 0; c < C; ++c) {
      const int64_t i = r * C + c;
      lp[i] = -2.f + rnd();
      old[i] = lp[i] + 0.05f * (rnd() - 0.5f);
      ref[i] = lp[i] + 0.1f * (rnd() - 0.5f);
      mask[i] = c < len ? 1.f : 0.f;
      val[i] = rnd() - 0.5f;
    }
    rew[r * C + len - 1] = rnd() > 0.5f ? 1.f : 0.f;
  }
  std::vector<float> adv(R * C), ret(R * C), gadv(R * C), gret(R * C), white(R * C), dlp(R * C), kl(R * C), dkl(R * C);
  EXPECT(cverl_grpo_outcome_advantage_f32_cpu(cview(rew, R, C), cview(mask, R, C), groups.data(), 1e-6f, 1,
                                              view(adv, R, C), view(ret, R, C)) == CVERL_OK);
  EXPECT(cverl_gae_advantage_return_f32_cpu(cview(rew, R, C), cview(val, R, C), cview(mask, R, C), 1.0f, 0.95f,
                                            view(gadv, R, C), view(gret, R, C)) == CVERL_OK);
  EXPECT(cverl_masked_whiten_f32_cpu(cview(adv, R, C), cview(mask, R, C), 1, view(white, R, C)) == CVERL_OK);
  cverl_ppo_loss_result_t res{};
  for (int mode = 0; mode < 3; ++mode) {
    EXPECT(cverl_ppo_clipped_loss_f32_cpu(cview(old, R, C), cview(lp, R, C), cview(white, R, C), cview(mask, R, C),
                                          0.2f, -1.f, -1.f, 3.0f, static_cast<cverl_loss_agg_mode_t>(mode), &res) ==
           CVERL_OK);
    EXPECT(std::isfinite(res.pg_loss));
    EXPECT(cverl_ppo_clipped_loss_backward_f32_cpu(cview(old, R, C), cview(lp, R, C), cview(white, R, C),
                                                   cview(mask, R, C), 0.2f, -1.f, -1.f, 3.0f,
                                                   static_cast<cverl_loss_agg_mode_t>(mode), view(dlp, R, C)) ==
           CVERL_OK);
  }
  for (int k = 0; k < 4; ++k) {
    EXPECT(cverl_kl_penalty_f32_cpu(cview(lp, R, C), cview(ref, R, C), static_cast<cverl_kl_penalty_t>(k),
                                    view(kl, R, C)) == CVERL_OK);
    EXPECT(cverl_kl_penalty_backward_f32_cpu(cview(lp, R, C), cview(ref, R, C), static_cast<cverl_kl_penalty_t>(k),
                                             view(dkl, R, C)) == CVERL_OK);
  }
  float sum = 0.f, mean = 0.f;
  EXPECT(cverl_masked_sum_f32_cpu(cview(kl, R, C), cview(mask, R, C), &sum) == CVERL_OK);
  EXPECT(cverl_masked_mean_f32_cpu(cview(kl, R, C), cview(mask, R, C), &mean) == CVERL_OK);
  EXPECT(std::isfinite(sum) && std::isfinite(mean));
  // validation: these must come back as errors without reading or writing through the bad views
  cverl_const_tensor2d_t null_view{nullptr, CVERL_DTYPE_F32, CVERL_DEVICE_CPU, R, C};
  EXPECT(cverl_masked_sum_f32_cpu(null_view, cview(mask, R, C), &sum) != CVERL_OK);
  EXPECT(cverl_masked_sum_f32_cpu(cview(kl, R, C), cview(mask, R, C - 1), &sum) != CVERL_OK);
  EXPECT(cverl_masked_sum_f32_cpu(cview(kl, R, C), cview(mask, R, C), nullptr) != CVERL_OK);
  EXPECT(cverl_ppo_clipped_loss_f32_cpu(cview(old, R, C), cview(lp, R, C), cview(white, R, C), cview(mask, R, C), 0.2f,
                                        -1.f, -1.f, 0.5f, CVERL_LOSS_AGG_TOKEN_MEAN, &res) != CVERL_OK);
}

// degenerate shapes and values: empty tensors, an all-zero mask, infinities - a status code, never a bad access
void rl_math_edges() {
  std::vector<float> one(1, 0.f), big(12);
  for (size_t i = 0; i < big.size(); ++i) big[i] = (i % 3 == 0) ? INFINITY : (i % 3 == 1 ? -1e30f : 1e30f);
  std::vector<float> zeros(12, 0.f), out(12), out2(12);
  std::vector<int64_t> groups(3, 0);
  float v = 0.f;
  for (int64_t r : {int64_t(0), int64_t(3)}) {
    for (int64_t c : {int64_t(0), int64_t(4)}) {
      const cverl_const_tensor2d_t x{big.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, r, c};
      const cverl_const_tensor2d_t m{zeros.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, r, c};
      const cverl_tensor2d_t o{out.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, r, c};
      const cverl_tensor2d_t o2{out2.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, r, c};
      (void)cverl_masked_sum_f32_cpu(x, m, &v);
      (void)cverl_masked_mean_f32_cpu(x, m, &v);
      (void)cverl_masked_whiten_f32_cpu(x, m, 1, o);
      (void)cverl_kl_penalty_f32_cpu(x, x, CVERL_KL_K3, o);
      (void)cverl_gae_advantage_return_f32_cpu(x, x, m, 1.0f, 0.95f, o, o2);
      (void)cverl_grpo_outcome_advantage_f32_cpu(x, m, groups.data(), 1e-6f, 1, o, o2);
      cverl_ppo_loss_result_t res{};
      (void)cverl_ppo_clipped_loss_f32_cpu(x, x, x, m, 0.2f, -1.f, -1.f, 3.0f, CVERL_LOSS_AGG_SEQ_MEAN_TOKEN_MEAN, &res);
      (void)cverl_ppo_clipped_loss_backward_f32_cpu(x, x, x, m, 0.2f, -1.f, -1.f, 3.0f, CVERL_LOSS_AGG_SEQ_MEAN_TOKEN_SUM, o);
    }
  }
  const cverl_const_tensor2d_t neg{one.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CPU, -1, 1};
  EXPECT(cverl_masked_sum_f32_cpu(neg, neg, &v) != CVERL_OK);
  const cverl_const_tensor2d_t cuda_view{one.data(), CVERL_DTYPE_F32, CVERL_DEVICE_CUDA, 1, 1};
  EXPECT(cverl_masked_sum_f32_cpu(cuda_view, cuda_view, &v) != CVERL_OK);   // a device view on the CPU entry point
}

void planner() {
  const int64_t dims[7] = {2, 2, 1, 2, 1, 1, 4};   // dp, pp, cp, tp, ep, sp, micro-batches
  int64_t coords[5];
  for (int64_t r = 0; r < 8; ++r) EXPECT(cverl_topology_coords(dims, 8, 8, r, coords) == 0);
  EXPECT(cverl_topology_coords(dims, 7, 8, 0, coords) != 0);
  int64_t ranks[8], count = 0;
  for (int axis = 0; axis < 4; ++axis) EXPECT(cverl_topology_group(dims, 8, 8, 3, axis, ranks, 8, &count) == 0);
  int64_t b = 0, e = 0;
  EXPECT(cverl_pipeline_layer_range(24, 4, 3, &b, &e) == 0 && e == 24);
  int32_t types[64];
  int64_t micro[64], n = 0, live = 0;
  EXPECT(cverl_pipeline_1f1b(1, 4, 8, types, micro, 64, &n, &live) == 0 && n == 16);
  EXPECT(cverl_pipeline_1f1b(1, 4, 8, types, micro, 3, &n, &live) != 0);          // capacity too small
  // many layouts, valid and not: every call must return (0 or an error), never touch memory past its capacities
  uint32_t s = 12345u;
  auto rnd = [&](int lo, int hi) { s = s * 1664525u + 1013904223u; return lo + static_cast<int>((s >> 10) % static_cast<uint32_t>(hi - lo + 1)); };
  for (int iter = 0; iter < 400; ++iter) {
    int64_t d[7] = {rnd(0, 3), rnd(0, 3), rnd(1, 2), rnd(1, 4), rnd(1, 2), 1, rnd(0, 6)};
    const int64_t prod = d[0] * d[1] * d[2] * d[3] * d[4];
    const int64_t w = rnd(0, 4) == 0 ? prod + rnd(-1, 1) : prod;
    const int64_t rank = rnd(-1, static_cast<int>(w > 0 ? w : 1));
    int64_t c5[5], out[4], cnt = 0;
    const int rc = cverl_topology_coords(d, w, rnd(1, 8), rank, c5);
    if (rc == 0) EXPECT(rank >= 0 && rank < w && w == prod);
    for (int axis = 0; axis < 5; ++axis) (void)cverl_topology_group(d, w, 8, rank, axis, out, rnd(0, 4), &cnt);
    int64_t lb = 0, le = 0;
    (void)cverl_pipeline_layer_range(rnd(0, 48), d[1], rnd(-1, 4), &lb, &le);
    int32_t t4[4];
    int64_t m4[4], n4 = 0, live4 = 0;
    (void)cverl_pipeline_1f1b(rnd(-1, 4), d[1], d[6], t4, m4, rnd(0, 4), &n4, &live4);
  }
  const int64_t numels[6] = {50, 10, 40, 30, 20, 60};
  int64_t owners[6];
  EXPECT(cverl_greedy_owners(numels, 6, 3, owners) == 0);
  EXPECT(cverl_greedy_owners(numels, 6, 0, owners) != 0);
}

void transport() {
  const std::string name = "/cverl_selftest_" + std::to_string(static_cast<long long>(getpid()));
  void* server = cverl_shm_transport_open(name.c_str(), 4096, 1);
  EXPECT(server != nullptr);
  if (!server) return;
  std::thread srv([&]() {
    std::vector<char> buf(4096);
    for (int i = 0; i < 50; ++i) {
      const int64_t n = cverl_shm_server_wait(server, buf.data(), 4096, 5000);
      EXPECT(n >= 0);
      if (n < 0) return;
      for (int64_t j = 0; j < n; ++j) buf[j] = static_cast<char>(buf[j] + 1);
      EXPECT(cverl_shm_server_reply(server, buf.data(), n, 0) == 0);
    }
  });
  void* client = cverl_shm_transport_open(name.c_str(), 4096, 0);
  EXPECT(client != nullptr);
  if (client) {
    std::vector<char> req(1000), resp(4096);
    for (int i = 0; i < 50; ++i) {
      for (size_t j = 0; j < req.size(); ++j) req[j] = static_cast<char>(i + j);
      const int64_t n = cverl_shm_client_call(client, req.data(), 1000, resp.data(), 4096, 5000);
      EXPECT(n == 1000);
      EXPECT(n == 1000 && resp[7] == static_cast<char>(req[7] + 1));
    }
    EXPECT(cverl_shm_client_call(client, req.data(), 5000, resp.data(), 4096, 100) == -1);   // request too large
  }
  srv.join();
  if (client) cverl_shm_transport_close(client);
  cverl_shm_transport_close(server);
}

void safetensors_round_trip() {
  const std::string path = "/tmp/cverl_selftest_" + std::to_string(static_cast<long long>(getpid())) + ".safetensors";
  std::vector<float> a(6);
  std::vector<int64_t> b(3);
  for (size_t i = 0; i < a.size(); ++i) a[i] = 0.5f * static_cast<float>(i);
  for (size_t i = 0; i < b.size(); ++i) b[i] = 7 - static_cast<int64_t>(i);
  const char* names[2] = {"layer.weight", "step \"q\""};
  const int dtypes[2] = {0, 3};       // F32, I64
  const int ndims[2] = {2, 1};
  const int64_t shapes[3] = {2, 3, 3};
  const void* data[2] = {a.data(), b.data()};
  EXPECT(cverl_st_write(path.c_str(), 2, names, dtypes, ndims, shapes, data) == 0);
  char err[256] = {0};
  void* h = cverl_st_open(path.c_str(), err, sizeof(err));
  EXPECT(h != nullptr);
  if (h) {
    EXPECT(cverl_st_count(h) == 2);
    EXPECT(cverl_st_name(h, 5) == nullptr);
    int dt = -1, nd = -1;
    int64_t shape8[8] = {0}, nbytes = 0;
    EXPECT(cverl_st_info(h, "layer.weight", &dt, &nd, shape8, &nbytes) == 0 && dt == 0 && nd == 2 && shape8[1] == 3 &&
           nbytes == 24);
    std::vector<float> back(6);
    EXPECT(cverl_st_read(h, "layer.weight", back.data(), 24) == 0 && back[5] == 2.5f);
    EXPECT(cverl_st_read(h, "layer.weight", back.data(), 20) != 0);       // wrong size: refused, nothing read
    EXPECT(cverl_st_info(h, "missing", &dt, &nd, shape8, &nbytes) != 0);
    cverl_st_close(h);
  }
  EXPECT(cverl_st_open("/tmp/cverl_selftest_no_such_file", err, sizeof(err)) == nullptr && err[0] != 0);
  std::remove(path.c_str());
  // a 24 MiB tensor read in pieces by three threads, a byte range of it, and ranges that are refused; the name
  // carries a control character (escaped on write) and the reader decodes it back
  std::vector<int32_t> big(6u << 20);
  for (size_t i = 0; i < big.size(); ++i) big[i] = static_cast<int32_t>(i * 2654435761u);
  const char* big_names[1] = {"big\ttensor"};
  const int big_dtypes[1] = {4}, big_ndims[1] = {1};
  const int64_t big_shape[1] = {static_cast<int64_t>(big.size())};
  const void* big_data[1] = {big.data()};
  EXPECT(cverl_st_write(path.c_str(), 1, big_names, big_dtypes, big_ndims, big_shape, big_data) == 0);
  h = cverl_st_open(path.c_str(), err, sizeof(err));
  EXPECT(h != nullptr);
  if (h) {
    const int64_t total = static_cast<int64_t>(big.size() * sizeof(int32_t));
    std::vector<int32_t> got(big.size());
    EXPECT(std::string(cverl_st_name(h, 0)) == "big\ttensor");
    EXPECT(cverl_st_read_range(h, "big\ttensor", 0, total, got.data(), 3) == 0 && got == big);
    std::fill(got.begin(), got.end(), 0);
    EXPECT(cverl_st_read(h, "big\ttensor", got.data(), total) == 0 && got == big);
    const int64_t off = 4 * 1000003, len = 4 * 2000001;
    EXPECT(cverl_st_read_range(h, "big\ttensor", off, len, got.data(), 2) == 0 &&
           std::memcmp(got.data(), big.data() + off / 4, static_cast<size_t>(len)) == 0);
    EXPECT(cverl_st_read_range(h, "big\ttensor", total - 8, 16, got.data(), 1) != 0);     // runs past the end
    EXPECT(cverl_st_read_range(h, "big\ttensor", -4, 8, got.data(), 1) != 0);
    EXPECT(cverl_st_read_range(h, "big\ttensor", 8, 0, got.data(), 4) == 0);              // empty range
    cverl_st_close(h);
  }
  std::remove(path.c_str());
}

void text_and_reward() {
  const char* text = "12 + 30 = 42";
  int64_t ids[8];
  const int64_t full = cverl_byte_encode(text, 12, 1, 1, 0, ids, 8);      // capacity smaller than the encoding
  EXPECT(full == 14 && ids[0] == 1 && ids[1] == 4 + '1');
  std::vector<int64_t> all(static_cast<size_t>(full));
  EXPECT(cverl_byte_encode(text, 12, 1, 1, 0, all.data(), full) == full);
  char out[32];
  const int64_t n = cverl_byte_decode(all.data(), full, 1, out, sizeof(out));
  EXPECT(n == 12 && std::memcmp(out, text, 12) == 0);
  EXPECT(cverl_byte_decode(all.data(), full, 0, out, 4) > 4);             // truncated write, full length returned
  char ans[64];
  EXPECT(cverl_gsm8k_extract("so the total is\n#### 1,234", 0, 0, ans, sizeof(ans)) == 1 && std::string(ans) == "1234");
  EXPECT(cverl_gsm8k_extract("no marker here", 0, 0, ans, sizeof(ans)) == 0);
  EXPECT(cverl_gsm8k_reward("#### 42", "#### 42", 0, 0, 1.0, 0.1, 0.0) == 1.0);
  EXPECT(cverl_gsm8k_reward("#### 41", "#### 42", 0, 0, 1.0, 0.1, 0.0) == 0.1);
  const std::string path = "/tmp/cverl_selftest_" + std::to_string(static_cast<long long>(getpid())) + ".jsonl";
  if (FILE* f = std::fopen(path.c_str(), "w")) {
    std::fputs("{\"prompt\": \"2+2?\", \"answer\": \"#### 4\"}\n{\"prompt\": \"a \\\"q\\\"\", \"answer\": \"x\"}\n", f);
    std::fclose(f);
    void* rows = cverl_jsonl_open(path.c_str(), "prompt", "answer", -1);
    EXPECT(rows != nullptr);
    if (rows) {
      EXPECT(cverl_jsonl_rows(rows) == 2);
      EXPECT(std::string(cverl_jsonl_get(rows, 0, 1)) == "#### 4");
      EXPECT(std::string(cverl_jsonl_get(rows, 1, 0)) == "a \"q\"");
      cverl_jsonl_close(rows);
    }
    void* none = cverl_jsonl_open(path.c_str(), "prompt", "answer", 0);      // 0 = no row, negative = all
    EXPECT(none != nullptr && cverl_jsonl_rows(none) == 0);
    if (none) cverl_jsonl_close(none);
    void* one = cverl_jsonl_open(path.c_str(), "prompt", "answer", 1);
    EXPECT(one != nullptr && cverl_jsonl_rows(one) == 1);
    if (one) cverl_jsonl_close(one);
    std::remove(path.c_str());
  }
}

// the rollout-batch builder on four threads (byte tokenizer): padding sides, truncation, reward placement, bad index
void rollout_batch() {
  const char* prompts[] = {"What is 2+2?", "unused", "hi"};
  const char* answers[] = {"#### 4", "0", "1"};
  const int64_t plen[] = {12, 6, 2};
  const char* responses[] = {"it is #### 4", "it is #### 5", "", "#### 1", "a much longer response than sixteen bytes #### 4"};
  int64_t rlen[5], sp[] = {0, 0, 2, 2, 0};
  for (int i = 0; i < 5; ++i) rlen[i] = static_cast<int64_t>(std::strlen(responses[i]));
  const int64_t given[] = {9, 8, 7}, goff[] = {0, 0, 0, 0, 3, 3};
  const uint8_t has[] = {0, 0, 0, 1, 0};
  const int64_t B = 5, P = 8, R = 16;
  std::vector<int64_t> pid(B * P), rid(B * R), gid(B);
  std::vector<float> mask(B * R), trew(B * R), rew(B);
  EXPECT(cverl_build_gsm8k_rollout_batch(0, nullptr, 0, prompts, plen, answers, 3, sp, responses, rlen, given, goff, has,
                                         B, P, R, 0, 1, 1, 2, 0, 300, 1.0, 0.0, 0.0, 4, pid.data(), rid.data(),
                                         mask.data(), trew.data(), rew.data(), gid.data()) == 0);
  EXPECT(rew[0] == 1.0f && rew[1] == 0.0f && rew[2] == 0.0f && rew[3] == 1.0f && rew[4] == 1.0f);
  EXPECT(pid[0] == 4 + 'W' && pid[7] == 4 + ' ');                       // first 8 bytes of the 12-byte prompt
  EXPECT(pid[2 * P] == 0 && pid[2 * P + 6] == 4 + 'h');                 // left padded
  EXPECT(rid[12] == 2 && mask[12] == 1.0f && mask[13] == 0.0f && trew[12] == 1.0f);   // 12 bytes, then the EOS
  EXPECT(rid[2 * R] == 2 && mask[2 * R] == 1.0f && mask[2 * R + 1] == 0.0f);          // empty text: the EOS alone
  EXPECT(rid[3 * R] == 9 && rid[3 * R + 2] == 7 && mask[3 * R + 2] == 1.0f && mask[3 * R + 3] == 0.0f);
  EXPECT(trew[3 * R + 2] == 1.0f && trew[4 * R + R - 1] == 1.0f && mask[4 * R + R - 1] == 1.0f);
  EXPECT(rid[4 * R + R - 1] == 4 + 'e');                                // cut at 16 bytes: no room for an EOS
  EXPECT(gid[2] == 2 && gid[4] == 0);
  EXPECT(cverl_build_gsm8k_rollout_batch(0, nullptr, 0, prompts, plen, answers, 3, sp, responses, rlen, given, goff, has,
                                         B, P, R, 1, 0, 1, 2, 0, 300, 1.0, 0.0, 0.0, 2, pid.data(), rid.data(),
                                         mask.data(), trew.data(), rew.data(), gid.data()) == 0);
  EXPECT(pid[0] == 1 && pid[1] == 4 + 'W' && mask[2 * R] == 0.0f && mask[12] == 0.0f);   // BOS in front, no EOS
  sp[1] = 3;                                                            // prompt index out of range
  EXPECT(cverl_build_gsm8k_rollout_batch(0, nullptr, 0, prompts, plen, answers, 3, sp, responses, rlen, nullptr, nullptr,
                                         nullptr, B, P, R, 0, 1, 1, 2, 0, 300, 1.0, 0.0, 0.0, 4, pid.data(), rid.data(),
                                         mask.data(), trew.data(), rew.data(), gid.data()) == 1);
  EXPECT(cverl_build_gsm8k_rollout_batch(1, nullptr, 0, prompts, plen, answers, 3, sp, responses, rlen, nullptr, nullptr,
                                         nullptr, B, P, R, 0, 1, 1, 2, 0, 300, 1.0, 0.0, 0.0, 4, pid.data(), rid.data(),
                                         mask.data(), trew.data(), rew.data(), gid.data()) == 1);   // BPE without a handle
}

// argv[1] (optional): a Hugging Face tokenizer.json; encode / decode round trips from two threads sharing one handle
void bpe(const char* tokenizer_json) {
  char err[256] = {0};
  void* h = cverl_bpe_open(tokenizer_json, err, sizeof(err));
  EXPECT(h != nullptr);
  if (!h) {
    std::fprintf(stderr, "bpe: %s\n", err);
    return;
  }
  EXPECT(cverl_bpe_vocab_size(h) > 0);
  auto work = [&](const char* text) {
    const int64_t len = static_cast<int64_t>(std::strlen(text));
    std::vector<int64_t> ids(256);
    const int64_t n = cverl_bpe_encode(h, text, len, ids.data(), 256);
    EXPECT(n > 0 && n <= 256);
    std::vector<char> out(512);
    const int64_t m = cverl_bpe_decode(h, ids.data(), n, 1, out.data(), 512);
    EXPECT(m == len && std::memcmp(out.data(), text, static_cast<size_t>(len)) == 0);
    int64_t two[2];
    EXPECT(cverl_bpe_encode(h, text, len, two, 2) == n);            // capacity smaller than the encoding
  };
  std::thread t1(work, "hello world, 123 + 456 = 579"), t2(work, "the quick brown fox\n  jumps");
  t1.join();
  t2.join();
  // batch encoding on four threads while a fifth thread encodes through the same handle: the batch must give
  // what one-by-one encoding gives, also when the output buffer is too small (count only) or the batch is empty
  const char* texts[] = {"hello world", "the quick brown fox", "", "123 + 456 = 579", "hello hello hello", "  \n\n x"};
  const int64_t n_texts = 6;
  int64_t lens[6], offsets[7], small_offsets[7];
  for (int i = 0; i < n_texts; ++i) lens[i] = static_cast<int64_t>(std::strlen(texts[i]));
  std::vector<int64_t> flat(512);
  std::thread side(work, "side thread: while the batch runs");
  const int64_t total = cverl_bpe_encode_batch(h, texts, lens, n_texts, 4, flat.data(), 512, offsets);
  side.join();
  EXPECT(total > 0 && total <= 512 && offsets[0] == 0 && offsets[n_texts] == total && offsets[2] == offsets[3]);
  for (int i = 0; i < n_texts; ++i) {
    std::vector<int64_t> one(256);
    const int64_t n = cverl_bpe_encode(h, texts[i], lens[i], one.data(), 256);
    EXPECT(n == offsets[i + 1] - offsets[i]);
    EXPECT(std::memcmp(one.data(), flat.data() + offsets[i], static_cast<size_t>(n) * sizeof(int64_t)) == 0);
  }
  int64_t tiny[3];
  EXPECT(cverl_bpe_encode_batch(h, texts, lens, n_texts, 2, tiny, 3, small_offsets) == total);
  EXPECT(cverl_bpe_encode_batch(h, texts, lens, 0, 2, tiny, 3, small_offsets) == 0 && small_offsets[0] == 0);
  cverl_bpe_close(h);
  EXPECT(cverl_bpe_open("/tmp/cverl_selftest_no_such_tokenizer.json", err, sizeof(err)) == nullptr);
}

// argv[2] (optional): a rollout-worker plugin (.so): load, generate into caller buffers, walk the parameters, unload
void plugin(const char* so_path) {
  char err[256] = {0};
  void* h = cverl_plugin_load(so_path, "{\"vocab_size\": 32}", err, sizeof(err));
  EXPECT(h != nullptr);
  if (!h) {
    std::fprintf(stderr, "plugin: %s\n", err);
    return;
  }
  const int64_t B = 2, P = 4, N = 3;
  std::vector<int64_t> ids(B * P, 5), mask(B * P, 1), lens(B, P), out_ids(B * N, -1), out_len(B, -1);
  std::vector<float> out_lp(B * N, 1.f);
  cverl_generate_args_t a{};
  a.token_ids = ids.data();
  a.attention_mask = mask.data();
  a.lengths = lens.data();
  a.batch = B;
  a.prompt_len = P;
  a.config.max_new_tokens = N;
  a.config.temperature = 1.0;
  a.config.top_p = 1.0;
  a.config.eos_token_id = -1;
  a.config.seed = 7;
  a.out_token_ids = out_ids.data();
  a.out_logprobs = out_lp.data();
  a.out_lengths = out_len.data();
  EXPECT(cverl_plugin_generate(h, &a) == 0);
  for (int64_t b = 0; b < B; ++b) EXPECT(out_len[b] >= 0 && out_len[b] <= N);
  const int64_t np = cverl_plugin_num_parameters(h);
  EXPECT(np >= 0);
  cverl_parameter_view_t view{};
  for (int64_t i = 0; i < np; ++i) EXPECT(cverl_plugin_parameter(h, i, &view) == 0 && view.name != nullptr);
  EXPECT(cverl_plugin_parameter(h, np, &view) != 0);                       // one past the end
  cverl_plugin_unload(h);
  EXPECT(cverl_plugin_load("/tmp/cverl_selftest_no_such_plugin.so", "{}", err, sizeof(err)) == nullptr && err[0] != 0);
}

}  // namespace

int main(int argc, char** argv) {
  if (argc > 1) bpe(argv[1]);
  if (argc > 2) plugin(argv[2]);
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < 4; ++t) pool.emplace_back(rl_math, t);
  planner();
  rl_math_edges();
  rollout_batch();
  for (auto& th : pool) th.join();
  safetensors_round_trip();
  text_and_reward();
  transport();
  if (g_failures) {
    std::fprintf(stderr, "%d checks failed\n", g_failures);
    return 1;
  }
  std::puts("host self-test passed");
  return 0;
}
