// Test fixture: a deterministic rollout-worker plugin.  Token t of row b is
// (last prompt token + t + 1) % vocab, log-prob -0.5; "vocab" and "eos_after" come from the
// config JSON; it owns one fp32 parameter of four elements.
#include "cverl/rollout_plugin.h"

#include <cstdlib>
#include <cstring>
#include <string>

namespace {
struct Fixture {
  cverl_rollout_worker_t api;
  int64_t vocab = 100;
  int64_t eos_after = -1;
  float weights[4] = {1.f, 2.f, 3.f, 4.f};
  int64_t generate_calls = 0;
};
int64_t json_i64(const std::string& s, const char* key, int64_t fallback) {
  const std::string k = std::string("\"") + key + "\"";
  const size_t at = s.find(k);
  if (at == std::string::npos) return fallback;
  const size_t colon = s.find(':', at);
  return colon == std::string::npos ? fallback : std::strtoll(s.c_str() + colon + 1, nullptr, 10);
}
int generate(void* self, const cverl_generate_args_t* a) {
  auto* f = static_cast<Fixture*>(self);
  ++f->generate_calls;
  const int64_t n = a->config.max_new_tokens;
  for (int64_t b = 0; b < a->batch; ++b) {
    const int64_t last = a->token_ids[b * a->prompt_len + a->prompt_len - 1];
    int64_t len = 0;
    for (int64_t t = 0; t < n; ++t) {
      const bool stop = f->eos_after >= 0 && t >= f->eos_after;
      a->out_token_ids[b * n + t] = stop ? a->config.eos_token_id : (last + t + 1) % f->vocab;
      a->out_logprobs[b * n + t] = -0.5f;
      ++len;
      if (stop) break;
    }
    for (int64_t t = len; t < n; ++t) a->out_token_ids[b * n + t] = 0, a->out_logprobs[b * n + t] = 0.f;
    a->out_lengths[b] = len;
  }
  return 0;
}
int64_t num_parameters(void*) { return 1; }
int parameter(void* self, int64_t index, cverl_parameter_view_t* out) {
  if (index != 0) return 1;
  auto* f = static_cast<Fixture*>(self);
  out->name = "fixture.weight";
  out->data = f->weights;
  out->dtype = 0;
  out->device = 0;
  out->ndim = 1;
  out->shape[0] = 4;
  return 0;
}
}  // namespace

extern "C" cverl_rollout_worker_t* cverl_create_rollout_worker(const char* config_json) {
  auto* f = new Fixture();
  const std::string cfg = config_json ? config_json : "";
  if (cfg.find("\"fail\"") != std::string::npos) {
    delete f;
    return nullptr;
  }
  f->vocab = json_i64(cfg, "vocab", 100);
  f->eos_after = json_i64(cfg, "eos_after", -1);
  f->api.self = f;
  f->api.generate = generate;
  f->api.num_parameters = num_parameters;
  f->api.parameter = parameter;
  return &f->api;
}

extern "C" void cverl_destroy_rollout_worker(cverl_rollout_worker_t* worker) {
  if (worker) delete static_cast<Fixture*>(worker->self);
}
