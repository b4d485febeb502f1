// Stand-alone exercise of the host runtime's C ABI, meant to be built with -fsanitize=address,undefined or
// -fsanitize=thread (python -m cverl_b200._build --sanitize address|thread) and run on a CPU box:
//   * the RL math entry points on ragged masks, from several threads at once (they share no state);
//   * argument validation paths (null data, shape mismatch) that must return an error, not touch memory;
//   * the topology planner, 1F1B schedule and greedy owner assignment;
//   * the shared-memory request / response transport with a server thread and a client thread.
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
#include "cverl/topology.h"

extern "C" {
void* cverl_shm_transport_open(const char* name, int64_t payload_capacity, int create);
void cverl_shm_transport_close(void* h);
int64_t cverl_shm_client_call(void* h, const void* request, int64_t request_size, void* response,
                              int64_t response_capacity, int64_t timeout_ms);
int64_t cverl_shm_server_wait(void* h, void* request, int64_t capacity, int64_t timeout_ms);
int cverl_shm_server_reply(void* h, const void* response, int64_t size, int status);
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

}  // namespace

int main() {
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < 4; ++t) pool.emplace_back(rl_math, t);
  planner();
  for (auto& th : pool) th.join();
  transport();
  if (g_failures) {
    std::fprintf(stderr, "%d checks failed\n", g_failures);
    return 1;
  }
  std::puts("host self-test passed");
  return 0;
}
