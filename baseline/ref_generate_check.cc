// Greedy generation with the reference's PolicyRolloutWorker (include/cverl/rollout/policy_worker.h:18-32: the full
// forward is run again for every new token) over its Qwen3_5CausalLmPolicy, printed as JSON for comparison with
// this package's cached decode.  Linked against the unmodified reference library.
//   ref_generate_check MODEL_DIR "1,2,3;4,5,6" MAX_NEW_TOKENS EOS_ID EOS_CHECK_INTERVAL
#include <iostream>
#include <sstream>

#include <nlohmann/json.hpp>
#include <torch/torch.h>

#include "cverl/rollout/policy_worker.h"
#include "cverl/torch/causal_lm_policy.h"

int main(int argc, char** argv) {
  if (argc < 6) return 2;
  try {
    torch::NoGradGuard no_grad;
    cverl::torch_backend::CausalLmPolicyOptions options;
    options.kind = cverl::torch_backend::CausalLmPolicyOptions::Kind::kQwen3_5;
    options.qwen_model_dir = argv[1];
    options.param_dtype = torch::kFloat32;
    auto policy = cverl::torch_backend::make_causal_lm_policy(options);
    std::vector<std::vector<int64_t>> rows;
    std::stringstream all(argv[2]);
    std::string row;
    while (std::getline(all, row, ';')) {
      std::vector<int64_t> ids;
      std::stringstream ss(row);
      std::string item;
      while (std::getline(ss, item, ','))
        if (!item.empty()) ids.push_back(std::stoll(item));
      rows.push_back(ids);
    }
    const int64_t B = static_cast<int64_t>(rows.size()), T = static_cast<int64_t>(rows[0].size());
    auto ids = torch::empty({B, T}, torch::kLong);
    for (int64_t b = 0; b < B; ++b)
      for (int64_t t = 0; t < T; ++t) ids[b][t] = rows[static_cast<size_t>(b)][static_cast<size_t>(t)];
    cverl::rollout::TokenBatch batch;
    batch.token_ids = ids;
    cverl::rollout::GenerationConfig cfg;
    cfg.max_new_tokens = std::stoll(argv[3]);
    cfg.temperature = 0.0;
    cfg.eos_token_id = std::stoll(argv[4]);
    cfg.eos_check_interval = std::stoll(argv[5]);
    cverl::rollout::PolicyRolloutWorker worker(policy);
    auto out = worker.generate(batch, cfg);
    auto flat_i = [](const torch::Tensor& t) {
      auto c = t.to(torch::kCPU).to(torch::kLong).contiguous().view({-1});
      return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
    };
    auto lp = out.logprobs.to(torch::kCPU).to(torch::kFloat32).contiguous().view({-1});
    nlohmann::json j;
    j["token_ids"] = flat_i(out.token_ids);
    j["shape"] = {out.token_ids.size(0), out.token_ids.size(1)};
    j["logprobs"] = std::vector<float>(lp.data_ptr<float>(), lp.data_ptr<float>() + lp.numel());
    if (out.lengths.defined()) j["lengths"] = flat_i(out.lengths);
    j["pad_id"] = policy->pad_id();
    std::cout << j.dump() << "\n";
  } catch (const std::exception& e) {
    std::cerr << "failed: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
