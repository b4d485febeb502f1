// Gradients of the reference's Qwen3_5CausalLmPolicy (its public class through make_causal_lm_policy,
// include/cverl/torch/causal_lm_policy.h:31-84) for a weighted negative log-likelihood of given response tokens,
// written as a safetensors file (the reference's own write_safetensors) for comparison with this package's
// backward pass.  Linked against the unmodified reference library.
//   ref_backward_check MODEL_DIR PROMPT_IDS RESPONSE_IDS OUT.safetensors      (ids: comma separated)
// loss = - sum_t (0.5 + 0.1 t) * log p(response[t] | prompt, response[:t])
#include <iostream>
#include <sstream>
#include <unordered_map>

#include <torch/torch.h>

#include "cverl/model/safetensors_writer.h"
#include "cverl/torch/causal_lm_policy.h"

static torch::Tensor parse_ids(const std::string& text) {
  std::vector<int64_t> v;
  std::stringstream ss(text);
  std::string item;
  while (std::getline(ss, item, ','))
    if (!item.empty()) v.push_back(std::stoll(item));
  return torch::tensor(v, torch::kLong).view({1, static_cast<int64_t>(v.size())});
}

int main(int argc, char** argv) {
  if (argc < 5) return 2;
  try {
    cverl::torch_backend::CausalLmPolicyOptions options;
    options.kind = cverl::torch_backend::CausalLmPolicyOptions::Kind::kQwen3_5;
    options.qwen_model_dir = argv[1];
    options.param_dtype = torch::kFloat32;
    auto policy = cverl::torch_backend::make_causal_lm_policy(options);
    const auto prompt = parse_ids(argv[2]), response = parse_ids(argv[3]);
    auto logits = policy->forward(prompt, response);                                  // [1, R, V] fp32
    auto lp = torch::log_softmax(logits.to(torch::kFloat32), -1).gather(-1, response.unsqueeze(-1)).squeeze(-1);
    auto w = torch::arange(response.size(1), torch::kFloat32).mul(0.1).add(0.5).view({1, -1});
    auto loss = -(lp * w).sum();
    loss.backward();
    std::unordered_map<std::string, torch::Tensor> grads;
    for (const auto& kv : policy->named_parameters()) {
      std::string name = kv.key();
      for (auto& c : name)
        if (c == '/') c = '.';
      if (kv.value().grad().defined()) grads[name] = kv.value().grad().detach().to(torch::kFloat32);
    }
    cverl::write_safetensors(argv[4], grads, "float32");
    std::cout.precision(12);
    std::cout << "loss=" << loss.item<double>() << " parameters=" << grads.size() << "\n";
  } catch (const std::exception& e) {
    std::cerr << "failed: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
