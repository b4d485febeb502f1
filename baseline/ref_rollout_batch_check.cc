// Runs the reference's build_gsm8k_rollout_batch (include/cverl/rollout/rollout_batch.h:44-49) with its byte
// tokenizer or its BPE tokenizer on cases given as JSON, and prints the six tensors as JSON for comparison with
// this package's builder.  Linked against the unmodified reference library.
//   ref_rollout_batch_check CASES.json [TOKENIZER.json]  >  OUT.json
// CASES.json: {"prompts": [...], "answers": [...], "samples": [{"prompt_index": i, "text": "...", "token_ids": [...]}],
//              "max_prompt_tokens": P, "max_response_tokens": R, "method": "strict"|"flexible", "add_eos": bool}
#include <fstream>
#include <iostream>
#include <memory>

#include <nlohmann/json.hpp>
#include <torch/torch.h>

#include "cverl/rollout/rollout_batch.h"
#include "cverl/text/byte_tokenizer.h"
#include "cverl/text/hf_bpe_tokenizer.h"

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  try {
    std::ifstream f(argv[1]);
    nlohmann::json in = nlohmann::json::parse(f);
    std::unique_ptr<cverl::text::Tokenizer> tok;
    if (argc > 2) {
      cverl::text::HfBpeTokenizerOptions o;
      o.tokenizer_json_path = argv[2];
      tok = std::make_unique<cverl::text::HfBpeTokenizer>(o);
    } else {
      tok = std::make_unique<cverl::text::ByteTokenizer>();
    }
    cverl::rollout::RolloutResponse response;
    for (const auto& s : in["samples"]) {
      cverl::rollout::RolloutSequence seq;
      seq.prompt_index = s["prompt_index"].get<size_t>();
      seq.text = s["text"].get<std::string>();
      for (const auto& t : s["token_ids"]) seq.token_ids.push_back(t.get<int32_t>());
      response.sequences.push_back(seq);
    }
    cverl::reward::Gsm8kRewardOptions ro;
    ro.method = in["method"].get<std::string>() == "flexible" ? cverl::reward::Gsm8kExtractionMethod::Flexible
                                                              : cverl::reward::Gsm8kExtractionMethod::Strict;
    cverl::rollout::RolloutBatchOptions bo;
    bo.max_prompt_tokens = in["max_prompt_tokens"].get<int64_t>();
    bo.max_response_tokens = in["max_response_tokens"].get<int64_t>();
    bo.add_eos = in["add_eos"].get<bool>();
    auto b = cverl::rollout::build_gsm8k_rollout_batch(response, in["prompts"].get<std::vector<std::string>>(),
                                                       in["answers"].get<std::vector<std::string>>(), ro, *tok, bo);
    auto vec_i = [](const torch::Tensor& t) {
      auto c = t.contiguous().view({-1});
      return std::vector<int64_t>(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + c.numel());
    };
    auto vec_f = [](const torch::Tensor& t) {
      auto c = t.contiguous().view({-1});
      return std::vector<float>(c.data_ptr<float>(), c.data_ptr<float>() + c.numel());
    };
    nlohmann::json out;
    out["pad_id"] = tok->pad_id();
    out["prompt_ids"] = vec_i(b.prompt_ids);
    out["response_ids"] = vec_i(b.response_ids);
    out["response_mask"] = vec_f(b.response_mask);
    out["group_ids"] = vec_i(b.group_ids);
    out["rewards"] = vec_f(b.scalar_rewards);
    out["token_rewards"] = vec_f(b.token_rewards);
    std::cout << out.dump() << "\n";
  } catch (const std::exception& e) {
    std::cerr << "failed: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
