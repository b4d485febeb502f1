// Loads a prompt / answer JSONL file with the reference's load_prompt_answer_jsonl
// (include/cverl/data/hf_dataset.h:11-16,42) and prints the rows as one JSON array of [prompt, answer] pairs, or
// {"error": "..."} when it refuses the file.  Linked against the unmodified reference library.
//   ref_jsonl_check FILE.jsonl PROMPT_FIELD ANSWER_FIELD MAX_EXAMPLES
#include <iostream>

#include <nlohmann/json.hpp>

#include "cverl/data/hf_dataset.h"

int main(int argc, char** argv) {
  if (argc < 5) return 2;
  nlohmann::json out;
  try {
    cverl::data::JsonlDatasetOptions o;
    o.path = argv[1];
    o.prompt_field = argv[2];
    o.answer_field = argv[3];
    o.max_examples = std::stoll(argv[4]);
    out = nlohmann::json::array();
    for (const auto& ex : cverl::data::load_prompt_answer_jsonl(o)) out.push_back({ex.prompt, ex.answer});
  } catch (const std::exception& e) {
    out = nlohmann::json{{"error", e.what()}};
  }
  std::cout << out.dump() << "\n";
  return 0;
}
