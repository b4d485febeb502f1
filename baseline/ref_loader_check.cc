// Loads a model directory with the reference's own HfModelLoader (its public class,
// include/cverl/model/hf_model_loader.h:32-42) and prints the tensor count, the element count and the sum of
// absolute values - what baseline/ref_loader_check.py compares with this package's reader on a directory this
// package wrote.  Linked against the unmodified reference object that baseline/build_ref.py compiled.
//   ref_loader_check MODEL_DIR
#include "cverl/model/hf_model_loader.h"
#include <iostream>
int main(int argc, char** argv) {
  try {
    cverl::HfModelLoader loader(argv[1]);
    loader.load_metadata();
    const auto& cfg = loader.config();
    std::cout << "model_type=" << cfg.model_type << " layers=" << cfg.num_hidden_layers << " tensors=" << loader.tensors().size() << "\n";
    double total = 0; size_t n = 0;
    for (const auto& t : loader.tensors()) {
      auto x = loader.load_tensor(t.name);
      total += x.to(torch::kFloat64).abs().sum().item<double>(); n += x.numel();
    }
    std::cout.precision(14);
    std::cout << "numel=" << n << " abs_sum=" << total << "\n";
  } catch (const std::exception& e) { std::cerr << "failed: " << e.what() << "\n"; return 1; }
  return 0;
}
