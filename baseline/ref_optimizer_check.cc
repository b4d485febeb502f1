// Five steps of the reference's optimizers (include/cverl/torch/fp32_master_adamw.h:14-79) on data both sides can
// state exactly - parameter p[i] = sin(0.37 i), gradient of step k g[i] = cos(0.11 i + k) / 3 - in the four modes
// {FlatAdamW, Fp32MasterAdamW} x {fp32 master weights, bf16 parameters without master copy}; the final parameters
// and moments are written with the reference's own safetensors writer.  Linked against the reference library.
//   ref_optimizer_check OUT.safetensors
#include <iostream>
#include <unordered_map>

#include <torch/torch.h>

#include "cverl/model/safetensors_writer.h"
#include "cverl/torch/fp32_master_adamw.h"

using cverl::torch_backend::FlatAdamW;
using cverl::torch_backend::Fp32MasterAdamW;
using cverl::torch_backend::Fp32MasterAdamWOptions;

static torch::Tensor param0(int64_t n) { return torch::sin(torch::arange(n, torch::kFloat32) * 0.37); }
static torch::Tensor grad_at(int64_t n, int k) { return torch::cos(torch::arange(n, torch::kFloat32) * 0.11 + k) / 3.0; }

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  try {
    const int64_t n = 1000;
    std::unordered_map<std::string, torch::Tensor> out;
    for (int master = 0; master < 2; ++master) {
      Fp32MasterAdamWOptions o;
      o.lr = 1.0e-2;
      o.beta1 = 0.9;
      o.beta2 = 0.95;
      o.eps = 1.0e-8;
      o.weight_decay = 0.01;
      o.use_master_weights = master != 0;
      const std::string tag = master ? "master" : "bf16";
      {  // flat shard
        auto p = master ? param0(n) : param0(n).to(torch::kBFloat16);
        FlatAdamW opt(p, o);
        for (int k = 0; k < 5; ++k) opt.step(grad_at(n, k));
        out["flat." + tag + ".param"] = opt.parameter_shard().to(torch::kFloat32);
        out["flat." + tag + ".exp_avg"] = opt.exp_avg();
        out["flat." + tag + ".exp_avg_sq"] = opt.exp_avg_sq();
      }
      {  // per-tensor: two tensors, gradients accumulated from .grad into the fp32 main gradient
        auto a = param0(n).slice(0, 0, 600).clone().to(torch::kBFloat16).requires_grad_(true);
        auto b = param0(n).slice(0, 600, n).clone().to(torch::kBFloat16).view({20, 20}).requires_grad_(true);
        Fp32MasterAdamW opt({a, b}, o);
        for (int k = 0; k < 5; ++k) {
          auto g = grad_at(n, k);
          a.mutable_grad() = g.slice(0, 0, 600).to(torch::kBFloat16);
          b.mutable_grad() = g.slice(0, 600, n).view({20, 20}).to(torch::kBFloat16);
          opt.accumulate_model_grads();
          opt.step();
          opt.zero_grad();
        }
        out["tensorwise." + tag + ".a"] = a.detach().to(torch::kFloat32);
        out["tensorwise." + tag + ".b"] = b.detach().to(torch::kFloat32);
        out["tensorwise." + tag + ".exp_avg_sq_b"] = opt.exp_avg_sq()[1];
      }
    }
    cverl::write_safetensors(argv[1], out, "float32");
    std::cout << "tensors=" << out.size() << "\n";
  } catch (const std::exception& e) {
    std::cerr << "failed: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
