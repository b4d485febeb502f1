// Reads a tensor archive written by cverl_b200.utils.checkpoint.save_archive with LibTorch's own
// torch::serialize::InputArchive - the reader the reference's trainer resumes with
// (tools/model/qwen3_5_pp_tp_ppo_trainer.cc:1274-1396) - and prints one line per requested key:
//   <key> <dtype> <numel> <sum as double>
//
//   g++ -std=c++17 read_archive_with_libtorch.cc -I<torch>/include -I<torch>/include/torch/csrc/api/include \
//       -L<torch>/lib -ltorch -ltorch_cpu -lc10 -Wl,-rpath,<torch>/lib -o read_archive
//   ./read_archive rank_0.pt flat_param_shard flat_exp_avg optim_step
#include <torch/torch.h>

#include <iostream>

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  try {
    torch::serialize::InputArchive archive;
    archive.load_from(argv[1]);
    for (int i = 2; i < argc; ++i) {
      torch::Tensor t;
      archive.read(argv[i], t);
      std::cout << argv[i] << " " << t.dtype() << " " << t.numel() << " " << t.to(torch::kFloat64).sum().item<double>()
                << "\n";
    }
  } catch (const std::exception& e) {
    std::cerr << "read failed: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
