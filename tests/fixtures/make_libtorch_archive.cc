// Writes tests/fixtures/libtorch_output_archive.pt: a tensor archive produced by LibTorch's own
// torch::serialize::OutputArchive, with the key names of a flat-optimizer rank file.  The Python
// checkpoint reader is tested against this file, so that a checkpoint written by a C++ LibTorch
// trainer (tensors stored as module parameters, not buffers) is known to load.
//
//   g++ -std=c++17 make_libtorch_archive.cc -I<torch>/include -I<torch>/include/torch/csrc/api/include \
//       -L<torch>/lib -ltorch -ltorch_cpu -lc10 -Wl,-rpath,<torch>/lib -o make_archive && ./make_archive out.pt
#include <torch/torch.h>

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  torch::serialize::OutputArchive archive;
  auto shard = torch::arange(8, torch::kFloat32).mul(0.25).to(torch::kBFloat16);
  archive.write("flat_param_shard", shard);
  archive.write("flat_exp_avg", torch::arange(8, torch::kFloat32).mul(0.5));
  archive.write("flat_exp_avg_sq", torch::arange(8, torch::kFloat32).mul(2.0));
  archive.write("param_0", torch::arange(6, torch::kFloat32).view({2, 3}).to(torch::kBFloat16));
  archive.write("optim_step", torch::tensor(static_cast<int64_t>(3), torch::kInt64));
  archive.save_to(argv[1]);
  return 0;
}
