// cverl_parallel_plan: prints the rank coordinates, every group, pipeline peers, layer range, the
// 1F1B schedule and the NCCL environment of one rank (reference CLI: tools/distributed/cverl_parallel_plan.cc).
//   cverl_parallel_plan --dp 2 --pp 2 --tp 2 --rank 5 --layers 24 --micro-batches 4
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <string>

#include "cverl/topology.h"

static int64_t arg_i64(int argc, char** argv, const char* name, int64_t fallback) {
  for (int i = 1; i + 1 < argc; ++i)
    if (std::strcmp(argv[i], name) == 0) return std::strtoll(argv[i + 1], nullptr, 10);
  return fallback;
}
static void print_group(const char* name, const std::vector<int64_t>& g) {
  std::printf("%s_group=[", name);
  for (size_t i = 0; i < g.size(); ++i) std::printf("%s%lld", i ? "," : "", static_cast<long long>(g[i]));
  std::printf("]\n");
}

static bool has_flag(int argc, char** argv, const char* name) {
  for (int i = 1; i < argc; ++i)
    if (std::strcmp(argv[i], name) == 0) return true;
  return false;
}

static void print_rank(const cverl::Topology& topo, const cverl::ParallelDims& d, int64_t rank, int64_t layers,
                       bool schedule) {
  auto info = topo.rank_info(rank);
  std::printf("rank=%lld dp=%lld pp=%lld cp=%lld tp=%lld ep=%lld sp=%lld\n", (long long)info.global_rank,
              (long long)info.data_rank, (long long)info.pipeline_rank, (long long)info.context_rank,
              (long long)info.tensor_rank, (long long)info.expert_rank, (long long)info.sequence_rank);
  print_group("data", info.data_group);
  print_group("pipeline", info.pipeline_group);
  print_group("context", info.context_group);
  print_group("tensor", info.tensor_group);
  print_group("expert", info.expert_group);
  print_group("sequence", info.sequence_group);
  print_group("model", info.model_group);
  auto peers = cverl::pipeline_peers(info.pipeline_group, info.pipeline_rank);
  std::printf("pipeline_prev=%lld pipeline_next=%lld\n", (long long)peers.prev_rank, (long long)peers.next_rank);
  if (layers > 0) {
    auto range = topo.pipeline_layer_range(layers, info.pipeline_rank);
    std::printf("layer_begin=%lld layer_end=%lld\n", (long long)range.first, (long long)range.second);
  }
  auto sched = cverl::pipeline_1f1b_schedule(info.pipeline_rank, d.pipeline, d.micro_batches);
  if (schedule) {
    std::printf("schedule=");
    for (const auto& a : sched)
      std::printf("%c%lld ", a.type == cverl::PipelineActionType::Forward ? 'F' : 'B', (long long)a.micro_batch);
    std::printf("\n");
  }
  std::printf("max_live_activations=%lld\n",
              (long long)cverl::pipeline_schedule_max_live_activations(sched, d.micro_batches));
}

int main(int argc, char** argv) {
  if (has_flag(argc, argv, "--help") || has_flag(argc, argv, "-h")) {
    std::printf("usage: cverl_parallel_plan --dp D --tp T --pp P --cp C [--ep E] [--sp S] [--micro-batches M] [--rank R]\n"
                "         [--world-size W] [--local-rank L] [--local-world-size LW] [--gpus-per-node G]\n"
                "         [--num-layers N | --layers N] [--all-ranks] [--no-schedule]\n"
                "Prints the coordinates, groups, pipeline peers, layer range, 1F1B schedule and peak live activations\n"
                "of one rank (or of every rank with --all-ranks), then the NCCL environment of the layout.\n");
    return 0;
  }
  try {
    cverl::ParallelDims d;
    d.data = arg_i64(argc, argv, "--dp", 1);
    d.pipeline = arg_i64(argc, argv, "--pp", 1);
    d.context = arg_i64(argc, argv, "--cp", 1);
    d.tensor = arg_i64(argc, argv, "--tp", 1);
    d.expert = arg_i64(argc, argv, "--ep", 1);
    d.sequence = arg_i64(argc, argv, "--sp", 1);
    d.micro_batches = arg_i64(argc, argv, "--micro-batches", d.pipeline);
    cverl::ClusterSpec c = cverl::cluster_spec_from_env();
    c.world_size = arg_i64(argc, argv, "--world-size", d.world());
    c.rank = arg_i64(argc, argv, "--rank", c.rank);
    c.local_rank = arg_i64(argc, argv, "--local-rank", c.local_rank);
    c.local_world_size = arg_i64(argc, argv, "--local-world-size", c.local_world_size);
    c.gpus_per_node = arg_i64(argc, argv, "--gpus-per-node", 8);
    // --num-layers is the reference's spelling, --layers this tool's older one
    const int64_t layers = arg_i64(argc, argv, "--num-layers", arg_i64(argc, argv, "--layers", 24));
    const bool schedule = !has_flag(argc, argv, "--no-schedule");      // --schedule is accepted and is the default
    cverl::Topology topo(d, c);
    std::printf("world_size=%lld\n", (long long)d.world());
    std::printf("parallel=dp%lld_pp%lld_cp%lld_tp%lld_ep%lld_sp%lld\n", (long long)d.data, (long long)d.pipeline,
                (long long)d.context, (long long)d.tensor, (long long)d.expert, (long long)d.sequence);
    std::printf("micro_batches=%lld\n", (long long)d.micro_batches);
    if (has_flag(argc, argv, "--all-ranks")) {
      for (int64_t r = 0; r < d.world(); ++r) print_rank(topo, d, r, layers, schedule);
    } else {
      print_rank(topo, d, c.rank, layers, schedule);
    }
    for (const auto& kv : topo.nccl_env()) std::printf("env %s=%s\n", kv.first.c_str(), kv.second.c_str());
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "cverl_parallel_plan: %s\n", e.what());
    return 1;
  }
}
