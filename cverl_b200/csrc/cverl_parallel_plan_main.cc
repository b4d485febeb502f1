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

int main(int argc, char** argv) {
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
    c.gpus_per_node = arg_i64(argc, argv, "--gpus-per-node", 8);
    const int64_t layers = arg_i64(argc, argv, "--layers", 24);
    cverl::Topology topo(d, c);
    auto info = topo.rank_info();
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
    auto range = topo.pipeline_layer_range(layers, info.pipeline_rank);
    std::printf("layer_begin=%lld layer_end=%lld\n", (long long)range.first, (long long)range.second);
    auto sched = cverl::pipeline_1f1b_schedule(info.pipeline_rank, d.pipeline, d.micro_batches);
    std::printf("schedule=");
    for (const auto& a : sched)
      std::printf("%c%lld ", a.type == cverl::PipelineActionType::Forward ? 'F' : 'B', (long long)a.micro_batch);
    std::printf("\nmax_live_activations=%lld\n",
                (long long)cverl::pipeline_schedule_max_live_activations(sched, d.micro_batches));
    for (const auto& kv : topo.nccl_env()) std::printf("env %s=%s\n", kv.first.c_str(), kv.second.c_str());
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "cverl_parallel_plan: %s\n", e.what());
    return 1;
  }
}
