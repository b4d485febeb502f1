// Dumps what the reference's Topology and pipeline schedule (include/cverl/distributed/topology.h:74-104,
// pipeline.h:45-50) say about a layout - validity, every rank's coordinates and groups, pipeline peers, layer
// ranges, the 1F1B action list and its peak of live activations, the NCCL environment - as JSON, for comparison
// with this package's planner.  Linked against the unmodified reference library.
//   ref_topology_check DP PP CP TP EP SP MICRO_BATCHES WORLD GPUS_PER_NODE NUM_LAYERS
#include <iostream>

#include <nlohmann/json.hpp>

#include "cverl/distributed/pipeline.h"
#include "cverl/distributed/topology.h"

int main(int argc, char** argv) {
  if (argc < 11) return 2;
  nlohmann::json out;
  try {
    cverl::distributed::ClusterSpec spec;
    spec.parallel.data_parallel = std::stoll(argv[1]);
    spec.parallel.pipeline_parallel = std::stoll(argv[2]);
    spec.parallel.context_parallel = std::stoll(argv[3]);
    spec.parallel.tensor_parallel = std::stoll(argv[4]);
    spec.parallel.expert_parallel = std::stoll(argv[5]);
    spec.parallel.sequence_parallel = std::stoll(argv[6]);
    spec.parallel.micro_batches = std::stoll(argv[7]);
    spec.world_size = std::stoll(argv[8]);
    spec.gpus_per_node = std::stoll(argv[9]);
    spec.local_world_size = std::min(spec.world_size, spec.gpus_per_node);
    const int64_t layers = std::stoll(argv[10]);
    cverl::distributed::Topology topology(spec);
    out["valid"] = true;
    out["ranks"] = nlohmann::json::array();
    for (int64_t r = 0; r < topology.world_size(); ++r) {
      const auto info = topology.rank_info(r);
      const auto peers = cverl::distributed::pipeline_peers(topology, info);
      const auto range = topology.pipeline_layer_range(layers, info.pipeline_rank);
      const auto actions = cverl::distributed::pipeline_1f1b_schedule(topology, info);
      nlohmann::json j;
      j["coords"] = {info.data_rank, info.pipeline_rank, info.context_rank, info.tensor_rank, info.expert_rank};
      j["sequence_rank"] = info.sequence_rank;
      j["data"] = info.data_group;
      j["pipeline"] = info.pipeline_group;
      j["context"] = info.context_group;
      j["tensor"] = info.tensor_group;
      j["expert"] = info.expert_group;
      j["sequence"] = info.sequence_group;
      j["model"] = info.model_group;
      j["prev"] = peers.previous_rank;
      j["next"] = peers.next_rank;
      j["layers"] = {range.begin, range.end};
      nlohmann::json sched = nlohmann::json::array();
      for (const auto& a : actions)
        sched.push_back({a.op == cverl::distributed::PipelineScheduleOp::Forward ? 0 : 1, a.micro_batch});
      j["schedule"] = sched;
      j["max_live"] = cverl::distributed::pipeline_schedule_max_live_activations(actions);
      out["ranks"].push_back(j);
    }
    out["nccl_env"] = topology.nccl_env();
  } catch (const std::exception& e) {
    out = nlohmann::json{{"valid", false}, {"error", e.what()}};
  }
  std::cout << out.dump() << "\n";
  return 0;
}
