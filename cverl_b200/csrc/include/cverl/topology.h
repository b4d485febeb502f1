// Rank <-> (dp, pp, cp, tp, ep) topology, pipeline layer ranges, 1F1B schedule.
// C++ twin of cverl_b200/parallel/topology.py and pipeline.py; behaviour as in the
// reference (src/distributed/topology.cc:53-224, src/distributed/pipeline.cc:41-121).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace cverl {

struct ParallelDims {
  int64_t data = 1, pipeline = 1, context = 1, tensor = 1, expert = 1, sequence = 1, micro_batches = 1;
  int64_t world() const { return data * pipeline * context * tensor * expert; }
};

struct ClusterSpec {
  int64_t world_size = 1, rank = 0, local_rank = 0, local_world_size = 1, node_rank = 0, gpus_per_node = 8;
};

struct NetworkPolicy {
  bool enable_p2p = true, enable_ib = true, enable_nvls = true;
  std::string socket_ifname, ib_hca, topo_file;
  int ib_gid_index = -1;
};

struct MemoryPolicy {
  bool activation_checkpointing = false, shard_optimizer_state = true, shard_gradients = false;
  bool offload_optimizer_to_cpu = false, offload_parameters_to_cpu = false;
};

struct ParallelRankInfo {
  int64_t global_rank = 0, data_rank = 0, pipeline_rank = 0, context_rank = 0, tensor_rank = 0, expert_rank = 0,
          sequence_rank = 0;
  std::vector<int64_t> data_group, pipeline_group, context_group, tensor_group, expert_group, sequence_group,
      model_group;
};

class Topology {
 public:
  Topology(ParallelDims dims, ClusterSpec cluster, NetworkPolicy network = {}, MemoryPolicy memory = {});
  const ParallelDims& dims() const { return dims_; }
  const ClusterSpec& cluster() const { return cluster_; }
  int64_t rank_of(int64_t dp, int64_t pp, int64_t cp, int64_t tp, int64_t ep) const;
  ParallelRankInfo rank_info(int64_t rank) const;
  ParallelRankInfo rank_info() const { return rank_info(cluster_.rank); }
  std::pair<int64_t, int64_t> pipeline_layer_range(int64_t num_layers, int64_t pipeline_rank) const;
  std::map<std::string, std::string> nccl_env() const;

 private:
  void validate() const;
  ParallelDims dims_;
  ClusterSpec cluster_;
  NetworkPolicy network_;
  MemoryPolicy memory_;
};

ClusterSpec cluster_spec_from_env();

enum class PipelineActionType { Forward, Backward };
struct PipelineAction {
  PipelineActionType type;
  int64_t micro_batch;
};
struct PipelinePeers {
  int64_t prev_rank = -1, next_rank = -1;
};

std::vector<PipelineAction> pipeline_1f1b_schedule(int64_t pipeline_rank, int64_t pipeline_size,
                                                   int64_t micro_batches);
int64_t pipeline_schedule_max_live_activations(const std::vector<PipelineAction>& actions, int64_t micro_batches);
PipelinePeers pipeline_peers(const std::vector<int64_t>& pipeline_group, int64_t pipeline_rank);

// Largest-first bin packing of parameters to data-parallel ranks (ZeRO-1 owners).
std::vector<int64_t> greedy_parameter_owners(const std::vector<int64_t>& numels, int64_t dp_size);

}  // namespace cverl

extern "C" {
// C entry points used by the Python bindings and tests.  All return 0 on success,
// 1 on invalid arguments.  `dims` = {dp, pp, cp, tp, ep, sp, micro_batches}.
int cverl_topology_coords(const int64_t* dims, int64_t world, int64_t gpus_per_node, int64_t rank,
                          int64_t* out_coords5);
int cverl_topology_group(const int64_t* dims, int64_t world, int64_t gpus_per_node, int64_t rank, int axis,
                         int64_t* out_ranks, int64_t capacity, int64_t* out_count);
int cverl_pipeline_layer_range(int64_t num_layers, int64_t pp_size, int64_t pp_rank, int64_t* begin, int64_t* end);
int cverl_pipeline_1f1b(int64_t pp_rank, int64_t pp_size, int64_t micro_batches, int32_t* out_types,
                        int64_t* out_micro, int64_t capacity, int64_t* out_count, int64_t* out_max_live);
int cverl_greedy_owners(const int64_t* numels, int64_t n, int64_t dp_size, int64_t* out_owners);
}
