// Topology, pipeline schedule and ZeRO owner assignment (host runtime).
#include "cverl/topology.h"

#include <algorithm>
#include <cstdlib>
#include <numeric>
#include <set>
#include <stdexcept>

namespace cverl {

Topology::Topology(ParallelDims dims, ClusterSpec cluster, NetworkPolicy network, MemoryPolicy memory)
    : dims_(dims), cluster_(cluster), network_(std::move(network)), memory_(memory) {
  validate();
}

void Topology::validate() const {
  const ParallelDims& d = dims_;
  if (d.data <= 0 || d.pipeline <= 0 || d.context <= 0 || d.tensor <= 0 || d.expert <= 0 || d.sequence <= 0 ||
      d.micro_batches <= 0)
    throw std::invalid_argument("parallel dimensions must be positive");
  if (d.world() != cluster_.world_size) throw std::invalid_argument("world size != dp*pp*cp*tp*ep");
  if (d.tensor > cluster_.gpus_per_node) throw std::invalid_argument("tensor parallel size must fit in one node");
  if (d.tensor % d.sequence != 0) throw std::invalid_argument("sequence parallel size must divide tensor size");
  if (d.micro_batches < d.pipeline) throw std::invalid_argument("micro_batches must be >= pipeline size");
  if (cluster_.rank < 0 || cluster_.rank >= cluster_.world_size) throw std::invalid_argument("rank out of range");
}

int64_t Topology::rank_of(int64_t dp, int64_t pp, int64_t cp, int64_t tp, int64_t ep) const {
  return ((((dp * dims_.pipeline + pp) * dims_.context + cp) * dims_.tensor + tp) * dims_.expert + ep);
}

ParallelRankInfo Topology::rank_info(int64_t rank) const {
  if (rank < 0 || rank >= dims_.world()) throw std::invalid_argument("rank out of range");
  ParallelRankInfo r;
  r.global_rank = rank;
  int64_t x = rank;
  r.expert_rank = x % dims_.expert;
  x /= dims_.expert;
  r.tensor_rank = x % dims_.tensor;
  x /= dims_.tensor;
  r.context_rank = x % dims_.context;
  x /= dims_.context;
  r.pipeline_rank = x % dims_.pipeline;
  r.data_rank = x / dims_.pipeline;
  r.sequence_rank = r.tensor_rank % dims_.sequence;
  const int64_t dp = r.data_rank, pp = r.pipeline_rank, cp = r.context_rank, tp = r.tensor_rank, ep = r.expert_rank;
  for (int64_t i = 0; i < dims_.data; ++i) r.data_group.push_back(rank_of(i, pp, cp, tp, ep));
  for (int64_t i = 0; i < dims_.pipeline; ++i) r.pipeline_group.push_back(rank_of(dp, i, cp, tp, ep));
  for (int64_t i = 0; i < dims_.context; ++i) r.context_group.push_back(rank_of(dp, pp, i, tp, ep));
  for (int64_t i = 0; i < dims_.tensor; ++i) r.tensor_group.push_back(rank_of(dp, pp, cp, i, ep));
  for (int64_t i = 0; i < dims_.expert; ++i) r.expert_group.push_back(rank_of(dp, pp, cp, tp, i));
  const int64_t seq_base = (tp / dims_.sequence) * dims_.sequence;
  for (int64_t i = 0; i < dims_.sequence; ++i) r.sequence_group.push_back(rank_of(dp, pp, cp, seq_base + i, ep));
  for (int64_t p = 0; p < dims_.pipeline; ++p)
    for (int64_t c = 0; c < dims_.context; ++c)
      for (int64_t t = 0; t < dims_.tensor; ++t)
        for (int64_t e = 0; e < dims_.expert; ++e) r.model_group.push_back(rank_of(dp, p, c, t, e));
  return r;
}

std::pair<int64_t, int64_t> Topology::pipeline_layer_range(int64_t num_layers, int64_t pipeline_rank) const {
  const int64_t pp = dims_.pipeline;
  if (num_layers < pp) throw std::invalid_argument("fewer layers than pipeline stages");
  if (pipeline_rank < 0 || pipeline_rank >= pp) throw std::invalid_argument("pipeline rank out of range");
  const int64_t base = num_layers / pp, rem = num_layers % pp;
  const int64_t begin = pipeline_rank * base + std::min(pipeline_rank, rem);
  return {begin, begin + base + (pipeline_rank < rem ? 1 : 0)};
}

std::map<std::string, std::string> Topology::nccl_env() const {
  std::map<std::string, std::string> env;
  env["NCCL_P2P_DISABLE"] = network_.enable_p2p ? "0" : "1";
  env["NCCL_IB_DISABLE"] = network_.enable_ib ? "0" : "1";
  env["NCCL_NVLS_ENABLE"] = network_.enable_nvls ? "1" : "0";
  env["NCCL_ASYNC_ERROR_HANDLING"] = "1";
  env["TORCH_NCCL_BLOCKING_WAIT"] = "0";
  if (!network_.socket_ifname.empty()) env["NCCL_SOCKET_IFNAME"] = network_.socket_ifname;
  if (!network_.ib_hca.empty()) env["NCCL_IB_HCA"] = network_.ib_hca;
  if (!network_.topo_file.empty()) env["NCCL_TOPO_FILE"] = network_.topo_file;
  if (network_.ib_gid_index >= 0) env["NCCL_IB_GID_INDEX"] = std::to_string(network_.ib_gid_index);
  return env;
}

static int64_t env_i64(const char* name, int64_t fallback) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  return std::strtoll(v, nullptr, 10);
}

ClusterSpec cluster_spec_from_env() {
  ClusterSpec c;
  c.world_size = env_i64("WORLD_SIZE", 1);
  c.rank = env_i64("RANK", 0);
  c.gpus_per_node = env_i64("CVERL_GPUS_PER_NODE", env_i64("LOCAL_WORLD_SIZE", std::min<int64_t>(c.world_size, 8)));
  const int64_t gpn = std::max<int64_t>(c.gpus_per_node, 1);
  c.local_rank = env_i64("LOCAL_RANK", c.rank % gpn);
  c.local_world_size = env_i64("LOCAL_WORLD_SIZE", gpn);
  c.node_rank = env_i64("NODE_RANK", c.rank / gpn);
  return c;
}

std::vector<PipelineAction> pipeline_1f1b_schedule(int64_t pipeline_rank, int64_t pipeline_size,
                                                   int64_t micro_batches) {
  if (pipeline_size <= 0 || pipeline_rank < 0 || pipeline_rank >= pipeline_size)
    throw std::invalid_argument("invalid pipeline rank/size");
  if (micro_batches < pipeline_size) throw std::invalid_argument("1F1B requires micro_batches >= pipeline size");
  const int64_t warmup = std::min(pipeline_size - pipeline_rank - 1, micro_batches);
  std::vector<PipelineAction> out;
  int64_t f = 0, b = 0;
  for (int64_t i = 0; i < warmup; ++i) out.push_back({PipelineActionType::Forward, f++});
  for (int64_t i = 0; i < micro_batches - warmup; ++i) {
    out.push_back({PipelineActionType::Forward, f++});
    out.push_back({PipelineActionType::Backward, b++});
  }
  while (b < micro_batches) out.push_back({PipelineActionType::Backward, b++});
  return out;
}

int64_t pipeline_schedule_max_live_activations(const std::vector<PipelineAction>& actions, int64_t micro_batches) {
  std::set<int64_t> fwd, bwd;
  int64_t live = 0, peak = 0;
  for (const auto& a : actions) {
    if (a.micro_batch < 0 || a.micro_batch >= micro_batches) throw std::invalid_argument("micro-batch out of range");
    if (a.type == PipelineActionType::Forward) {
      if (!fwd.insert(a.micro_batch).second) throw std::invalid_argument("micro-batch forwarded twice");
      peak = std::max(peak, ++live);
    } else {
      if (!fwd.count(a.micro_batch) || !bwd.insert(a.micro_batch).second)
        throw std::invalid_argument("backward without a matching forward");
      --live;
    }
  }
  if (static_cast<int64_t>(fwd.size()) != micro_batches || static_cast<int64_t>(bwd.size()) != micro_batches)
    throw std::invalid_argument("schedule does not cover every micro-batch");
  return peak;
}

PipelinePeers pipeline_peers(const std::vector<int64_t>& group, int64_t pipeline_rank) {
  const int64_t n = static_cast<int64_t>(group.size());
  if (pipeline_rank < 0 || pipeline_rank >= n) throw std::invalid_argument("pipeline rank out of range");
  PipelinePeers p;
  if (pipeline_rank > 0) p.prev_rank = group[pipeline_rank - 1];
  if (pipeline_rank + 1 < n) p.next_rank = group[pipeline_rank + 1];
  return p;
}

std::vector<int64_t> greedy_parameter_owners(const std::vector<int64_t>& numels, int64_t dp_size) {
  if (dp_size <= 0) throw std::invalid_argument("dp_size must be positive");
  std::vector<int64_t> order(numels.size());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return numels[a] > numels[b]; });
  std::vector<int64_t> load(dp_size, 0), owners(numels.size(), 0);
  for (int64_t i : order) {
    const int64_t r = std::min_element(load.begin(), load.end()) - load.begin();
    owners[i] = r;
    load[r] += numels[i];
  }
  return owners;
}

}  // namespace cverl

namespace {
cverl::Topology make_topology(const int64_t* d, int64_t world, int64_t gpn, int64_t rank) {
  cverl::ParallelDims dims;
  dims.data = d[0], dims.pipeline = d[1], dims.context = d[2], dims.tensor = d[3], dims.expert = d[4];
  dims.sequence = d[5], dims.micro_batches = d[6];
  cverl::ClusterSpec c;
  c.world_size = world, c.rank = rank, c.gpus_per_node = gpn;
  return cverl::Topology(dims, c);
}
}  // namespace

extern "C" {

int cverl_topology_coords(const int64_t* dims, int64_t world, int64_t gpn, int64_t rank, int64_t* out) {
  try {
    auto info = make_topology(dims, world, gpn, rank).rank_info();
    out[0] = info.data_rank, out[1] = info.pipeline_rank, out[2] = info.context_rank, out[3] = info.tensor_rank,
    out[4] = info.expert_rank;
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

int cverl_topology_group(const int64_t* dims, int64_t world, int64_t gpn, int64_t rank, int axis, int64_t* out_ranks,
                         int64_t capacity, int64_t* out_count) {
  try {
    auto info = make_topology(dims, world, gpn, rank).rank_info();
    const std::vector<int64_t>* g = nullptr;
    switch (axis) {
      case 0: g = &info.data_group; break;
      case 1: g = &info.pipeline_group; break;
      case 2: g = &info.context_group; break;
      case 3: g = &info.tensor_group; break;
      case 4: g = &info.expert_group; break;
      case 5: g = &info.sequence_group; break;
      case 6: g = &info.model_group; break;
      default: return 1;
    }
    if (static_cast<int64_t>(g->size()) > capacity) return 1;
    std::copy(g->begin(), g->end(), out_ranks);
    *out_count = static_cast<int64_t>(g->size());
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

int cverl_pipeline_layer_range(int64_t num_layers, int64_t pp_size, int64_t pp_rank, int64_t* begin, int64_t* end) {
  try {
    cverl::ParallelDims d;
    d.pipeline = pp_size, d.micro_batches = pp_size;
    cverl::ClusterSpec c;
    c.world_size = pp_size;
    auto r = cverl::Topology(d, c).pipeline_layer_range(num_layers, pp_rank);
    *begin = r.first, *end = r.second;
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

int cverl_pipeline_1f1b(int64_t pp_rank, int64_t pp_size, int64_t micro_batches, int32_t* out_types,
                        int64_t* out_micro, int64_t capacity, int64_t* out_count, int64_t* out_max_live) {
  try {
    auto s = cverl::pipeline_1f1b_schedule(pp_rank, pp_size, micro_batches);
    if (static_cast<int64_t>(s.size()) > capacity) return 1;
    for (size_t i = 0; i < s.size(); ++i) {
      out_types[i] = s[i].type == cverl::PipelineActionType::Forward ? 0 : 1;
      out_micro[i] = s[i].micro_batch;
    }
    *out_count = static_cast<int64_t>(s.size());
    if (out_max_live) *out_max_live = cverl::pipeline_schedule_max_live_activations(s, micro_batches);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

int cverl_greedy_owners(const int64_t* numels, int64_t n, int64_t dp_size, int64_t* out_owners) {
  try {
    auto o = cverl::greedy_parameter_owners(std::vector<int64_t>(numels, numels + n), dp_size);
    std::copy(o.begin(), o.end(), out_owners);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}
}
