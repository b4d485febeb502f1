// Kernels that communicate by themselves over NVLink through peer-mapped ("symmetric") buffers:
// plain P2P loads and stores on pointers that every rank of a group obtained by opening the
// others' allocations (CUDA IPC).  No library collective is involved on these paths.
//
//  * symm_barrier           flag exchange with bounded waits (release / acquire at system scope)
//  * reduce_scatter_sumsq   ZeRO gradient reduce-scatter: each rank pulls its shard of every peer's
//                           flat fp32 gradient, sums, scales (mean) and accumulates the squared norm
//                           for global-norm clipping, in one pass
//  * reduce_scatter_acc     bucketed ZeRO-2: the same pull, accumulated into the shard gradient, the reader clearing
//                           the source so that the bucket buffer can be reused
//  * flat_adamw_allgather   FlatAdamW on the local shard whose bf16 result is stored straight into
//                           every peer's parameter buffer: the parameter all-gather rides on the
//                           optimizer's own stores
//  * broadcast_store        trainer -> rollout weight push: one read of the source, one store per peer
//  * sum_parts              second half of the tensor-parallel all-reduce whose first half is the GEMM
//                           epilogue's mirror stores into every peer (gemm_tcgen05.cu)
//
// The reference does these with ncclReduceScatter / ATen ops / ncclAllGather / ncclBroadcast
// (src/distributed/optimizer_sharding.cc:463-733, src/distributed/weight_sync.cc:140-189).
#include "ptx.cuh"

namespace cvb {

constexpr int MAX_PEERS = 8;
constexpr int SY_THREADS = 256;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags[peer] is that peer's flag array (int[MAX_PEERS]); slot [rank] of it belongs to this rank.
// Every rank stores `epoch` into its slot on every peer, then waits until all slots of its own
// array have reached `epoch`.  A wait that runs out sets *status and returns.
__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int* status) {
  const int t = threadIdx.x;
  __threadfence_system();
  if (t < world) {
    st_release_sys(static_cast<int*>(flags.p[t]) + rank, epoch);
    const int* mine = static_cast<const int*>(flags.p[rank]) + t;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > CVB_WAIT_BUDGET_CYCLES) {
        atomicCAS(status, 0, ERR_WAIT_PEER);
        break;
      }
      __nanosleep(64);
    }
  }
  __threadfence_system();
}

// out[i] = scale * sum_p grads[p][begin + i],  sq += sum out[i]^2      (i in [0, n), n % 4 == 0)
__global__ void __launch_bounds__(SY_THREADS)
reduce_scatter_sumsq_kernel(PeerPtrs grads, int world, int rank, long long begin, long long n, float scale,
                            float* __restrict__ out, float* __restrict__ sq) {
  __shared__ float sh[SY_THREADS / 32];
  float acc = 0.f;
  const long long nv = n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * SY_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * SY_THREADS) {
    float4 v[MAX_PEERS];               // start at home, then walk the peers; all loads issued before the first add
#pragma unroll
    for (int k = 0; k < MAX_PEERS; ++k) {
      if (k < world) {
        const int p = (rank + k) % world;
        v[k] = *reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[p]) + begin + i * 4);
      }
    }
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < MAX_PEERS; ++k) {
      if (k < world) { s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w; }
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    *reinterpret_cast<float4*>(out + i * 4) = s;
    acc += (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < SY_THREADS / 32 ? sh[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) atomicAdd(sq, r);
  }
}

// Bucketed ZeRO-2: out[i] += scale * sum_p grads[p][begin + i]; with zero_src the reader also clears what it read
// (every element of a gradient bucket is read by exactly one rank, its owner, so the clear needs no second pass
// on the source GPU - only the barrier that tells it the bucket buffer is free again).
__global__ void __launch_bounds__(SY_THREADS)
reduce_scatter_acc_kernel(PeerPtrs grads, int world, int rank, long long begin, long long n, float scale,
                          float* __restrict__ out, int zero_src) {
  const long long nv = n / 4;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = static_cast<long long>(blockIdx.x) * SY_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * SY_THREADS) {
    // all peers' loads are issued before the first use: eight independent 16-byte requests in flight per thread
    float4 v[MAX_PEERS];
#pragma unroll
    for (int k = 0; k < MAX_PEERS; ++k) {
      if (k < world) {
        const int p = (rank + k) % world;
        v[k] = *reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[p]) + begin + i * 4);
      }
    }
    float4 s = zero;
#pragma unroll
    for (int k = 0; k < MAX_PEERS; ++k) {
      if (k < world) {
        s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w;
        if (zero_src) {
          const int p = (rank + k) % world;
          *reinterpret_cast<float4*>(static_cast<float*>(grads.p[p]) + begin + i * 4) = zero;
        }
      }
    }
    float4 o = *reinterpret_cast<const float4*>(out + i * 4);
    o.x += s.x * scale; o.y += s.y * scale; o.z += s.z * scale; o.w += s.w * scale;
    *reinterpret_cast<float4*>(out + i * 4) = o;
  }
}

struct AdamBcastArgs {
  float* grad;          // local fp32 gradient shard [n]
  float* master;        // local fp32 master shard or nullptr
  float* m;
  float* v;
  const float* clip;    // device scalar or nullptr
  PeerPtrs params;      // every rank's FULL bf16 parameter buffer
  int world, rank;
  long long begin, n;   // this rank's shard inside the full buffer
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
};

__global__ void __launch_bounds__(SY_THREADS)
flat_adamw_allgather_kernel(const AdamBcastArgs a) {
  const float cs = a.clip ? a.clip[0] : 1.f;
  const float step_size = a.lr / a.bc1, decay = 1.f - a.lr * a.weight_decay, inv_bc2 = 1.f / a.bc2;
  const long long nv = a.n / 4;
  __nv_bfloat16* home = static_cast<__nv_bfloat16*>(a.params.p[a.rank]) + a.begin;
  for (long long i = static_cast<long long>(blockIdx.x) * SY_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * SY_THREADS) {
    const float4 g = *reinterpret_cast<const float4*>(a.grad + i * 4);
    float4 m = *reinterpret_cast<const float4*>(a.m + i * 4);
    float4 v = *reinterpret_cast<const float4*>(a.v + i * 4);
    float p[4];
    if (a.master) {
      const float4 pm = *reinterpret_cast<const float4*>(a.master + i * 4);
      p[0] = pm.x, p[1] = pm.y, p[2] = pm.z, p[3] = pm.w;
    } else {
      const uint2 pb = *reinterpret_cast<const uint2*>(home + i * 4);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pb);
      const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
      p[0] = f0.x, p[1] = f0.y, p[2] = f1.x, p[3] = f1.y;
    }
    const float gg[4] = {g.x * cs, g.y * cs, g.z * cs, g.w * cs};
    float mm[4] = {m.x, m.y, m.z, m.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gg[j];
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gg[j] * gg[j];
      p[j] = p[j] * decay;
      p[j] -= step_size * mm[j] / (sqrtf(vv[j] * inv_bc2) + a.eps);
    }
    *reinterpret_cast<float4*>(a.m + i * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(a.v + i * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (a.master) *reinterpret_cast<float4*>(a.master + i * 4) = make_float4(p[0], p[1], p[2], p[3]);
    uint2 o;
    o.x = pack_bf16x2(p[0], p[1]);
    o.y = pack_bf16x2(p[2], p[3]);
#pragma unroll 1
    for (int k = 0; k < a.world; ++k) {  // the all-gather: one store per rank, local copy included
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.params.p[(a.rank + k) % a.world]) + a.begin;
      *reinterpret_cast<uint2*>(dst + i * 4) = o;
    }
  }
}

// dst[p][i] = src[i] for every listed peer (16-byte vectors; nbytes % 16 == 0)
__global__ void __launch_bounds__(SY_THREADS)
broadcast_store_kernel(const uint4* __restrict__ src, PeerPtrs dst, int n_dst, long long nvec) {
  for (long long i = static_cast<long long>(blockIdx.x) * SY_THREADS + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * SY_THREADS) {
    const uint4 v = src[i];
#pragma unroll 1
    for (int k = 0; k < n_dst; ++k) static_cast<uint4*>(dst.p[k])[i] = v;
  }
}

// out[i] = sum_r parts[r * slot_stride + i]   (bf16 in, fp32 sum, bf16 out; 8 elements per thread)
// The addends are the per-rank partial products that the GEMM epilogues of a tensor-parallel group stored
// into every member's copy of `parts` (mirror stores): summing the local copy completes the all-reduce.
__global__ void __launch_bounds__(SY_THREADS)
sum_parts_kernel(const __nv_bfloat16* __restrict__ parts, long long slot_stride, int world,
                 __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = static_cast<long long>(blockIdx.x) * SY_THREADS + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * SY_THREADS) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int r = 0; r < world; ++r) {
      const uint4 u = *reinterpret_cast<const uint4*>(parts + r * slot_stride + i * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}

static int sy_grid(long long nvec) {
  long long b = (nvec + SY_THREADS - 1) / SY_THREADS;
  if (b > 148 * 8) b = 148 * 8;
  return b < 1 ? 1 : static_cast<int>(b);
}
static bool fill(PeerPtrs* pp, void* const* ptrs, int n) {
  if (n <= 0 || n > MAX_PEERS) return false;
  for (int i = 0; i < MAX_PEERS; ++i) pp->p[i] = i < n ? ptrs[i] : nullptr;
  return true;
}

}  // namespace cvb

using namespace cvb;
#define ST(s) static_cast<cudaStream_t>(s)

extern "C" int cvb_symm_barrier(void* const* flag_ptrs, int rank, int world, int epoch, int* status, void* stream) {
  PeerPtrs f;
  if (!fill(&f, flag_ptrs, world)) return -1;
  symm_barrier_kernel<<<1, 32, 0, ST(stream)>>>(f, rank, world, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_reduce_scatter_sumsq(void* const* grad_ptrs, int world, int rank, long long begin, long long n,
                                        float scale, float* out, float* sq, void* stream) {
  PeerPtrs g;
  if (!fill(&g, grad_ptrs, world) || n % 4 || begin % 4) return -1;
  if (n == 0) return 0;
  reduce_scatter_sumsq_kernel<<<sy_grid(n / 4), SY_THREADS, 0, ST(stream)>>>(g, world, rank, begin, n, scale, out, sq);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_reduce_scatter_acc(void* const* grad_ptrs, int world, int rank, long long begin, long long n,
                                      float scale, float* out, int zero_src, int max_blocks, void* stream) {
  PeerPtrs g;
  if (!fill(&g, grad_ptrs, world) || n % 4 || begin % 4 || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  if (n == 0) return 0;
  int grid = sy_grid(n / 4);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;   // leave SMs to the backward pass it overlaps
  reduce_scatter_acc_kernel<<<grid, SY_THREADS, 0, ST(stream)>>>(g, world, rank, begin, n, scale, out, zero_src);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_flat_adamw_allgather(float* grad, float* master, float* m, float* v, const float* clip,
                                        void* const* param_ptrs, int world, int rank, long long begin, long long n,
                                        float lr, float beta1, float beta2, float eps, float weight_decay,
                                        long long step, void* stream) {
  AdamBcastArgs a{};
  if (!fill(&a.params, param_ptrs, world) || n % 4 || begin % 4) return -1;
  if (n == 0) return 0;
  a.grad = grad; a.master = master; a.m = m; a.v = v; a.clip = clip; a.world = world; a.rank = rank;
  a.begin = begin; a.n = n; a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = static_cast<float>(1.0 - pow(static_cast<double>(beta1), static_cast<double>(step)));
  a.bc2 = static_cast<float>(1.0 - pow(static_cast<double>(beta2), static_cast<double>(step)));
  flat_adamw_allgather_kernel<<<sy_grid(n / 4), SY_THREADS, 0, ST(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_broadcast_store(const void* src, void* const* dst_ptrs, int n_dst, long long nbytes, void* stream) {
  PeerPtrs d;
  if (!fill(&d, dst_ptrs, n_dst) || nbytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15)) return -1;
  if (nbytes == 0) return 0;
  broadcast_store_kernel<<<sy_grid(nbytes / 16), SY_THREADS, 0, ST(stream)>>>(static_cast<const uint4*>(src), d, n_dst,
                                                                              nbytes / 16);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_sum_parts(const void* parts, long long slot_stride, int world, void* out, long long n,
                             void* stream) {
  if (world <= 0 || world > MAX_PEERS || n % 8 || slot_stride % 8 ||
      ((reinterpret_cast<uintptr_t>(parts) | reinterpret_cast<uintptr_t>(out)) & 15))
    return -1;
  if (n == 0) return 0;
  sum_parts_kernel<<<sy_grid(n / 8), SY_THREADS, 0, ST(stream)>>>(static_cast<const __nv_bfloat16*>(parts), slot_stride,
                                                                  world, static_cast<__nv_bfloat16*>(out), n / 8);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------
// Row scatter / gather over peer memory: the expert-parallel dispatch and combine.
// Row i of a local [n, row_bytes] matrix corresponds to row `peer_row[i]` of the symmetric matrix on group
// member `peer_rank[i]` (negative rank = skip).  scatter pushes local rows to the peers, gather pulls them
// back; one warp moves one row in 16-byte pieces, so a 4 KB activation row is eight coalesced requests.
// A dispatch is scatter + flag barrier, a combine is flag barrier + gather; their backward passes are each
// other.  The reference does four ncclSend/ncclRecv all-to-alls per MoE layer
// (src/distributed/expert_parallel.cc:43-167).
// ---------------------------------------------------------------------------------------------------
namespace cvb {

template <bool GATHER>
__global__ void __launch_bounds__(SY_THREADS)
p2p_rows_kernel(uint8_t* local, PeerPtrs peers, int world, const int* __restrict__ peer_rank,
                const long long* __restrict__ peer_row, long long n, int row_vec /* 16-byte vectors per row */,
                long long capacity_rows, int* status) {
  const long long row = (static_cast<long long>(blockIdx.x) * SY_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n) return;
  const int pr = peer_rank[row];
  if (pr < 0) return;                                   // an entry marked "not routed"
  const long long dst = peer_row[row];
  // a rank outside the group or a row outside the peer's buffer is skipped and reported, never dereferenced
  if (pr >= world || dst < 0 || dst >= capacity_rows) {
    if (lane == 0 && status != nullptr) atomicCAS(status, 0, ERR_BAD_ARG);
    return;
  }
  uint4* mine = reinterpret_cast<uint4*>(local) + row * row_vec;
  uint4* theirs = reinterpret_cast<uint4*>(peers.p[pr]) + dst * row_vec;
  for (int c = lane; c < row_vec; c += 32) {
    if (GATHER) mine[c] = theirs[c];
    else theirs[c] = mine[c];
  }
}

}  // namespace cvb

// Row movers.  `capacity_rows` is the number of rows of every peer buffer and `status` the device status word:
// an entry whose rank is not in [0, world) or whose row is not in [0, capacity_rows) is skipped and sets
// ERR_BAD_ARG there; a negative rank marks an entry to leave out silently.
extern "C" int cvb_p2p_scatter_rows(const void* local, void* const* peer_ptrs, int world, const int* peer_rank,
                                    const long long* peer_row, long long n, long long row_bytes,
                                    long long capacity_rows, int* status, void* stream) {
  PeerPtrs pp;
  if (!fill(&pp, peer_ptrs, world) || row_bytes % 16 || (reinterpret_cast<uintptr_t>(local) & 15) ||
      capacity_rows <= 0) return -1;
  if (n <= 0) return 0;
  const long long blocks = (n * 32 + SY_THREADS - 1) / SY_THREADS;
  p2p_rows_kernel<false><<<static_cast<unsigned>(blocks), SY_THREADS, 0, ST(stream)>>>(
      static_cast<uint8_t*>(const_cast<void*>(local)), pp, world, peer_rank, peer_row, n,
      static_cast<int>(row_bytes / 16), capacity_rows, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_p2p_gather_rows(void* local, void* const* peer_ptrs, int world, const int* peer_rank,
                                   const long long* peer_row, long long n, long long row_bytes,
                                   long long capacity_rows, int* status, void* stream) {
  PeerPtrs pp;
  if (!fill(&pp, peer_ptrs, world) || row_bytes % 16 || (reinterpret_cast<uintptr_t>(local) & 15) ||
      capacity_rows <= 0) return -1;
  if (n <= 0) return 0;
  const long long blocks = (n * 32 + SY_THREADS - 1) / SY_THREADS;
  p2p_rows_kernel<true><<<static_cast<unsigned>(blocks), SY_THREADS, 0, ST(stream)>>>(
      static_cast<uint8_t*>(local), pp, world, peer_rank, peer_row, n, static_cast<int>(row_bytes / 16),
      capacity_rows, status);
  return static_cast<int>(cudaGetLastError());
}
