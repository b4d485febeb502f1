// Fused MoE router: top-k selection + softmax over the router logits, forward and backward.
//
// One warp per token.  Forward reads the token's E logits (fp32, produced by the tcgen05 GEMM with the
// fp32 epilogue), picks the k largest by k rounds of warp arg-max, and writes the expert ids and the
// routing weights: softmax over the selected logits (norm_topk_prob) or the selected entries of the
// softmax over all experts.  Backward turns d(weights) into d(logits) with the softmax Jacobian in the
// same one-warp-per-token layout; the dense [T, E] gradient then feeds the router's two small GEMMs.
//
// The reference composes matmul / topk / softmax / gather ATen ops (src/model/qwen3_5_text.cc:713-760).
#include "ptx.cuh"

namespace cvb {

constexpr int RT_THREADS = 256;
constexpr int RT_MAX_PER_LANE = 8;  // E <= 256

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) v = ov, i = oi;
  }
}

// logits [T, E] fp32 -> idx [T, k] int64, w [T, k] fp32
__global__ void __launch_bounds__(RT_THREADS)
router_topk_fwd_kernel(const float* __restrict__ logits, long long T, int E, int k, int norm_topk,
                       long long* __restrict__ idx, float* __restrict__ w) {
  const long long tok = (static_cast<long long>(blockIdx.x) * RT_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  const int per = (E + 31) / 32;
  float v[RT_MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    float x = (j < per && e < E) ? logits[tok * E + e] : -INFINITY;
    // -inf marks "not a candidate"; a NaN or infinite logit becomes a finite extreme, so that k experts are always
    // found and every id written is inside [0, E) (ids index tables further down the layer)
    if (j < per && e < E) x = (x != x) ? -3.0e38f : fminf(fmaxf(x, -3.0e38f), 3.0e38f);
    v[j] = x;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float denom_all = 0.f;
  if (!norm_topk) {
#pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) denom_all += (v[j] > -INFINITY) ? __expf(v[j] - mx) : 0.f;
    denom_all = warp_sum(denom_all);
  }
  float sel_val = 0.f;   // lane r keeps the r-th selected logit
  int sel_idx = 0;
  float denom_k = 0.f;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j)
      if (v[j] > bv) bv = v[j], bi = j * 32 + lane;
    warp_argmax(bv, bi);
    if ((bi & 31) == lane) {   // remove the winner from its owner's candidates
#pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j)
        if (j == (bi >> 5)) v[j] = -INFINITY;
    }
    if (bi >= E) bi = r < E ? r : 0;                   // cannot happen for k <= E; keeps the id inside the table
    if (lane == r) sel_val = bv, sel_idx = bi;
    denom_k += __expf(bv - mx);                       // first winner is the global max: exponents <= 0
  }
  if (lane < k) {
    const float p = __expf(sel_val - mx) / (norm_topk ? denom_k : denom_all);
    idx[tok * k + lane] = sel_idx;
    w[tok * k + lane] = p;
  }
}

// dlogits [T, E] fp32 from dw [T, k]
__global__ void __launch_bounds__(RT_THREADS)
router_topk_bwd_kernel(const float* __restrict__ logits, const long long* __restrict__ idx,
                       const float* __restrict__ w, const float* __restrict__ dw, long long T, int E, int k,
                       int norm_topk, float* __restrict__ dlogits) {
  const long long tok = (static_cast<long long>(blockIdx.x) * RT_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  const float wi = lane < k ? w[tok * k + lane] : 0.f;
  const float di = lane < k ? dw[tok * k + lane] : 0.f;
  const int ei = lane < k ? static_cast<int>(idx[tok * k + lane]) : -1;
  const float dot = warp_sum(wi * di);   // sum_i w_i dw_i
  float mx = -INFINITY, denom = 1.f;
  const int per = (E + 31) / 32;
  if (!norm_topk) {
    for (int j = 0; j < per; ++j) {
      const int e = j * 32 + lane;
      if (e < E) mx = fmaxf(mx, logits[tok * E + e]);
    }
    mx = warp_max(mx);
    float s = 0.f;
    for (int j = 0; j < per; ++j) {
      const int e = j * 32 + lane;
      if (e < E) s += __expf(logits[tok * E + e] - mx);
    }
    denom = warp_sum(s);
  }
  for (int j = 0; j < per; ++j) {
    const int e = j * 32 + lane;
    if (e >= E) continue;
    float g = norm_topk ? 0.f : -(__expf(logits[tok * E + e] - mx) / denom) * dot;
    dlogits[tok * E + e] = g;
  }
  __syncwarp();
  if (lane < k) {   // selected experts: w_i (dw_i - dot) replaces / adds to the dense term
    const float g = wi * (di - dot);
    if (norm_topk) dlogits[tok * E + ei] = g;
    else dlogits[tok * E + ei] = wi * di - wi * dot;
  }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_router_topk_fwd(const float* logits, long long T, int E, int k, int norm_topk, long long* idx,
                                   float* w, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 32 * RT_MAX_PER_LANE || k <= 0 || k > 32 || k > E) return -1;
  const long long blocks = (T * 32 + RT_THREADS - 1) / RT_THREADS;
  router_topk_fwd_kernel<<<static_cast<unsigned>(blocks), RT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, T, E, k, norm_topk, idx, w);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_router_topk_bwd(const float* logits, const long long* idx, const float* w, const float* dw,
                                   long long T, int E, int k, int norm_topk, float* dlogits, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 32 * RT_MAX_PER_LANE || k <= 0 || k > 32 || k > E) return -1;
  const long long blocks = (T * 32 + RT_THREADS - 1) / RT_THREADS;
  router_topk_bwd_kernel<<<static_cast<unsigned>(blocks), RT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, idx, w, dw, T, E, k, norm_topk, dlogits);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------
// Expert-layout bookkeeping for the grouped expert GEMM, in four small launches and no host read.
//
// Given one expert id per (token, k) entry, the grouped GEMM wants the entries grouped by expert, every expert's
// segment padded to a multiple of 128 rows, and a table naming the expert of each 128-row tile.  The layout keeps
// the entries of an expert in their original order (a stable counting sort), so that results do not depend on
// the block schedule:
//   1. expert_rank_kernel    per 256 entries: each entry's rank among the same-expert entries of its block
//                            (warp match + per-warp counts), and the block's per-expert counts
//   2. expert_prefix_kernel  a warp per expert: exclusive prefix of the block counts over the blocks;
//      expert_offsets_kernel one block: the padded segment bounds and the tile table
//   3. expert_place_kernel   row of every entry = padded segment start + prefix of its block + rank in block
// The reference (and the tensor-op fallback of this package) builds the same layout from bincount, sort, cumsum,
// index_put_, nonzero and index_select calls with host reads of the capacities
// (src/distributed/expert_parallel.cc:116-136, src/model/qwen3_5_text.cc:882-923).
// ---------------------------------------------------------------------------------------------------
namespace cvb {

constexpr int EL_THREADS = 256;
constexpr int EL_MAX_E = 257;     // 256 experts + the bucket of unused entries (id == E)

__global__ void __launch_bounds__(EL_THREADS)
expert_rank_kernel(const long long* __restrict__ ids, long long n, int E, int* __restrict__ rank_in_block,
                   int* __restrict__ block_counts, int* __restrict__ bad) {
  __shared__ int warp_cnt[EL_THREADS / 32][EL_MAX_E];
  const int t = threadIdx.x, w = t >> 5, lane = t & 31;
  for (int i = t; i < (EL_THREADS / 32) * EL_MAX_E; i += EL_THREADS) (&warp_cnt[0][0])[i] = 0;
  __syncthreads();
  const long long i = static_cast<long long>(blockIdx.x) * EL_THREADS + t;
  long long e64 = i < n ? ids[i] : -1;
  if (i < n && (e64 < 0 || e64 >= E)) {       // an id outside the table: reported, entry parked on the last row
    atomicCAS(bad, 0, ERR_BAD_ARG);
    e64 = -1;
  }
  const int e = static_cast<int>(e64);
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int r_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && r_warp == 0) warp_cnt[w][e] = __popc(peers);
  __syncthreads();
  int base = 0;
  if (e >= 0) {
    for (int ww = 0; ww < w; ++ww) base += warp_cnt[ww][e];
    rank_in_block[i] = base + r_warp;
  }
  for (int ee = t; ee < E; ee += EL_THREADS) {
    int s = 0;
#pragma unroll
    for (int ww = 0; ww < EL_THREADS / 32; ++ww) s += warp_cnt[ww][ee];
    block_counts[static_cast<long long>(blockIdx.x) * E + ee] = s;
  }
}

// block_counts [nblocks, E] -> exclusive prefix over blocks in place, totals [E]: one warp per expert walks the
// blocks 32 at a time with a shuffle scan
__global__ void __launch_bounds__(EL_THREADS)
expert_prefix_kernel(int* __restrict__ block_counts, int nblocks, int E, int* __restrict__ totals) {
  const int e = blockIdx.x * (EL_THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= E) return;
  int carry = 0;
  for (int b0 = 0; b0 < nblocks; b0 += 32) {
    const int b = b0 + lane;
    const int c = b < nblocks ? block_counts[static_cast<long long>(b) * E + e] : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (b < nblocks) block_counts[static_cast<long long>(b) * E + e] = carry + incl - c;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) totals[e] = carry;
}

// totals [E] -> offsets [E + 1] (padded segment bounds, int32) and tile_group [n_tiles] (expert of each tile_m-row
// tile, -1 past the end)
__global__ void __launch_bounds__(EL_THREADS)
expert_offsets_kernel(const int* __restrict__ totals, int E, int tile_m, int* __restrict__ offsets,
                      int* __restrict__ tile_group, int n_tiles) {
  __shared__ int padded[EL_MAX_E + 1];
  const int t = threadIdx.x;
  for (int e = t; e < E; e += EL_THREADS) padded[e + 1] = (totals[e] + tile_m - 1) / tile_m * tile_m;
  __syncthreads();
  if (t == 0) {
    padded[0] = 0;
    for (int e = 0; e < E; ++e) padded[e + 1] += padded[e];
  }
  __syncthreads();
  for (int e = t; e <= E; e += EL_THREADS) offsets[e] = padded[e];
  for (int tile = t; tile < n_tiles; tile += EL_THREADS) {
    const int row = tile * tile_m;
    int g = -1;
    if (row < padded[E]) {
      int lo = 0, hi = E;                      // first e with padded[e + 1] > row
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (padded[mid + 1] > row) hi = mid; else lo = mid + 1;
      }
      g = lo;
    }
    tile_group[tile] = g;
  }
}

__global__ void __launch_bounds__(EL_THREADS)
expert_place_kernel(const long long* __restrict__ ids, long long n, int E, const int* __restrict__ rank_in_block,
                    const int* __restrict__ block_prefix, const int* __restrict__ offsets,
                    long long* __restrict__ row_of_entry, long long last_row) {
  const long long i = static_cast<long long>(blockIdx.x) * EL_THREADS + threadIdx.x;
  if (i >= n) return;
  const long long e = ids[i];
  if (e < 0 || e >= E) {                      // already reported by expert_rank_kernel; any valid row will do
    row_of_entry[i] = last_row;
    return;
  }
  // bucket E - 1 is the "unused" bucket: offsets[E - 1] is the end of the last real segment
  long long r = offsets[e] + block_prefix[static_cast<long long>(blockIdx.x) * E + e] + rank_in_block[i];
  row_of_entry[i] = r <= last_row ? r : last_row;
}

}  // namespace cvb

// ids in [0, E) name an expert; id == E marks an unused entry (placed after the last segment, as the tensor-op
// version does); anything else sets *bad = ERR_BAD_ARG.  scratch: int32 [n + (nblocks + 1) * (E + 1)] with
// nblocks = ceil(n / 256).  Every row written is inside [0, n_tiles * tile_m).
extern "C" int cvb_expert_layout(const long long* ids, long long n, int E, int tile_m, int* scratch, int* offsets,
                                 int* tile_group, int n_tiles, long long* row_of_entry, int* bad, void* stream) {
  using namespace cvb;
  if (E <= 0 || E + 1 > EL_MAX_E || tile_m <= 0 || n < 0 || n >= (1ll << 31) - EL_THREADS || n_tiles <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nblocks = static_cast<int>((n + EL_THREADS - 1) / EL_THREADS);
  const int Eb = E + 1;
  int* rank = scratch;
  int* counts = scratch + n;
  int* totals = counts + static_cast<long long>(nblocks) * Eb;
  if (nblocks > 0)
    expert_rank_kernel<<<nblocks, EL_THREADS, 0, st>>>(ids, n, Eb, rank, counts, bad);
  expert_prefix_kernel<<<(Eb + EL_THREADS / 32 - 1) / (EL_THREADS / 32), EL_THREADS, 0, st>>>(counts, nblocks, Eb, totals);
  expert_offsets_kernel<<<1, EL_THREADS, 0, st>>>(totals, E, tile_m, offsets, tile_group, n_tiles);
  if (nblocks > 0)
    expert_place_kernel<<<nblocks, EL_THREADS, 0, st>>>(ids, n, Eb, rank, counts, offsets, row_of_entry,
                                                        static_cast<long long>(n_tiles) * tile_m - 1);
  return static_cast<int>(cudaGetLastError());
}
