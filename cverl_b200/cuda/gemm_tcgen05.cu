// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] (+)= alpha * A[M,K] * B[N,K]^T        fp32 accumulation in TMEM
//
// * operands are staged by TMA (128-byte swizzle) into a multi-stage smem ring,
// * one elected thread issues tcgen05.mma (UMMA 128 x BN x 16, cta_group::1),
// * accumulators live in TMEM and are double buffered (2 x BN columns), so the
//   epilogue of tile i overlaps the main loop of tile i+1,
// * four epilogue warps drain TMEM with tcgen05.ld and run one of several
//   fused epilogues (bf16 / fp32 store, fp32 atomic accumulate for split-K and
//   gradient accumulation, streaming log-sum-exp for the tied LM head, and the
//   softmax-gradient tile for its backward).
//
// Either operand may be K-major (row = M or N index, K contiguous) or MN-major
// (row = K index, M or N contiguous); the three layouts that a linear layer
// needs (y = x W^T, dx = dy W, dW = dy^T x) map to (K,K), (K,MN), (MN,MN).
//
// Grouped variants (MoE experts): `tile_group` assigns each 128-row M tile to
// an expert whose weight block is selected by a row offset in B; with
// `k_group_offsets` each expert owns a K range (dW of grouped experts).
//
// The reference framework runs every linear layer through a library GEMM
// (src/model/qwen3_5_text.cc:86-89, src/distributed/parallel_ops.cc:32-35).
#include "ptx.cuh"
#include "gemm_tcgen05.h"

#include <mutex>
#include <unordered_map>
#include <vector>
#include <cstring>
#include <cstdio>

namespace cvb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // warp0 TMA, warp1 MMA, warps 2-5 epilogue

template <int BN>
struct TileCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  // epilogue staging for mirrored stores: per epilogue warp 32 rows x 64 bf16, rows padded to 144 bytes
  static constexpr int STG_ROW = 144;
  static constexpr int STG_WARP = 32 * STG_ROW;
  static constexpr int STG_OFF = STAGES * STAGE_BYTES + 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + 4 * STG_WARP;
};

struct WorkItem {
  int mb, nb, kb0, kb1, group;
  bool valid;
};

__device__ __forceinline__ WorkItem decode_item(const GemmParams& p, int item) {
  WorkItem w;
  w.group = 0;
  w.valid = true;
  int t;
  if (p.k_group_offsets != nullptr) {
    const int per = p.m_tiles * p.n_tiles;
    w.group = item / per;
    t = item - w.group * per;
    w.kb0 = p.k_group_offsets[w.group] / BK;
    w.kb1 = p.k_group_offsets[w.group + 1] / BK;
    if (w.kb1 <= w.kb0) w.valid = false;
  } else {
    // tile-fastest: the items that run at the same time are different tiles over the same K range, so they
    // share A and B panels in L2
    const int mn = p.m_tiles * p.n_tiles;
    const int ks = item / mn;
    t = item - ks * mn;
    w.kb0 = ks * p.kb_per_split;
    w.kb1 = min(p.kblocks, w.kb0 + p.kb_per_split);
  }
  const int per_group = p.group_m * p.n_tiles;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m_first = g * p.group_m;
  const int gsize = min(p.group_m, p.m_tiles - m_first);
  w.mb = m_first + r % gsize;
  w.nb = r / gsize;
  if (p.tile_group != nullptr) {
    w.group = p.tile_group[w.mb];
    if (w.group < 0) w.valid = false;
  }
  return w;
}

// The work items of one CTA pair, in the order in which its three roles walk them: items first, first + count,
// first + 2 count, ... of p.total_items, skipping the invalid ones.
struct ItemWalk {
  int item, stride;
  __device__ ItemWalk(int first, int count) : item(first), stride(count) {}
  __device__ bool next(const GemmParams& p, WorkItem& w) {
    while (item < p.total_items) {
      w = decode_item(p, item);
      item += stride;
      if (w.valid) return true;
    }
    return false;
  }
};

// One accumulator slab of 128 rows x BN columns: the four epilogue warps drain it from TMEM (warp quadrant q
// reads lanes 32q..32q+31 at `taddr`) and run the epilogue selected by p.epi.  m0 = first global row of the slab,
// n0 = first global column, nb = index of the N tile (partial-softmax slot), stg_warp = this warp's staging.
template <int BN>
__device__ __forceinline__ void epilogue_slab(const GemmParams& p, int m0, int n0, int nb, uint32_t taddr,
                                              long long c_off, uint8_t* stg_warp, int q, int lane) {
  using Cfg = TileCfg<BN>;
  const int row = m0 + q * 32 + lane;
  const bool row_ok = row < p.M;

  // per-row state of the streaming-softmax epilogues
  float run_max = -INFINITY, run_sum = 0.f;
  long long tgt = -1;
  float row_lse = 0.f, row_g = 0.f;
  if (p.epi == EPI_LSE_PARTIAL && row_ok) tgt = p.targets[row];
  if (p.epi == EPI_SOFTMAX_GRAD && row_ok) {
    tgt = p.targets[row];
    row_lse = p.lse[row];
    row_g = p.gscale[row];
  }

#pragma unroll 1
  for (int c = 0; c < BN; c += 32) {
    uint32_t r[32];
    __syncwarp();
    tmem_ld_32x32(taddr + c, r);
    tmem_ld_wait();
    const int col0 = n0 + c;
    if (p.staged_store) {
      // Staged bf16 store (N % 64 == 0): two 32-column chunks of this warp's 32 rows are staged in
      // shared memory, then written out as 128-byte row segments (8 lanes per row) to the local C and
      // to every mirror: full-line stores keep the L2 / NVLink writes efficient.
      if (col0 < p.N) {
        uint8_t* stg = stg_warp;
        uint8_t* mine = stg + lane * Cfg::STG_ROW + (c & 32) * 2;
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[g8 * 8 + 0]) * p.alpha, __uint_as_float(r[g8 * 8 + 1]) * p.alpha);
          o.y = pack_bf16x2(__uint_as_float(r[g8 * 8 + 2]) * p.alpha, __uint_as_float(r[g8 * 8 + 3]) * p.alpha);
          o.z = pack_bf16x2(__uint_as_float(r[g8 * 8 + 4]) * p.alpha, __uint_as_float(r[g8 * 8 + 5]) * p.alpha);
          o.w = pack_bf16x2(__uint_as_float(r[g8 * 8 + 6]) * p.alpha, __uint_as_float(r[g8 * 8 + 7]) * p.alpha);
          *reinterpret_cast<uint4*>(mine + g8 * 16) = o;
        }
        if (c & 32) {
          __syncwarp();
          const int cbase = n0 + (c & ~63);
#pragma unroll 1
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3), ch = lane & 7;
            const int grow = m0 + q * 32 + rr;
            if (grow < p.M) {
              const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * Cfg::STG_ROW + ch * 16);
              const long long off = c_off + static_cast<long long>(grow) * p.ldc + cbase + ch * 8;
              if (p.row_addr != nullptr) {
                // per-row destination (MoE combine): the row's home buffer gets it, address 0 drops the row
                const long long dst = p.row_addr[grow];
                if (dst != 0) *reinterpret_cast<uint4*>(dst + static_cast<long long>(cbase + ch * 8) * 2) = o;
              } else if (p.scatter_rows > 0) {
                // reduce-scatter epilogue: the row block's owner gets the tile, nobody else
                *reinterpret_cast<uint4*>(
                    reinterpret_cast<__nv_bfloat16*>(p.scatter_base[grow / p.scatter_rows]) + off) = o;
              } else {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + off) = o;
#pragma unroll 1
                for (int m = 0; m < p.n_mirror; ++m)
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.mirror[m]) + off) = o;
              }
            }
          }
          __syncwarp();
        }
      }
      continue;
    }
    if (!row_ok || col0 >= p.N) continue;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
    if (p.epi == EPI_STORE_BF16) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        if (col0 + g8 * 8 < p.N) {
          uint4 o;
          o.x = pack_bf16x2(v[g8 * 8 + 0], v[g8 * 8 + 1]);
          o.y = pack_bf16x2(v[g8 * 8 + 2], v[g8 * 8 + 3]);
          o.z = pack_bf16x2(v[g8 * 8 + 4], v[g8 * 8 + 5]);
          o.w = pack_bf16x2(v[g8 * 8 + 6], v[g8 * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + g8 * 8) = o;
        }
      }
    } else if (p.epi == EPI_STORE_F32) {
      float* dst = reinterpret_cast<float*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
      for (int g4 = 0; g4 < 8; ++g4) {
        if (col0 + g4 * 4 < p.N)
          *reinterpret_cast<float4*>(dst + g4 * 4) =
              make_float4(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2], v[g4 * 4 + 3]);
      }
    } else if (p.epi == EPI_ATOMIC_F32) {
      float* dst = reinterpret_cast<float*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
      for (int g4 = 0; g4 < 8; ++g4) {
        if (col0 + g4 * 4 < p.N)
          red_add_v4_f32(dst + g4 * 4, v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2], v[g4 * 4 + 3]);
      }
    } else if (p.epi == EPI_LSE_PARTIAL) {
      // streaming max / sum-exp over this tile's columns; pick the target logit
      float cmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) cmax = fmaxf(cmax, v[i]);
      const float nmax = fmaxf(run_max, cmax);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) s += __expf(v[i] - nmax);
      run_sum = run_sum * __expf(run_max - nmax) + s;
      run_max = nmax;
      if (tgt >= col0 && tgt < col0 + 32) {
        float tv = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i == tgt) tv = v[i];
        p.tgt_logit[row] = tv;
      }
    } else {  // EPI_SOFTMAX_GRAD: d = g * (onehot - exp(logit - lse)) as bf16
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float pr = __expf(v[i] - row_lse);
        v[i] = row_g * (((col0 + i) == tgt ? 1.f : 0.f) - pr);
      }
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        if (col0 + g8 * 8 < p.N) {
          uint4 o;
          o.x = pack_bf16x2(v[g8 * 8 + 0], v[g8 * 8 + 1]);
          o.y = pack_bf16x2(v[g8 * 8 + 2], v[g8 * 8 + 3]);
          o.z = pack_bf16x2(v[g8 * 8 + 4], v[g8 * 8 + 5]);
          o.w = pack_bf16x2(v[g8 * 8 + 6], v[g8 * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + g8 * 8) = o;
        }
      }
    }
  }
  if (p.epi == EPI_LSE_PARTIAL && row_ok) {
    p.part_max[static_cast<long long>(nb) * p.M + row] = run_max;
    p.part_sum[static_cast<long long>(nb) * p.M + row] = run_sum;
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const GemmParams p) {
  using Cfg = TileCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                       // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;        // [STAGES]
  uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;    // [2]
  uint64_t* tempty_bar = bars + 2 * Cfg::STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_items = p.total_items;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;         // stages with a copy that may still be in flight
      uint32_t armed_parity = 0;  // parity of that copy's phase
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const WorkItem w = decode_item(p, item);
        if (!w.valid) continue;
        const int m0 = w.mb * BM;
        const int n0 = w.nb * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
            if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), &tmA, &full_bar[stage], m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0 + w.group * p.b_group_rows);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + 64 * j,
                          k0 + w.group * p.b_group_rows);
          }
          armed |= (1u << stage);
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        // leave no copy in flight: wait (bounded) for every armed stage to land
        for (int s = 0; s < Cfg::STAGES; ++s) {
          if (armed & (1u << s)) {
            int dummy = 0;
            mbar_wait_bounded(&full_bar[s], (armed_parity >> s) & 1, &dummy);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, /*bf16*/ 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // K-major: 8-row groups are 1024 B apart; one UMMA_K step = 32 B along the row.
      // MN-major: 64-element MN groups are (64*BK*2) B apart (LBO), 8-row K groups 1024 B (SBO);
      //           one UMMA_K step = 16 K rows = 2048 B.
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 2048 : 32;
      constexpr uint32_t B_KSTEP = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const WorkItem w = decode_item(p, item);
        if (!w.valid) continue;
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = umma_smem_desc(sa + k * A_KSTEP, A_LBO, 1024);
            const uint64_t bd = umma_smem_desc(sb + k * B_KSTEP, B_LBO, 1024);
            umma_bf16(tmem_d, ad, bd, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees this smem stage when the MMAs retire
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete
        ++local_tile;
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    int local_tile = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const WorkItem w = decode_item(p, item);
      if (!w.valid) continue;
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      bool ok = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      epilogue_slab<BN>(p, w.mb * BM, w.nb * BN, w.nb, taddr, static_cast<long long>(w.group) * p.c_group_stride,
                        smem + Cfg::STG_OFF + q * Cfg::STG_WARP, q, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      ++local_tile;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair kernel: 256 x 256 x 64 tiles on two SMs (cluster of two CTAs, cta_group::2).
//
// A single UMMA spans the pair: CTA r stages rows [128 r, 128 r + 128) of the A tile and rows
// [128 r, 128 r + 128) of the B (N) tile, and holds rows [128 r, 128 r + 128) of the accumulator in its own
// TMEM.  Per k-block each SM therefore moves 32 KB through shared memory for 256 x 256 x 64 MACs of the pair,
// against 48 KB for 128 x 256 x 64 in the single-CTA kernel: half the shared-memory traffic per FLOP, and a
// six-stage ring in the same footprint.
//
// Barriers (every CTA owns a set at the same offsets):
//   full[s]   of the even CTA: one arrival (its producer's expect_tx of both CTAs' bytes) + both CTAs' TMA bytes
//   empty[s]  of each CTA: the even CTA's MMA thread commits to both (multicast commit)
//   tfull[a]  of each CTA: committed to both by the MMA thread when a tile's accumulator is complete
//   tempty[a] of the even CTA: 8 arrivals, one per epilogue warp of the pair
// Grouped (MoE) modes and CTA-limited launches stay on the single-CTA kernel.
// ---------------------------------------------------------------------------
struct PairCfg {
  static constexpr int BN = 256;
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = 128 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int TMEM_COLS = 512;
  static constexpr int STG_WARP = TileCfg<256>::STG_WARP;
  static constexpr int STG_OFF = STAGES * STAGE_BYTES + 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + 4 * STG_WARP;
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using Cfg = PairCfg;
  constexpr int BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::STAGES;
  uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;
  uint64_t* tempty_bar = bars + 2 * Cfg::STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = its peer
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before either CTA signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      ItemWalk walk(pair, n_pairs);
      WorkItem w;
      while (ok && walk.next(p, w)) {
        const int m0 = w.mb * 256 + static_cast<int>(rank) * 128;   // this CTA's rows of A
        const int n0 = w.nb * BN + static_cast<int>(rank) * 128;    // this CTA's rows of B
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
            if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
          const uint32_t fb = mapa_cluster(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * (64 * BK * 2), &tmA, fb, m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmB, fb, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + j * (64 * BK * 2), &tmB, fb, n0 + 64 * j, k0);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        // A wait ran out somewhere in the pair.  This CTA's copies report to the even CTA's barriers, so it
        // cannot wait on them itself: give the copies in flight a bounded time to land before the CTA ends.
        const long long t0 = clock64();
        while (clock64() - t0 < (1ll << 21)) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(256, BN, /*bf16*/ 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 2048 : 32;
      constexpr uint32_t B_KSTEP = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      ItemWalk walk(pair, n_pairs);
      WorkItem w;
      while (ok && walk.next(p, w)) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = umma_smem_desc(sa + k * A_KSTEP, A_LBO, 1024);
            const uint64_t bd = umma_smem_desc(sb + k * B_KSTEP, B_LBO, 1024);
            umma_bf16_pair(tmem_d, ad, bd, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage], 3);  // frees this stage in both CTAs when the MMAs retire
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc], 3);  // accumulator complete, in both CTAs
        ++local_tile;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
    const int q = warp & 3;
    int local_tile = 0;
    ItemWalk walk(pair, n_pairs);
    WorkItem w;
    while (walk.next(p, w)) {
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      bool ok = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          if (!*abort_flag) atomicCAS(p.status, 0, ERR_WAIT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      epilogue_slab<BN>(p, w.mb * 256 + static_cast<int>(rank) * 128, w.nb * BN, w.nb, taddr, 0,
                        smem + Cfg::STG_OFF + q * Cfg::STG_WARP, q, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&tempty_bar[acc]), 0));
      ++local_tile;
    }
  }

  // Neither CTA may leave (or free tensor memory) while its peer can still signal its barriers or while
  // MMAs of the pair may still write its TMEM: every role of both CTAs ends here.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D bf16 tensor map with 128-byte swizzle. `inner` is the contiguous extent.
static int encode_tensor_map_2d_impl(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                                     uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                                     uint32_t box_outer);
static inline int encode_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                                       uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                                       uint32_t box_outer) {
  return encode_tensor_map_2d_impl(out, base, elem_bytes, inner, outer, row_stride_bytes, box_inner, box_outer);
}

// A tensor map is a pure function of (base, element size, extents, row stride, box): training re-issues the same
// few hundred (pointer, shape) pairs every step - weights, the flat gradient, cached activation buffers - so the
// encoded maps are kept in a small per-thread table (the forward and the autograd thread each have one; no lock)
// and the driver call is made only on a miss.
namespace {
struct MapKey {
  const void* base;
  uint64_t inner, outer, stride;
  uint32_t box_inner, box_outer;
  int elem;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride &&
           box_inner == o.box_inner && box_outer == o.box_outer && elem == o.elem;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int MAP_CACHE_SLOTS = 8192;  // power of two
inline uint64_t map_hash(const MapKey& k) {
  uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
  h ^= (k.inner + 0x632BE59BD9B4E019ull) * 0xC2B2AE3D27D4EB4Full;
  h ^= (k.outer << 20) ^ (k.stride << 7) ^ (static_cast<uint64_t>(k.box_inner) << 40) ^
       (static_cast<uint64_t>(k.box_outer) << 52) ^ static_cast<uint64_t>(k.elem);
  h ^= h >> 29;
  return h * 0xBF58476D1CE4E5B9ull;
}
}  // namespace

int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  static const bool cache_on = [] { const char* e = getenv("CVERL_B200_TMAP_CACHE"); return !(e && e[0] == '0'); }();
  static thread_local MapSlot* table = nullptr;
  const MapKey key{base, inner, outer, row_stride_bytes, box_inner, box_outer, elem_bytes};
  MapSlot* slot = nullptr;
  if (cache_on) {
    if (!table) table = static_cast<MapSlot*>(calloc(MAP_CACHE_SLOTS, sizeof(MapSlot)));
    if (table) {
      uint64_t i = map_hash(key) & (MAP_CACHE_SLOTS - 1);
      for (int probe = 0; probe < 8; ++probe, i = (i + 1) & (MAP_CACHE_SLOTS - 1)) {
        if (table[i].used && table[i].key == key) {
          *out = table[i].map;
          return 0;
        }
        if (!table[i].used) {
          slot = &table[i];
          break;
        }
      }
      if (!slot) slot = &table[map_hash(key) & (MAP_CACHE_SLOTS - 1)];  // full neighbourhood: overwrite
    }
  }
  const int rc = encode_tensor_map_2d(out, base, elem_bytes, inner, outer, row_stride_bytes, box_inner, box_outer);
  if (rc == 0 && slot) {
    slot->key = key;
    slot->map = *out;
    slot->used = true;
  }
  return rc;
}

static int encode_tensor_map_2d_impl(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                                     uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                                     uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  // The driver call needs this thread to have a current context.  Autograd runs backward on
  // its own threads, where the runtime binds the primary context only at its first call.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[cverl_b200] cuTensorMapEncodeTiled failed (%d): base=%p elem=%d dims={%llu,%llu} stride=%llu box={%u,%u}\n",
            static_cast<int>(r), base, elem_bytes, static_cast<unsigned long long>(inner),
            static_cast<unsigned long long>(outer), static_cast<unsigned long long>(row_stride_bytes), box_inner,
            box_outer);
    return static_cast<int>(r);
  }
  return 0;
}

static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                  cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  static bool attr_set = false;
  auto kern = gemm_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  kern<<<grid, NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// Number of CTA pairs that can be resident at once (0 = pairs cannot be launched here).
template <bool A_MN, bool B_MN>
static int pair_capacity() {
  static int cached = -1;
  if (cached >= 0) return cached;
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return cached = 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * num_sms(), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  return cached = n;
}

template <bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int pairs,
                       cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<A_MN, B_MN>, ta, tb, p));
}

static int pair_capacity_for(bool a_mn, bool b_mn) {
  if (!a_mn && !b_mn) return pair_capacity<false, false>();
  if (!a_mn && b_mn) return pair_capacity<false, true>();
  if (a_mn && b_mn) return pair_capacity<true, true>();
  return pair_capacity<true, false>();
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_gemm_bf16(const CvbGemmArgs* a, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  if (!a->status) return -2;
  // vector stores / reductions in the epilogue need 16-byte aligned output rows
  if (a->C != nullptr) {
    const int64_t c_elem = (a->epi == EPI_STORE_BF16 || a->epi == EPI_SOFTMAX_GRAD) ? 2 : 4;
    if ((reinterpret_cast<uintptr_t>(a->C) & 15) || ((a->ldc * c_elem) & 15)) return -5;
  }
  // TMA needs 16-byte aligned bases and row strides
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) ||
      ((a->lda * 2) & 15) || ((a->ldb * 2) & 15))
    return -3;
  const int bn = a->block_n == 128 ? 128 : 256;
  // CTA-pair kernel (256 x 256 tiles over two SMs) for the plain, ungrouped shapes that fill at least one tile
  static const bool pair_off = [] { const char* e = getenv("CVERL_B200_GEMM_PAIR"); return e && e[0] == '0'; }();
  int pairs = 0;
  if (!pair_off && bn == 256 && !a->tile_group && !a->k_group_offsets && a->b_total_rows == 0 && a->max_ctas <= 0 &&
      a->M > 128 && a->N > 128)
    pairs = pair_capacity_for(a->a_mn != 0, a->b_mn != 0);
  const int bm = pairs > 0 ? 256 : BM;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.C = a->C;
  p.ldc = a->ldc;
  p.alpha = a->alpha;
  p.epi = a->epi;
  p.m_tiles = (a->M + bm - 1) / bm;
  p.n_tiles = (a->N + bn - 1) / bn;
  p.kblocks = (a->K + BK - 1) / BK;
  p.tile_group = a->tile_group;
  p.b_group_rows = a->b_group_rows;
  p.k_group_offsets = a->k_group_offsets;
  p.c_group_stride = a->c_group_stride;
  p.targets = a->targets;
  p.part_max = a->part_max;
  p.part_sum = a->part_sum;
  p.tgt_logit = a->tgt_logit;
  p.lse = a->lse;
  p.gscale = a->gscale;
  p.status = a->status;
  if (a->n_mirror < 0 || a->n_mirror > 7 || (a->n_mirror > 0 && (a->epi != EPI_STORE_BF16 || a->N % 64 != 0)))
    return -6;
  p.n_mirror = a->n_mirror;
  {
    // Default: stage every bf16 store whose N allows it.  CVERL_B200_GEMM_DIRECT_STORE=1 keeps the
    // register -> global path for comparison.
    static const bool direct = [] { const char* e = getenv("CVERL_B200_GEMM_DIRECT_STORE"); return e && e[0] == '1'; }();
    p.staged_store = (a->epi == EPI_STORE_BF16 && a->N % 64 == 0 &&
                      (a->n_mirror > 0 || a->scatter_rows > 0 || a->row_addr != nullptr || !direct)) ? 1 : 0;
  }
  p.row_addr = nullptr;
  if (a->row_addr != nullptr) {
    if (a->epi != EPI_STORE_BF16 || a->N % 64 != 0 || a->n_mirror != 0 || a->scatter_rows != 0 ||
        a->k_group_offsets != nullptr)
      return -6;
    p.row_addr = a->row_addr;
  }
  p.scatter_rows = 0;
  if (a->scatter_rows != 0) {
    // every 128-row slab of a tile must have one owner, and the table must cover all M rows
    if (a->scatter_rows < 0 || a->scatter_rows % 128 != 0 || a->epi != EPI_STORE_BF16 || a->N % 64 != 0 ||
        a->n_mirror != 0 || a->tile_group != nullptr || (a->M + a->scatter_rows - 1) / a->scatter_rows > 8)
      return -6;
    p.scatter_rows = a->scatter_rows;
    for (int b = 0; b < 8; ++b) p.scatter_base[b] = nullptr;
    for (int b = 0; b < (a->M + a->scatter_rows - 1) / a->scatter_rows; ++b) {
      if (!a->scatter_base[b] || (reinterpret_cast<uintptr_t>(a->scatter_base[b]) & 15)) return -6;
      p.scatter_base[b] = a->scatter_base[b];
    }
  }
  for (int m = 0; m < a->n_mirror; ++m) {
    if (!a->mirror[m] || (reinterpret_cast<uintptr_t>(a->mirror[m]) & 15)) return -6;
    p.mirror[m] = a->mirror[m];
  }
  const int sms = pairs > 0 ? pairs : num_sms();  // concurrent tiles
  int split = a->split_k;
  const int mn_tiles = p.m_tiles * p.n_tiles;
  if (a->k_group_offsets) {
    split = 1;
    p.total_items = mn_tiles * a->num_groups;
  } else {
    if (split <= 0) {  // auto: only atomically accumulating epilogues may split K
      split = 1;
      if (a->epi == EPI_ATOMIC_F32 && mn_tiles < 8 * sms) {
        // Few tiles and a long K (weight gradients): pick the split whose number of waves x k-blocks per item
        // is smallest; every item also pays for its pipeline fill and atomic epilogue (measured on the weight-
        // gradient shapes of the 0.8B model: worth about 24 k-blocks, a smaller figure over-splits wide outputs).
        static const int item_cost = [] { const char* e = getenv("CVERL_B200_GEMM_SPLIT_COST"); return e ? atoi(e) : 24; }();
        const int max_split = p.kblocks / 8 > 16 ? 16 : (p.kblocks / 8 > 0 ? p.kblocks / 8 : 1);
        long long best = -1;
        for (int s = 1; s <= max_split; ++s) {
          const long long waves = (static_cast<long long>(mn_tiles) * s + sms - 1) / sms;
          const long long cost = waves * ((p.kblocks + s - 1) / s + item_cost);
          if (best < 0 || cost < best) {
            best = cost;
            split = s;
          }
        }
      }
    }
    if (split > 1 && a->epi != EPI_ATOMIC_F32) return -4;
    if (split > p.kblocks) split = p.kblocks;
    p.kb_per_split = (p.kblocks + split - 1) / split;
    split = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;
    p.total_items = mn_tiles * split;
  }
  p.split_k = split;
  if (!a->k_group_offsets) p.kb_per_split = (p.kblocks + split - 1) / split;
  // rasterisation: walk group_m M-tiles per N-tile so that the CTAs running at
  // the same time share B tiles (weights) and a band of A tiles in L2
  p.group_m = a->group_m > 0 ? a->group_m : 16;
  if (p.group_m > p.m_tiles) p.group_m = p.m_tiles;

  CUtensorMap ta, tb;
  int rc;
  // A: K-major [rows = a_rows, K] or MN-major [rows = K, M]
  if (!a->a_mn)
    rc = make_tensor_map_2d(&ta, a->A, 2, a->K, a->M, a->lda * 2, BK, BM);
  else
    rc = make_tensor_map_2d(&ta, a->A, 2, a->M, a->K, a->lda * 2, 64, BK);
  if (rc) return -10 - (rc > 0 ? 0 : 1);
  const uint64_t b_rows = a->b_total_rows > 0 ? a->b_total_rows : (a->b_mn ? a->K : a->N);
  if (!a->b_mn)
    rc = make_tensor_map_2d(&tb, a->B, 2, a->K, b_rows, a->ldb * 2, BK, pairs > 0 ? 128 : bn);
  else
    rc = make_tensor_map_2d(&tb, a->B, 2, a->N, b_rows, a->ldb * 2, 64, BK);
  if (rc) return -12;

  int grid = p.total_items < sms ? p.total_items : sms;
  if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;
  if (grid <= 0) return 0;
  if (pairs > 0) {
    if (!a->a_mn && !a->b_mn) return launch_pair<false, false>(ta, tb, p, grid, stream);
    if (!a->a_mn && a->b_mn) return launch_pair<false, true>(ta, tb, p, grid, stream);
    if (a->a_mn && a->b_mn) return launch_pair<true, true>(ta, tb, p, grid, stream);
    return launch_pair<true, false>(ta, tb, p, grid, stream);
  }

#define CVB_LAUNCH(BN_)                                                            \
  do {                                                                             \
    if (!a->a_mn && !a->b_mn) return launch<BN_, false, false>(ta, tb, p, grid, stream); \
    if (!a->a_mn && a->b_mn) return launch<BN_, false, true>(ta, tb, p, grid, stream);   \
    if (a->a_mn && a->b_mn) return launch<BN_, true, true>(ta, tb, p, grid, stream);     \
    return launch<BN_, true, false>(ta, tb, p, grid, stream);                      \
  } while (0)
  if (bn == 256) CVB_LAUNCH(256);
  CVB_LAUNCH(128);
#undef CVB_LAUNCH
}
