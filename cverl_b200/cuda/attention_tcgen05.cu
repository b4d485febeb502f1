// Causal / blockwise GQA attention on tcgen05 (head dim 128 or 256), forward pass.
//
// One CTA per (128-query block, query head, batch).  Q stays in shared memory; K / V stream through two
// TMA buffers in blocks of 64 keys.  Per key block:
//     S  = Q K^T            tcgen05 MMA, M = 128, N = 64, K = D         -> TMEM
//     P  = exp2(S c - m)    one thread per query row (a TMEM lane is a row: no shuffles), running max m
//                           and sum l in registers, bf16 P written to shared memory
//     O += P V              tcgen05 MMA, M = 128, N = D, K = 64, V read MN-major from the TMA tile
// The accumulator O lives in TMEM for the whole CTA; it is rescaled only when a row's maximum has grown
// by more than 2^8 since the last rescale (the stale maximum keeps P <= 256, exactness is kept because
// l uses the same maximum).  Query / key position offsets make the same kernel serve the hops of
// context-parallel ring attention: it returns the un-merged (O, LSE) of one key range.
//
// The reference calls at::scaled_dot_product_attention (src/model/qwen3_5_text.cc:1068-1075) and, for
// context parallelism, a scalar SIMT kernel (cuda/cp_attention_cuda.cu).
#include "ptx.cuh"
#include "gemm_tcgen05.h"

namespace cvb {

constexpr int AT_THREADS = 128;
constexpr int AT_BQ = 128;   // queries per CTA
constexpr int AT_BK = 64;    // keys per block

template <int D>
struct AttSmem {
  static constexpr int Q = 0;                       // D/64 boxes [128 x 64]
  static constexpr int K = D * 256;                 // 2 buffers x D/64 boxes [64 x 64]
  static constexpr int V = K + 2 * D * 128;
  static constexpr int P = V + 2 * D * 128;         // [128 x 64] bf16
  static constexpr int BARS = P + 16384;
  static constexpr int BYTES = BARS + 256 + 1024;
};

struct AttArgs {
  __nv_bfloat16* out;   // [B, Sq, Hq, D]
  float* lse;           // [B, Hq, Sq]  natural-log LSE of the scaled scores (-inf for a fully masked row)
  int Sq, Skv, Hq, Hkv, B;
  float scale_log2;     // softmax scale * log2(e)
  int causal;
  long long q_pos0, k_pos0;   // positions of query 0 and key 0 (causal: key_pos <= query_pos)
  int* status;
};

__device__ __forceinline__ uint32_t asw128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttArgs a) {
  using SM = AttSmem<D>;
  constexpr int NB = D / 64;            // 64-column boxes per row
  constexpr uint32_t KV_BYTES = 2u * D * 128u;  // one K block + one V block
  constexpr uint32_t TCOLS = (D == 256) ? 512 : 256;  // S (64) + O (D), rounded up to a power of two
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BARS);
  uint64_t *bar_q = bars, *bar_kv = bars + 1 /* [2] */, *bar_s = bars + 3, *bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  // 1-D grid, last query block first: under the causal mask it sees the most keys, so the longest CTAs are
  // scheduled first and the launch ends with short ones.
  const int per_block = a.Hq * a.B;
  const int q0 = (a.Sq / AT_BQ - 1 - static_cast<int>(blockIdx.x / per_block)) * AT_BQ;
  const int h = (blockIdx.x % per_block) % a.Hq;
  const int hk = h / (a.Hq / a.Hkv);
  const long long b = (blockIdx.x % per_block) / a.Hq;
  const uint32_t sb = smem_u32(smem);

  // key blocks this query block can see
  int nblk = a.Skv / AT_BK;
  if (a.causal) {
    const long long last_q = a.q_pos0 + q0 + AT_BQ - 1;
    const long long lim = last_q - a.k_pos0;         // largest visible key index
    nblk = lim < 0 ? 0 : static_cast<int>(min(static_cast<long long>(nblk), lim / AT_BK + 1));
  }

  auto load_kv = [&](int j) {
    const int buf = j & 1;
    const int krow = static_cast<int>(b * a.Skv + static_cast<long long>(j) * AT_BK);
    mbar_arrive_expect_tx(&bar_kv[buf], KV_BYTES);
#pragma unroll
    for (int c = 0; c < NB; ++c) {
      tma_load_2d(smem + SM::K + buf * (D * 128) + c * 8192, &tmK, &bar_kv[buf], hk * D + c * 64, krow);
      tma_load_2d(smem + SM::V + buf * (D * 128) + c * 8192, &tmV, &bar_kv[buf], hk * D + c * 64, krow);
    }
  };

  if (tid == 0) {
    mbar_init(bar_q, 1); mbar_init(&bar_kv[0], 1); mbar_init(&bar_kv[1], 1); mbar_init(bar_s, 1); mbar_init(bar_o, 1);
    *abort_flag = 0;
    mbar_fence_init();
    if (nblk > 0) {
      mbar_arrive_expect_tx(bar_q, D * 256);
      const int qrow = static_cast<int>(b * a.Sq + q0);
#pragma unroll
      for (int c = 0; c < NB; ++c) tma_load_2d(smem + SM::Q + c * 16384, &tmQ, bar_q, h * D + c * 64, qrow);
      load_kv(0);
      if (nblk > 1) load_kv(1);
    }
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, TCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  constexpr uint32_t TC_S = 0, TC_O = 64;

  float m = -INFINITY, m_used = -INFINITY, l = 0.f;
  const long long qpos = a.q_pos0 + q0 + tid;
  bool ok = true;
  if (nblk > 0) {
    if (!mbar_wait_bounded(bar_q, 0, abort_flag)) {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_FULL);
      *abort_flag = 1;
    }
    __syncthreads();
    ok = !*abort_flag;
  }
  for (int j = 0; j < nblk && ok; ++j) {
    const int buf = j & 1;
    const uint32_t ph = (j >> 1) & 1, pj = j & 1;
    // ---- S = Q K^T -------------------------------------------------------------------------------------
    if (tid == 0) {
      if (mbar_wait_bounded(&bar_kv[buf], ph, abort_flag)) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(128, AT_BK, 1, 0, 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kb = k >> 2, ks = (k & 3) * 32;
          umma_bf16(tmem_base + TC_S, umma_smem_desc(sb + SM::Q + kb * 16384 + ks, 16, 1024),
                    umma_smem_desc(sb + SM::K + buf * (D * 128) + kb * 8192 + ks, 16, 1024), idesc, k > 0);
        }
        umma_commit(bar_s);
      } else {
        if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_FULL);
        *abort_flag = 1;
      }
    }
    if (!mbar_wait_bounded(bar_s, pj, abort_flag)) {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
      *abort_flag = 1;
    }
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    // ---- softmax of this block, one row per thread -------------------------------------------------------
    {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem + TC_S, r0);
      tmem_ld_32x32(tmem + TC_S + 32, r1);
      tmem_ld_wait();
      const long long kbase = a.k_pos0 + static_cast<long long>(j) * AT_BK;
      const bool diag = a.causal && (kbase + AT_BK - 1 > a.q_pos0 + q0);
      // number of visible keys of this row in the block
      int vis = AT_BK;
      if (diag) {
        const long long v64 = qpos - kbase + 1;
        vis = v64 < 0 ? 0 : (v64 > AT_BK ? AT_BK : static_cast<int>(v64));
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i < vis) mx = fmaxf(mx, __uint_as_float(r0[i]));
        if (32 + i < vis) mx = fmaxf(mx, __uint_as_float(r1[i]));
      }
      mx *= a.scale_log2;   // scale > 0
      m = fmaxf(m, mx);
      const bool want = (m > m_used + 8.f) || (m_used == -INFINITY && m > -INFINITY);
      if (__any_sync(0xffffffffu, want)) {   // warp-uniform: tcgen05.ld / st are warp-collective
        const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m);
        m_used = m;
        l *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tmem_ld_32x32(tmem + TC_O + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem + TC_O + c0, o);
          }
          tmem_st_wait();
        }
      }
      float p[64];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        p[i] = (i < vis) ? exp2f(__uint_as_float(r0[i]) * a.scale_log2 - m_used) : 0.f;
        p[32 + i] = (32 + i < vis) ? exp2f(__uint_as_float(r1[i]) * a.scale_log2 - m_used) : 0.f;
        sum += p[i] + p[32 + i];
      }
      l += sum;
      uint8_t* prow = smem + SM::P;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 u;
        u.x = pack_bf16x2(p[8 * c + 0], p[8 * c + 1]);
        u.y = pack_bf16x2(p[8 * c + 2], p[8 * c + 3]);
        u.z = pack_bf16x2(p[8 * c + 4], p[8 * c + 5]);
        u.w = pack_bf16x2(p[8 * c + 6], p[8 * c + 7]);
        *reinterpret_cast<uint4*>(prow + asw128(tid, c)) = u;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // ---- O += P V ----------------------------------------------------------------------------------------
    if (tid == 0) {
      constexpr uint32_t idesc = umma_idesc(128, D, 1, 0, 1);
#pragma unroll
      for (int k = 0; k < AT_BK / 16; ++k)
        umma_bf16(tmem_base + TC_O, umma_smem_desc(sb + SM::P + k * 32, 16, 1024),
                  umma_smem_desc(sb + SM::V + buf * (D * 128) + k * 2048, 8192, 1024), idesc, (j > 0 || k > 0));
      umma_commit(bar_o);
    }
    if (!mbar_wait_bounded(bar_o, pj, abort_flag)) {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
      *abort_flag = 1;
    }
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 2 < nblk) load_kv(j + 2);   // this buffer is free again
  }
  if (!ok && tid == 0) {   // leave no copy in flight
    int dummy = 0;
    mbar_wait_bounded(&bar_kv[0], 0, &dummy);
    mbar_wait_bounded(&bar_kv[1], 0, &dummy);
  }
  if (ok) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* orow = a.out + ((b * a.Sq + q0 + tid) * a.Hq + h) * D;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t o[32];
      if (nblk > 0) {
        tmem_ld_32x32(tmem + TC_O + c0, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 u;
        u.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
        u.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
        u.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
        u.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
        *reinterpret_cast<uint4*>(orow + c0 + 8 * c) = u;
      }
    }
    a.lse[(b * a.Hq + h) * a.Sq + q0 + tid] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TCOLS);
  }
}

template <int D>
static int launch_fwd(const void* q, const void* k, const void* v, void* out, float* lse, long long B, int Sq,
                      int Skv, int Hq, int Hkv, float scale, int causal, long long q_pos0, long long k_pos0,
                      int* status, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  if (make_tensor_map_2d(&mq, q, 2, static_cast<uint64_t>(Hq) * D, B * Sq, static_cast<uint64_t>(Hq) * D * 2, 64, 128) ||
      make_tensor_map_2d(&mk, k, 2, static_cast<uint64_t>(Hkv) * D, B * Skv, static_cast<uint64_t>(Hkv) * D * 2, 64, 64) ||
      make_tensor_map_2d(&mv, v, 2, static_cast<uint64_t>(Hkv) * D, B * Skv, static_cast<uint64_t>(Hkv) * D * 2, 64, 64))
    return -10;
  AttArgs a{};
  a.out = static_cast<__nv_bfloat16*>(out); a.lse = lse; a.Sq = Sq; a.Skv = Skv; a.Hq = Hq; a.Hkv = Hkv;
  a.B = static_cast<int>(B);
  a.scale_log2 = scale * 1.4426950408889634f; a.causal = causal; a.q_pos0 = q_pos0; a.k_pos0 = k_pos0;
  a.status = status;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attention_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             AttSmem<D>::BYTES) != cudaSuccess)
      return -11;
    attr = true;
  }
  dim3 grid(static_cast<unsigned>((Sq / AT_BQ) * Hq * B));
  attention_fwd_kernel<D><<<grid, AT_THREADS, AttSmem<D>::BYTES, st>>>(mq, mk, mv, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace cvb

using namespace cvb;

// q: bf16 [B, Sq, Hq, D]; k, v: bf16 [B, Skv, Hkv, D] (all contiguous); out: bf16 [B, Sq, Hq, D];
// lse: fp32 [B, Hq, Sq].  D in {128, 256}; Sq % 128 == 0; Skv % 64 == 0; Hq % Hkv == 0.
// causal != 0 masks keys whose position (k_pos0 + index) exceeds the query's (q_pos0 + index).
extern "C" int cvb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, long long B,
                                 int Sq, int Skv, int Hq, int Hkv, int D, float scale, int causal, long long q_pos0,
                                 long long k_pos0, int* status, void* stream) {
  if (B <= 0 || Sq <= 0 || Skv <= 0) return 0;
  if (Sq % AT_BQ || Skv % AT_BK || Hkv <= 0 || Hq % Hkv || !(scale > 0.f)) return -1;
  if (B * Sq > 0x7fffffffLL || B * Skv > 0x7fffffffLL) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 128) return launch_fwd<128>(q, k, v, out, lse, B, Sq, Skv, Hq, Hkv, scale, causal, q_pos0, k_pos0, status, st);
  if (D == 256) return launch_fwd<256>(q, k, v, out, lse, B, Sq, Skv, Hq, Hkv, scale, causal, q_pos0, k_pos0, status, st);
  return -1;
}

// =================================================================================================
// Backward.
//
// One CTA per (128-key block, query head, batch) walks the query blocks (64 queries) that can see it.
// Everything is computed transposed, keys on the TMEM lanes, so that each thread owns one key row:
//     S^T  = K Q^T          dP^T = V dO^T                    (M = 128 keys, N = 64 queries, K = D)
//     P^T  = exp2(S^T c - LSE_q)        dS^T = P^T (dP^T - Delta_q) * scale
//     dV  += P^T dO         dK  += dS^T Q                    (N = D, K = 64; dO / Q read MN-major)
//     dQ^T = K^T dS^T                                        (M = D in chunks of 128, N = 64, K = 128 keys)
// dV and dK stay in TMEM for the whole CTA; dQ^T of each (key block, query block) pair is added to a
// transposed fp32 buffer [B, Hq, D, Sq] with 16-byte vector reductions (a thread holds 64 consecutive
// queries of one d), and a last kernel turns that buffer into bf16 [B, Sq, Hq, D].
// TMEM has 512 columns: with D = 128 everything fits in one kernel (MODE 0); with D = 256 the work is
// split into a dV kernel (MODE 1: S^T, dV) and a dK / dQ kernel (MODE 2: S^T, dP^T, dK, dQ^T).
// A CTA walks the query blocks of EVERY query head of its GQA group, so dK / dV come out already summed.
// =================================================================================================
constexpr int AB_BKV = 128;  // keys per CTA
constexpr int AB_BQ = 64;    // queries per step
// Two warpgroups: warps w and w + 4 share TMEM lane quadrant w (the same 32 keys) and split the 32-column chunks
// of every TMEM -> registers hand-off between the two MMA rounds of a step.
constexpr int AB_THREADS = 256;

template <int D, int MODE>
struct AttBwdCfg {
  static constexpr bool NEED_V = MODE != 1;
  static constexpr bool NEED_PT = MODE != 2;
  static constexpr bool NEED_DS = MODE != 1;
  static constexpr int NBUF = (MODE == 2 && D == 256) ? 1 : 2;
  static constexpr int K = 0;                                   // D/64 boxes [128 x 64]
  static constexpr int V = K + D * 256;
  static constexpr int Q = V + (NEED_V ? D * 256 : 0);          // NBUF x D/64 boxes [64 x 64]
  static constexpr int DO = Q + NBUF * D * 128;
  static constexpr int PT = DO + NBUF * D * 128;                // [128 x 64] bf16
  static constexpr int DS = PT + (NEED_PT ? 16384 : 0);
  static constexpr int VEC = DS + (NEED_DS ? 16384 : 0);        // lse2[NBUF][64], delta[NBUF][64]
  static constexpr int BARS = VEC + 1024;
  static constexpr int BYTES = BARS + 256 + 1024;
  static constexpr uint32_t TC_S = 0, TC_DP = 64;
  static constexpr uint32_t TC_DV = (MODE == 1) ? 64 : 128;
  static constexpr uint32_t TC_DK = (MODE == 0) ? 128 + D : 128;
  static constexpr uint32_t TC_DQ = 384;
};

struct AttBwdArgs {
  const float* lse;      // [B, Hq, Sq] natural log
  const float* delta;    // [B, Hq, Sq] rowsum(dO * O)
  __nv_bfloat16* dk;     // [B, Skv, Hkv, D]
  __nv_bfloat16* dv;     // [B, Skv, Hkv, D]
  float* dqt;            // [B, Hq, D, Sq] fp32, zero-initialised, accumulated with reductions
  int Sq, Skv, Hq, Hkv, B;
  float scale, scale_log2;
  int causal;
  long long q_pos0, k_pos0;
  int* status;
};

template <int D, int MODE>
__global__ void __launch_bounds__(AB_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const AttBwdArgs a) {
  using C = AttBwdCfg<D, MODE>;
  constexpr int NB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BARS);
  uint64_t *bar_kv = bars, *bar_q = bars + 1 /* [2] */, *bar_1 = bars + 3, *bar_2 = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_lse2 = reinterpret_cast<float*>(smem + C::VEC);         // [NBUF][64]
  float* s_delta = s_lse2 + 2 * AB_BQ;

  const int tid = threadIdx.x;
  const int wg = tid >> 7;      // warpgroup: every second 32-column chunk
  const int lt = tid & 127;     // key row of this thread = its TMEM lane
  const int warp = lt >> 5;     // TMEM lane quadrant
  // 1-D grid with the key block slowest: causal key blocks near the start see the most queries, so the
  // longest CTAs are scheduled first and the tail of the launch consists of short ones.
  const int per_block = a.Hkv * a.B;                        // (kv head, batch) pairs per key block
  const int k0 = (blockIdx.x / per_block) * AB_BKV;
  const int hk = (blockIdx.x % per_block) % a.Hkv;
  const long long b = (blockIdx.x % per_block) / a.Hkv;
  const int group = a.Hq / a.Hkv;                           // query heads that share this kv head
  const uint32_t sb = smem_u32(smem);
  const long long kpos = a.k_pos0 + k0 + lt;

  const int nq = a.Sq / AB_BQ;
  int m_begin = 0;
  if (a.causal) {   // first query block with a query at or after this block's first key
    const long long need = a.k_pos0 + k0 - a.q_pos0 - (AB_BQ - 1);
    m_begin = need <= 0 ? 0 : static_cast<int>((need + AB_BQ - 1) / AB_BQ);
    if (m_begin > nq) m_begin = nq;
  }
  const int per_head = nq - m_begin;          // query blocks per head that see this key block
  const int steps = per_head * group;         // dK / dV accumulate over every query head of the GQA group

  auto load_q = [&](int it) {
    const int buf = it % C::NBUF;
    const int m = m_begin + it % per_head;
    const int h = hk * group + it / per_head;
    const int qrow = static_cast<int>(b * a.Sq + static_cast<long long>(m) * AB_BQ);
    mbar_arrive_expect_tx(&bar_q[buf], 2u * D * 128u);
#pragma unroll
    for (int c = 0; c < NB; ++c) {
      tma_load_2d(smem + C::Q + buf * (D * 128) + c * 8192, &tmQ, &bar_q[buf], h * D + c * 64, qrow);
      tma_load_2d(smem + C::DO + buf * (D * 128) + c * 8192, &tmDO, &bar_q[buf], h * D + c * 64, qrow);
    }
  };

  if (tid == 0) {
    mbar_init(bar_kv, 1); mbar_init(&bar_q[0], 1); mbar_init(&bar_q[1], 1); mbar_init(bar_1, 1); mbar_init(bar_2, 1);
    *abort_flag = 0;
    mbar_fence_init();
    if (steps > 0) {
      mbar_arrive_expect_tx(bar_kv, (C::NEED_V ? 2u : 1u) * D * 256u);
      const int krow = static_cast<int>(b * a.Skv + k0);
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        tma_load_2d(smem + C::K + c * 16384, &tmK, bar_kv, hk * D + c * 64, krow);
        if (C::NEED_V) tma_load_2d(smem + C::V + c * 16384, &tmV, bar_kv, hk * D + c * 64, krow);
      }
      load_q(0);
      if (C::NBUF == 2 && steps > 1) load_q(1);
    }
  }
  if (tid < 32) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  bool ok = true;
  if (steps > 0) {
    if (!mbar_wait_bounded(bar_kv, 0, abort_flag)) {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_FULL);
      *abort_flag = 1;
    }
    __syncthreads();
    ok = !*abort_flag;
  }
  for (int it = 0; it < steps && ok; ++it) {
    const int buf = it % C::NBUF;
    const int m = m_begin + it % per_head;
    const int h = hk * group + it / per_head;
    const uint32_t phq = (it / C::NBUF) & 1, pit = it & 1;
    const uint32_t qb = sb + C::Q + buf * (D * 128), dob = sb + C::DO + buf * (D * 128);
    // per-query scalars of this block
    if (tid < AB_BQ) {
      const long long qi = (b * a.Hq + h) * a.Sq + static_cast<long long>(m) * AB_BQ + tid;
      s_lse2[buf * AB_BQ + tid] = a.lse[qi] * 1.4426950408889634f;
      s_delta[buf * AB_BQ + tid] = a.delta[qi];
    }
    // ---- MMA phase 1: S^T = K Q^T (and dP^T = V dO^T) ---------------------------------------------------------
    if (tid == 0) {
      if (mbar_wait_bounded(&bar_q[buf], phq, abort_flag)) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(128, AB_BQ, 1, 0, 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kb = k >> 2, ks = (k & 3) * 32;
          umma_bf16(tmem_base + C::TC_S, umma_smem_desc(sb + C::K + kb * 16384 + ks, 16, 1024),
                    umma_smem_desc(qb + kb * 8192 + ks, 16, 1024), idesc, k > 0);
        }
        if (C::NEED_DS) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t kb = k >> 2, ks = (k & 3) * 32;
            umma_bf16(tmem_base + C::TC_DP, umma_smem_desc(sb + C::V + kb * 16384 + ks, 16, 1024),
                      umma_smem_desc(dob + kb * 8192 + ks, 16, 1024), idesc, k > 0);
          }
        }
        umma_commit(bar_1);
      } else {
        if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_FULL);
        *abort_flag = 1;
      }
    }
    if (!mbar_wait_bounded(bar_1, pit, abort_flag)) {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
      *abort_flag = 1;
    }
    __syncthreads();   // also publishes s_lse2 / s_delta
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    // ---- P^T and dS^T rows (one key per thread) ------------------------------------------------------------
    {
      const long long qbase = a.q_pos0 + static_cast<long long>(m) * AB_BQ;
      const bool diag = a.causal && (kpos > qbase);      // some query of the block is before this key
      // queries [first_vis, 64) see this key
      int first_vis = 0;
      if (diag) {
        const long long f = kpos - qbase;
        first_vis = f > AB_BQ ? AB_BQ : static_cast<int>(f);
      }
#pragma unroll 1
      for (int c0 = wg * 32; c0 < AB_BQ; c0 += 64) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tmem + C::TC_S + c0, rs);
        if (C::NEED_DS) tmem_ld_32x32(tmem + C::TC_DP + c0, rp);
        tmem_ld_wait();
        float p[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int qi = c0 + i;
          const float l2 = s_lse2[buf * AB_BQ + qi];
          const bool vis = qi >= first_vis && l2 > -INFINITY;
          p[i] = vis ? exp2f(__uint_as_float(rs[i]) * a.scale_log2 - l2) : 0.f;
          if (C::NEED_DS) ds[i] = p[i] * (__uint_as_float(rp[i]) - s_delta[buf * AB_BQ + qi]) * a.scale;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t off = asw128(lt, (c0 >> 3) + c);
          if (C::NEED_PT) {
            uint4 u;
            u.x = pack_bf16x2(p[8 * c + 0], p[8 * c + 1]); u.y = pack_bf16x2(p[8 * c + 2], p[8 * c + 3]);
            u.z = pack_bf16x2(p[8 * c + 4], p[8 * c + 5]); u.w = pack_bf16x2(p[8 * c + 6], p[8 * c + 7]);
            *reinterpret_cast<uint4*>(smem + C::PT + off) = u;
          }
          if (C::NEED_DS) {
            uint4 u;
            u.x = pack_bf16x2(ds[8 * c + 0], ds[8 * c + 1]); u.y = pack_bf16x2(ds[8 * c + 2], ds[8 * c + 3]);
            u.z = pack_bf16x2(ds[8 * c + 4], ds[8 * c + 5]); u.w = pack_bf16x2(ds[8 * c + 6], ds[8 * c + 7]);
            *reinterpret_cast<uint4*>(smem + C::DS + off) = u;
          }
        }
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // ---- MMA phase 2: dV += P^T dO, dK += dS^T Q, dQ^T = K^T dS^T -------------------------------------------
    if (tid == 0) {
      constexpr uint32_t id_acc = umma_idesc(128, D, 1, 0, 1);
      if (C::NEED_PT) {
#pragma unroll
        for (int k = 0; k < AB_BQ / 16; ++k)
          umma_bf16(tmem_base + C::TC_DV, umma_smem_desc(sb + C::PT + k * 32, 16, 1024),
                    umma_smem_desc(dob + k * 2048, 8192, 1024), id_acc, (it > 0 || k > 0));
      }
      if (C::NEED_DS) {
#pragma unroll
        for (int k = 0; k < AB_BQ / 16; ++k)
          umma_bf16(tmem_base + C::TC_DK, umma_smem_desc(sb + C::DS + k * 32, 16, 1024),
                    umma_smem_desc(qb + k * 2048, 8192, 1024), id_acc, (it > 0 || k > 0));
        constexpr uint32_t id_dq = umma_idesc(128, AB_BQ, 1, 1, 1);
#pragma unroll
        for (int ch = 0; ch < D / 128; ++ch) {
#pragma unroll
          for (int k = 0; k < AB_BKV / 16; ++k)
            umma_bf16(tmem_base + C::TC_DQ + ch * AB_BQ,
                      umma_smem_desc(sb + C::K + ch * 32768 + k * 2048, 16384, 1024),
                      umma_smem_desc(sb + C::DS + k * 2048, 16, 1024), id_dq, k > 0);
        }
      }
      umma_commit(bar_2);
    }
    if (!mbar_wait_bounded(bar_2, pit, abort_flag)) {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
      *abort_flag = 1;
    }
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && it + C::NBUF < steps) load_q(it + C::NBUF);   // Q / dO buffer is free again
    if (C::NEED_DS) {
      // dQ^T chunk rows: lane = d, 64 consecutive queries -> vector reductions into [B, Hq, D, Sq]
#pragma unroll 1
      for (int ch = 0; ch < D / 128; ++ch) {
        float* dst = a.dqt + ((b * a.Hq + h) * D + ch * 128 + lt) * static_cast<long long>(a.Sq) +
                     static_cast<long long>(m) * AB_BQ;
#pragma unroll 1
        for (int c0 = wg * 32; c0 < AB_BQ; c0 += 64) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + C::TC_DQ + ch * AB_BQ + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            red_add_v4_f32(dst + c0 + i, __uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                           __uint_as_float(r[i + 3]));
        }
      }
      tc_fence_before();
      __syncthreads();   // dQ^T columns are reused by the next step
      tc_fence_after();
    }
  }
  if (!ok && tid == 0) {   // leave no copy in flight
    int dummy = 0;
    mbar_wait_bounded(&bar_q[0], 0, &dummy);
    mbar_wait_bounded(&bar_q[1], 0, &dummy);
  }
  if (ok) {
    const long long orow = ((b * a.Skv + k0 + lt) * a.Hkv + hk) * D;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      if ((which == 0 && !C::NEED_PT) || (which == 1 && !C::NEED_DS)) continue;
      __nv_bfloat16* dst = (which == 0 ? a.dv : a.dk) + orow;
      const uint32_t tc = which == 0 ? C::TC_DV : C::TC_DK;
#pragma unroll 1
      for (int c0 = wg * 32; c0 < D; c0 += 64) {
        uint32_t o[32];
        if (steps > 0) {
          tmem_ld_32x32(tmem + tc + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]), __uint_as_float(o[8 * c + 1]));
          u.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]), __uint_as_float(o[8 * c + 3]));
          u.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]), __uint_as_float(o[8 * c + 5]));
          u.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]), __uint_as_float(o[8 * c + 7]));
          *reinterpret_cast<uint4*>(dst + c0 + 8 * c) = u;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid < 32) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, q] = sum_d dO[b, q, h, d] * O[b, q, h, d]     (one warp per (token, head) row)
__global__ void __launch_bounds__(256)
attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                       float* __restrict__ delta, long long B, int Sq, int Hq, int D) {
  const long long row = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;   // (b*Sq + q)*Hq + h
  const int lane = threadIdx.x & 31;
  if (row >= B * Sq * Hq) return;
  const __nv_bfloat16* po = o + row * D;
  const __nv_bfloat16* pd = d_o + row * D;
  float acc = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    const uint4 a = *reinterpret_cast<const uint4*>(po + c), g = *reinterpret_cast<const uint4*>(pd + c);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __bfloat1622float2(pa[j]), y = __bfloat1622float2(pg[j]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long long h = row % Hq, bq = row / Hq, q = bq % Sq, b = bq / Sq;
    delta[(b * Hq + h) * Sq + q] = acc;
  }
}

// dq[b, q, h, d] (bf16) = dqt[b, h, d, q] (fp32): 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
attention_dq_transpose_kernel(const float* __restrict__ dqt, __nv_bfloat16* __restrict__ dq, int Sq, int Hq, int D) {
  __shared__ float tile[32][33];
  const long long bh = blockIdx.z;
  const long long b = bh / Hq, h = bh % Hq;
  const int q0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  const float* src = dqt + (bh * D + d0) * static_cast<long long>(Sq) + q0;
#pragma unroll
  for (int r = ty; r < 32; r += 8) tile[r][tx] = src[static_cast<long long>(r) * Sq + tx];   // [d][q]
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8)
    dq[((b * Sq + q0 + r) * Hq + h) * D + d0 + tx] = __float2bfloat16_rn(tile[tx][r]);
}

template <int D, int MODE>
static int launch_bwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                      const AttBwdArgs& a, long long B, cudaStream_t st) {
  using C = AttBwdCfg<D, MODE>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attention_bwd_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::BYTES) !=
        cudaSuccess)
      return -11;
    attr = true;
  }
  dim3 grid(static_cast<unsigned>((a.Skv / AB_BKV) * a.Hkv * B));
  attention_bwd_kernel<D, MODE><<<grid, AB_THREADS, C::BYTES, st>>>(mq, mk, mv, mdo, a);
  return static_cast<int>(cudaGetLastError());
}

// q, o, d_o: bf16 [B, Sq, Hq, D]; k, v: bf16 [B, Skv, Hkv, D]; lse: fp32 [B, Hq, Sq] from the forward.
// Scratch: delta fp32 [B, Hq, Sq]; dqt fp32 [B, Hq, D, Sq], zeroed by the caller.
// Outputs: dq bf16 [B, Sq, Hq, D]; dk, dv bf16 [B, Skv, Hkv, D] (summed over the query heads of each GQA group).
// Sq % 64 == 0, Skv % 128 == 0.
extern "C" int cvb_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                 const float* lse, float* delta, float* dqt, void* dq, void* dk, void* dv, long long B,
                                 int Sq, int Skv, int Hq, int Hkv, int D, float scale, int causal, long long q_pos0,
                                 long long k_pos0, int* status, void* stream) {
  if (B <= 0 || Sq <= 0 || Skv <= 0) return 0;
  if (Sq % AB_BQ || Skv % AB_BKV || Hkv <= 0 || Hq % Hkv || !(scale > 0.f) || (D != 128 && D != 256)) return -1;
  if (B * Sq > 0x7fffffffLL || B * Skv > 0x7fffffffLL) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mq, mk, mv, mdo;
  const uint64_t qc = static_cast<uint64_t>(Hq) * D, kc = static_cast<uint64_t>(Hkv) * D;
  if (make_tensor_map_2d(&mq, q, 2, qc, B * Sq, qc * 2, 64, 64) || make_tensor_map_2d(&mdo, d_o, 2, qc, B * Sq, qc * 2, 64, 64) ||
      make_tensor_map_2d(&mk, k, 2, kc, B * Skv, kc * 2, 64, 128) || make_tensor_map_2d(&mv, v, 2, kc, B * Skv, kc * 2, 64, 128))
    return -10;
  const long long rows = B * Sq * Hq;
  attention_delta_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, B, Sq, Hq, D);
  AttBwdArgs a{};
  a.lse = lse; a.delta = delta; a.dk = static_cast<__nv_bfloat16*>(dk); a.dv = static_cast<__nv_bfloat16*>(dv);
  a.dqt = dqt; a.Sq = Sq; a.Skv = Skv; a.Hq = Hq; a.Hkv = Hkv; a.B = static_cast<int>(B); a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f; a.causal = causal; a.q_pos0 = q_pos0; a.k_pos0 = k_pos0; a.status = status;
  int rc;
  if (D == 128) {
    rc = launch_bwd<128, 0>(mq, mk, mv, mdo, a, B, st);
  } else {
    rc = launch_bwd<256, 1>(mq, mk, mv, mdo, a, B, st);
    if (rc == 0) rc = launch_bwd<256, 2>(mq, mk, mv, mdo, a, B, st);
  }
  if (rc != 0) return rc;
  dim3 tg(Sq / 32, D / 32, static_cast<unsigned>(B * Hq));
  attention_dq_transpose_kernel<<<tg, 256, 0, st>>>(dqt, static_cast<__nv_bfloat16*>(dq), Sq, Hq, D);
  return static_cast<int>(cudaGetLastError());
}
