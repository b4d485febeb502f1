// Gated-DeltaNet chunk-local backward on tcgen05 (C = 64 tokens, dk = dv = 128).
//
// One CTA per (batch, head, chunk) turns the upstream gradient dO, the scan's dVn / dS_next and the
// saved chunk-start state into dq, dk, dv, dbeta and dg.  With K^ = rk k, Q~ = rq q (rq carries the
// query scale), c the cumulative log-decay and T = (I + A)^-1:
//
//   dW   = -dVn S^T          dQd  = dO S^T            dKdec = Vn dS_next^T      dP = tril(dO Vn^T)
//   dVb  = T^T dVn           dKb  = T^T dW            dv = beta dVb
//   M1   = (dKb Ks^T + dVb V^T) diag(beta)            (Ks_j = e^{c_j} K^_j)
//   dA   = -stril(M1 T^T)    dG = dA beta_t e^{c_t-c_u}
//   dQ~  = e^{c} dQd + dPd K^                         (dPd = dP e^{c_t-c_u})
//   dK^  = dPd^T Q~ + (dG + dG^T) K^ + e^{c_C-c} dKdec + beta e^{c} dKb
//   dbeta= <dVb, v> + e^{c}<dKb, K^> + sum_u dA e^{c_t-c_u} G
//   dc_t = <dQ~, Q~> + 2 (sum_u dG G + beta e^{c} <dKb, K^>) - <dK^, K^>      (+ dgam on the last token)
//   dg   = suffix sum of dc inside the chunk; then the l2-norm backward gives dq, dk.
//
// The dc line uses that c enters only as e^{+c} on queries / "row" keys and e^{-c} on "column"
// keys, so its gradient is a difference of row dot products; dgam = <dS_next, S_next> comes from
// gdn_state_dot.  Every product runs as M = 128 tcgen05 MMAs: two 64-row operands are stacked
// ([Q;K], [dVn;dO], [Gs';dPd']) or the unused half reads don't-care rows (a zero tile where the
// accumulator is shared).  TMEM lanes 0-63 carry the key-side results, lanes 64-127 the query-side
// and 64 x 64 ones.  The CTA has two warpgroups: warps w and w + 4 may both read TMEM lane quadrant w, so
// every TMEM -> registers -> shared-memory hand-off between two MMA rounds is split by columns (each
// warpgroup takes every second 32-column chunk), and a token row's scalar results are the sum of two
// partial sums exchanged through shared memory.
// Intermediate operands go back to shared memory as bf16 rows in the 128-byte swizzle.
//
// The reference back-propagates token by token (cuda/qwen_linear_attention_cuda.cu:212-330).
#include "ptx.cuh"
#include "gemm_tcgen05.h"

namespace cvb {

constexpr int BC = 64;
constexpr int BD = 128;
constexpr int BTHREADS = 256;  // two warpgroups: warps w and w + 4 share TMEM lane quadrant w and split the columns

__device__ __forceinline__ uint32_t bsw128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

struct BwdArgs {
  const float* beta;   // [B, T, H]
  const float* Tm;     // [items, 64, 64]
  const float* aux;    // [items, 3, 64]: c, rq (with scale), rk
  const float* dgam;   // [items]
  __nv_bfloat16 *dq, *dk, *dv;  // [B, T, H, 128] with token stride d_stride (elements)
  long long d_stride;
  float* dbeta;        // [B, T, H]
  float* dg;           // [B, T, H]
  int T, H, n_chunks;
  long long items;     // B * H * n_chunks
  float scale;
  int* status;
};

// Shared-memory map (bytes).  Regions are reused once their first tenant is dead.
struct BwdSmem {
  static constexpr int PT = 0;            // dPd^T' [u][t]                      (8 KB)
  static constexpr int Z0 = 8192;         // zeros                               (8 KB)
  static constexpr int QK = 16384;        // Q0 | K0 | Q1 | K1                   (32 KB)
  static constexpr int V = 49152;         // V0 | V1                             (16 KB)
  static constexpr int VN = 65536;        // Vn0 | Vn1                           (16 KB)
  static constexpr int DS = 81920;        // dS_next^T: 2 x [128 x 64]           (32 KB)
  static constexpr int T = 114688;        // T bf16 [64][64]                     (8 KB)
  static constexpr int M1 = 122880;       // M1 bf16 [64][64]                    (8 KB)
  static constexpr int KS = 131072;       // Ks0 | Ks1                           (16 KB)
  static constexpr int DD = 147456;       // dVn0 | dO0 | dVn1 | dO1, later junk | dKb0 | dKb1 | dVb0   (32 KB)
  static constexpr int SS = 180224;       // S^T: 2 x [128 x 64], later dW (16 KB; then dVb1) | Gs' | dPd'  (32 KB)
  static constexpr int DW = SS;
  static constexpr int GP = SS + 16384;
  static constexpr int SC = 212992;       // scalars                             (6 KB)
  static constexpr int BARS = SC + 6144;
  static constexpr int BYTES = BARS + 256 + 1024;
};

// TMEM columns
constexpr uint32_t TC_D1 = 0;     // [Q;K] K^T
constexpr uint32_t TC_SL = 64;    // dP, then M1, then dA
constexpr uint32_t TC_ACC = 128;  // -dW | dQd, then dK^ (lanes 0-63) and dQ~ (lanes 64-127)
constexpr uint32_t TC_DX = 256;   // dVb, then dKdec
constexpr uint32_t TC_DK = 384;   // dKb

#define BWD_WAIT(bar, code)                                    \
  {                                                            \
    const bool ok_ = mbar_wait_bounded(bar, ph, abort_flag);   \
    if (!ok_) {                                                \
      if (!*abort_flag) atomicCAS(a.status, 0, code);          \
      *abort_flag = 1;                                         \
    }                                                          \
    __syncthreads();                                           \
    if (*abort_flag) goto done;                                \
    tc_fence_after();                                          \
  }
#define BWD_PUBLISH()          \
  {                            \
    fence_proxy_async_smem();  \
    tc_fence_before();         \
    __syncthreads();           \
    tc_fence_after();          \
  }

// 8 fp32 -> one 16-byte vector of bf16
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 x = __bfloat1622float2(p[j]);
    f[2 * j] = x.x;
    f[2 * j + 1] = x.y;
  }
}
// 32 consecutive elements [c0, c0+32) of row t of a [64 x 128] bf16 operand held as two swizzled [64 x 64] tiles
// `tile_stride` bytes apart
__device__ __forceinline__ void load_row32(const uint8_t* tiles, int tile_stride, int t, int c0, float* f) {
  const uint8_t* base = tiles + (c0 >> 6) * tile_stride;
  const int ch0 = (c0 & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) unpack8(*reinterpret_cast<const uint4*>(base + bsw128(t, ch0 + j)), f + 8 * j);
}
__device__ __forceinline__ void store_row32(uint8_t* tiles, int tile_stride, int t, int c0, const float* f) {
  uint8_t* base = tiles + (c0 >> 6) * tile_stride;
  const int ch0 = (c0 & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(base + bsw128(t, ch0 + j)) = pack8(f + 8 * j);
}
__device__ __forceinline__ void store_global32(__nv_bfloat16* dst, const float* f) {
#pragma unroll
  for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(dst + 8 * j) = pack8(f + 8 * j);
}

__global__ void __launch_bounds__(BTHREADS, 1)
gdn_chunk_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmDVn, const __grid_constant__ CUtensorMap tmVn,
                     const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmDS,
                     const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BwdSmem::BARS);
  uint64_t *bar_load = bars, *bar_p1 = bars + 1, *bar_d7a = bars + 2, *bar_m1 = bars + 3, *bar_da = bars + 4,
           *bar_acc = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_c = reinterpret_cast<float*>(smem + BwdSmem::SC);  // [64] each
  float* s_beta = s_c + 64;
  float* s_rk = s_c + 128;
  float* s_rq = s_c + 192;
  float* s_ec = s_c + 256;
  float* s_rowdgg = s_c + 320;  // [2][64]: per-warpgroup partial row sums from here on
  float* s_dba = s_c + 448;
  float* s_dc = s_c + 576;      // [2][64]: query side, key side
  float* s_dbv = s_c + 704;
  float* s_dotkb = s_c + 832;
  float* s_bk = s_c + 960;
  float* s_aq = s_c + 1088;

  const int tid = threadIdx.x;
  const int wg = tid >> 7;     // warpgroup: takes every second 32-column chunk of each stage
  const int lt = tid & 127;
  const int warp = lt >> 5;    // TMEM lane quadrant
  const bool lo = lt < BC;
  const int t = lt & 63;
  const uint32_t sb = smem_u32(smem);
  uint32_t tmem_base = 0, tmem = 0;
  uint32_t ph = 0;  // every barrier completes once per item: wait parity = item counter & 1

  // TMA loads of one item, in two parts on the same barrier: `rest` (everything but the Q | K tiles) can be
  // issued as soon as the previous item's last MMA round has retired, `qk` only after its final row pass.
  auto issue_loads = [&](long long it_, bool rest, bool qk) {
    const int ci = static_cast<int>(it_ % a.n_chunks);
    const long long cbh = it_ / a.n_chunks;
    const int col = static_cast<int>(cbh % a.H) * BD;
    const int r0 = static_cast<int>((cbh / a.H) * a.T + static_cast<long long>(ci) * BC);
    const int crow = static_cast<int>(it_ * BC), srow = static_cast<int>(it_ * BD);
    if (rest) {
      mbar_arrive_expect_tx(bar_load, 163840);  // the whole item, Q | K included
      tma_load_2d(smem + BwdSmem::V, &tmV, bar_load, col, r0);
      tma_load_2d(smem + BwdSmem::V + 8192, &tmV, bar_load, col + 64, r0);
      tma_load_2d(smem + BwdSmem::DD, &tmDVn, bar_load, 0, crow);
      tma_load_2d(smem + BwdSmem::DD + 8192, &tmDO, bar_load, col, r0);
      tma_load_2d(smem + BwdSmem::DD + 16384, &tmDVn, bar_load, 64, crow);
      tma_load_2d(smem + BwdSmem::DD + 24576, &tmDO, bar_load, col + 64, r0);
      tma_load_2d(smem + BwdSmem::VN, &tmVn, bar_load, 0, crow);
      tma_load_2d(smem + BwdSmem::VN + 8192, &tmVn, bar_load, 64, crow);
      tma_load_2d(smem + BwdSmem::SS, &tmS, bar_load, 0, srow);
      tma_load_2d(smem + BwdSmem::SS + 16384, &tmS, bar_load, 64, srow);
      tma_load_2d(smem + BwdSmem::DS, &tmDS, bar_load, 0, srow);
      tma_load_2d(smem + BwdSmem::DS + 16384, &tmDS, bar_load, 64, srow);
    }
    if (qk) {
      tma_load_2d(smem + BwdSmem::QK, &tmQ, bar_load, col, r0);
      tma_load_2d(smem + BwdSmem::QK + 8192, &tmK, bar_load, col, r0);
      tma_load_2d(smem + BwdSmem::QK + 16384, &tmQ, bar_load, col + 64, r0);
      tma_load_2d(smem + BwdSmem::QK + 24576, &tmK, bar_load, col + 64, r0);
    }
  };

  if (tid == 0) {
    for (int k = 0; k < 6; ++k) mbar_init(bars + k, 1);
    *abort_flag = 0;
    mbar_fence_init();
    if (static_cast<long long>(blockIdx.x) < a.items) issue_loads(blockIdx.x, true, true);
  }
  if (tid < 32) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  {
    uint4* z = reinterpret_cast<uint4*>(smem + BwdSmem::Z0) + tid * 2;   // the zero tile, written once
#pragma unroll
    for (int j = 0; j < 2; ++j) z[j] = make_uint4(0u, 0u, 0u, 0u);
  }
  BWD_PUBLISH();
  tmem_base = *tmem_slot;
  tmem = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  // Persistent CTA: items blockIdx.x, blockIdx.x + gridDim.x, ...  Barriers, TMEM and the zero tile are set up
  // once, and most of the next item's 160 KB is in flight while the current item's last stage runs.
#pragma unroll 1
  for (long long item = blockIdx.x; item < a.items; item += gridDim.x, ph ^= 1u) {
  const int i = static_cast<int>(item % a.n_chunks);
  const long long bh = item / a.n_chunks;
  const int h = static_cast<int>(bh % a.H);
  const long long b = bh / a.H;
  const long long row0 = b * a.T + static_cast<long long>(i) * BC;
  if (tid < BC) {
    const float* ax = a.aux + item * 3 * BC;
    const float c = ax[t];
    s_c[t] = c;
    s_rq[t] = ax[BC + t];
    s_rk[t] = ax[2 * BC + t];
    s_ec[t] = __expf(c);
    s_beta[t] = a.beta[(row0 + t) * a.H + h];
  }
  {
    // T (fp32, row-major) -> bf16 tile in the 128-byte swizzle
    const int r = tid >> 2, quarter = tid & 3;
    const float4* src = reinterpret_cast<const float4*>(a.Tm + (item * BC + r) * BC + quarter * 16);
    float f[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 x = src[j];
      f[4 * j] = x.x, f[4 * j + 1] = x.y, f[4 * j + 2] = x.z, f[4 * j + 3] = x.w;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
      *reinterpret_cast<uint4*>(smem + BwdSmem::T + bsw128(r, quarter * 2 + j)) = pack8(f + 8 * j);
  }
  BWD_PUBLISH();
  BWD_WAIT(bar_load, ERR_WAIT_FULL);

  // ---- stage 1: D1 = [Q;K] K^T, dP = dO Vn^T, [-dW ; dQd] = [dVn;dO] S^T, dVb = T^T dVn -------------------
  if (tid == 0) {
    constexpr uint32_t ID_KK64 = umma_idesc(128, 64, 1, 0, 0);
    constexpr uint32_t ID_KM128 = umma_idesc(128, 128, 1, 0, 1);
    constexpr uint32_t ID_MM128 = umma_idesc(128, 128, 1, 1, 1);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t kb = k >> 2, ks = (k & 3) * 32;
      umma_bf16(tmem_base + TC_D1, umma_smem_desc(sb + BwdSmem::QK + kb * 16384 + ks, 16, 1024),
                umma_smem_desc(sb + BwdSmem::QK + 8192 + kb * 16384 + ks, 16, 1024), ID_KK64, k > 0);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t kb = k >> 2, ks = (k & 3) * 32;
      umma_bf16(tmem_base + TC_SL, umma_smem_desc(sb + BwdSmem::DD + 8192 + kb * 16384 + ks, 16, 1024),
                umma_smem_desc(sb + BwdSmem::VN + kb * 8192 + ks, 16, 1024), ID_KK64, k > 0);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t kb = k >> 2, ks = (k & 3) * 32;
      umma_bf16(tmem_base + TC_ACC, umma_smem_desc(sb + BwdSmem::DD + kb * 16384 + ks, 16, 1024),
                umma_smem_desc(sb + BwdSmem::SS + k * 2048, 16384, 1024), ID_KM128, k > 0);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_bf16(tmem_base + TC_DX, umma_smem_desc(sb + BwdSmem::T + k * 2048, 8192, 1024),
                umma_smem_desc(sb + BwdSmem::DD + k * 2048, 16384, 1024), ID_MM128, k > 0);
    umma_commit(bar_p1);
  }
  if (!lo) {  // Ks_j = e^{c_j} rk_j k_j while the tensor cores run
    const float fk = s_ec[t] * s_rk[t];
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      float f[32];
      load_row32(smem + BwdSmem::QK + 8192, 16384, t, c0, f);
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] *= fk;
      store_row32(smem + BwdSmem::KS, 8192, t, c0, f);
    }
  }
  BWD_WAIT(bar_p1, ERR_WAIT_TMEM_FULL);

  // ---- stage 2: lanes 0-63 dump dW (bf16 rows) and clear their half of ACC; lanes 64-127 scale dQd by e^{c} ----
  {
    const float e = s_ec[t];
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_ACC + c0, r);
      tmem_ld_wait();
      if (lo) {
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = -__uint_as_float(r[j]);
        store_row32(smem + BwdSmem::DW, 8192, t, c0, f);
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * e);
      }
      tmem_st_32x32(tmem + TC_ACC + c0, r);
    }
    tmem_st_wait();
  }
  BWD_PUBLISH();

  // ---- stage 3: dKb = T^T dW; meanwhile lanes 0-63 turn dP into the dPd' and dPd^T' operand tiles ----------
  if (tid == 0) {
    constexpr uint32_t ID_MM128 = umma_idesc(128, 128, 1, 1, 1);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_bf16(tmem_base + TC_DK, umma_smem_desc(sb + BwdSmem::T + k * 2048, 8192, 1024),
                umma_smem_desc(sb + BwdSmem::DW + k * 2048, 8192, 1024), ID_MM128, k > 0);
    umma_commit(bar_d7a);
  }
  if (warp < 2) {
    const float ct = s_c[t], rqt = s_rq[t];
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BC; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_SL + c0, r);
      tmem_ld_wait();
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int u = c0 + j;
        const float pd = (u <= t) ? __uint_as_float(r[j]) * __expf(ct - s_c[u]) : 0.f;
        f[j] = pd * s_rk[u];
        *reinterpret_cast<__nv_bfloat16*>(smem + BwdSmem::PT + bsw128(u, t >> 3) + (t & 7) * 2) =
            __float2bfloat16_rn(pd * rqt);
      }
      store_row32(smem + BwdSmem::GP + 8192, 8192, t, c0, f);
    }
    fence_proxy_async_smem();
  }
  BWD_WAIT(bar_d7a, ERR_WAIT_TMEM_FULL);

  // ---- stage 4 (lanes 0-63): dv, <dVb, v>, <dKb, k>; dVb and dKb rows go back as bf16 operands -------------
  if (warp < 2) {
    const float bt = s_beta[t];
    __nv_bfloat16* dvrow = a.dv + (row0 + t) * a.d_stride + h * BD;
    float dbv = 0.f, dot_kb = 0.f;
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_DX + c0, r);
      tmem_ld_wait();
      float f[32], x[32];
      load_row32(smem + BwdSmem::V, 8192, t, c0, x);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        f[j] = __uint_as_float(r[j]);
        dbv += f[j] * x[j];
      }
      // dVb k-blocks sit at DD + 24 KB and DD + 32 KB
      store_row32(smem + BwdSmem::DD + 24576, 8192, t, c0, f);
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] *= bt;
      store_global32(dvrow + c0, f);
    }
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_DK + c0, r);
      tmem_ld_wait();
      float f[32], x[32];
      load_row32(smem + BwdSmem::QK + 8192, 16384, t, c0, x);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        f[j] = __uint_as_float(r[j]);
        dot_kb += f[j] * x[j];
      }
      store_row32(smem + BwdSmem::DD + 8192, 8192, t, c0, f);  // dKb k-blocks at DD + 8 KB and DD + 16 KB
    }
    s_dbv[wg * BC + t] = dbv;      // this warpgroup's half of <dVb, v> and <dKb, k>
    s_dotkb[wg * BC + t] = dot_kb;
  }
  BWD_PUBLISH();

  // ---- stage 5: M1 = dKb Ks^T + dVb V^T into lanes 64-127 (A tiles addressed 8 KB low) ---------------------
  if (tid == 0) {
    constexpr uint32_t ID_KK64 = umma_idesc(128, 64, 1, 0, 0);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t blk = k >> 2, ks = (k & 3) * 32;
      const uint32_t bt = (blk < 2 ? BwdSmem::KS + blk * 8192 : BwdSmem::V + (blk - 2) * 8192) + ks;
      umma_bf16(tmem_base + TC_SL, umma_smem_desc(sb + BwdSmem::DD + blk * 8192 + ks, 16, 1024),
                umma_smem_desc(sb + bt, 16, 1024), ID_KK64, k > 0);
    }
    umma_commit(bar_m1);
  }
  BWD_WAIT(bar_m1, ERR_WAIT_TMEM_FULL);

  // ---- stage 6 (lanes 64-127): M1 diag(beta) -> bf16 rows -------------------------------------------------
  if (warp >= 2) {
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BC; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_SL + c0, r);
      tmem_ld_wait();
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]) * s_beta[c0 + j];
      store_row32(smem + BwdSmem::M1, 8192, t, c0, f);
    }
  }
  BWD_PUBLISH();

  // ---- stage 7: dA_raw = M1 T^T (lanes 64-127), dKdec = Vn dS_next^T (lanes 0-63) ---------------------------
  if (tid == 0) {
    constexpr uint32_t ID_KK64 = umma_idesc(128, 64, 1, 0, 0);
    constexpr uint32_t ID_KM128 = umma_idesc(128, 128, 1, 0, 1);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_bf16(tmem_base + TC_SL, umma_smem_desc(sb + BwdSmem::T + k * 32, 16, 1024),
                umma_smem_desc(sb + BwdSmem::T + k * 32, 16, 1024), ID_KK64, k > 0);
    umma_commit(bar_da);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t kb = k >> 2, ks = (k & 3) * 32;
      umma_bf16(tmem_base + TC_DX, umma_smem_desc(sb + BwdSmem::VN + kb * 8192 + ks, 16, 1024),
                umma_smem_desc(sb + BwdSmem::DS + k * 2048, 16384, 1024), ID_KM128, k > 0);
    }
  }
  BWD_WAIT(bar_da, ERR_WAIT_TMEM_FULL);

  // ---- stage 8 (lanes 64-127): dA, dG, their row sums, and the symmetric Gs' operand ------------------------
  if (warp >= 2) {
    const float ct = s_c[t], bt = s_beta[t], rkt = s_rk[t];
    float rowdgg = 0.f, dba = 0.f;
    uint8_t* gs = smem + BwdSmem::GP;
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BC; c0 += 64) {
      uint32_t ra[32], rg[32];
      tmem_ld_32x32(tmem + TC_SL + c0, ra);
      tmem_ld_32x32(tmem + TC_D1 + c0, rg);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int u = c0 + j;
        if (u < t) {
          const float da = -__uint_as_float(ra[j]);
          const float dec = __expf(ct - s_c[u]);
          const float gn = rkt * s_rk[u] * __uint_as_float(rg[j]);
          const float dgv = da * bt * dec;
          rowdgg += dgv * gn;
          dba += da * dec * gn;
          *reinterpret_cast<__nv_bfloat16*>(gs + bsw128(t, u >> 3) + (u & 7) * 2) = __float2bfloat16_rn(dgv * s_rk[u]);
          *reinterpret_cast<__nv_bfloat16*>(gs + bsw128(u, t >> 3) + (t & 7) * 2) = __float2bfloat16_rn(dgv * rkt);
        } else if (u == t) {
          *reinterpret_cast<__nv_bfloat16*>(gs + bsw128(t, u >> 3) + (u & 7) * 2) = __float2bfloat16_rn(0.f);
        }
      }
    }
    s_rowdgg[wg * BC + t] = rowdgg;
    s_dba[wg * BC + t] = dba;
  }
  BWD_PUBLISH();

  // ---- stage 9: ACC += [Gs'; dPd'] K + [dPd^T'; 0] Q -------------------------------------------------------
  if (tid == 0) {
    constexpr uint32_t ID_KM128 = umma_idesc(128, 128, 1, 0, 1);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_bf16(tmem_base + TC_ACC, umma_smem_desc(sb + BwdSmem::GP + k * 32, 16, 1024),
                umma_smem_desc(sb + BwdSmem::QK + 8192 + k * 2048, 16384, 1024), ID_KM128, 1u);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_bf16(tmem_base + TC_ACC, umma_smem_desc(sb + BwdSmem::PT + k * 32, 16, 1024),
                umma_smem_desc(sb + BwdSmem::QK + k * 2048, 16384, 1024), ID_KM128, 1u);
    umma_commit(bar_acc);  // also covers dKdec
  }
  BWD_WAIT(bar_acc, ERR_WAIT_TMEM_FULL);
  // Every shared-memory region but Q | K is dead from here on (the final stage reads Q | K, TMEM and scalars):
  // start the next item's loads into them.
  if (tid == 0 && item + gridDim.x < a.items) {
    fence_proxy_async_smem();
    issue_loads(item + gridDim.x, true, false);
  }

  // ---- stage 10: finish one token row per thread pair (the two warpgroups split the columns) ---------------
  // pass 1: the row's dot product with its own (normalised) input, half per warpgroup
  if (warp < 2) {
    // key side: dK^ = ACC + e^{c_C - c_t} dKdec + beta_t e^{c_t} dKb
    const float edec = __expf(s_c[BC - 1] - s_c[t]);
    const float bek = s_beta[t] * s_ec[t];
    float bk = 0.f;
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32], r3[32], r7[32];
      tmem_ld_32x32(tmem + TC_ACC + c0, r);
      tmem_ld_32x32(tmem + TC_DX + c0, r3);
      tmem_ld_32x32(tmem + TC_DK + c0, r7);
      tmem_ld_wait();
      float x[32];
      load_row32(smem + BwdSmem::QK + 8192, 16384, t, c0, x);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float v = __uint_as_float(r[j]) + edec * __uint_as_float(r3[j]) + bek * __uint_as_float(r7[j]);
        bk += v * x[j];
        r[j] = __float_as_uint(v);
      }
      tmem_st_32x32(tmem + TC_ACC + c0, r);
    }
    tmem_st_wait();
    s_bk[wg * BC + t] = bk;
  } else {
    // query side: dQ~ is complete in ACC
    float aq = 0.f;
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_ACC + c0, r);
      tmem_ld_wait();
      float x[32];
      load_row32(smem + BwdSmem::QK, 16384, t, c0, x);
#pragma unroll
      for (int j = 0; j < 32; ++j) aq += __uint_as_float(r[j]) * x[j];
    }
    s_aq[wg * BC + t] = aq;
  }
  __syncthreads();
  // pass 2: the l2-norm backward with the full dot product
  if (warp < 2) {
    const float rkt = s_rk[t];
    const float bk = s_bk[t] + s_bk[BC + t];
    const float coef = rkt * rkt * bk;
    __nv_bfloat16* dkrow = a.dk + (row0 + t) * a.d_stride + h * BD;
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_ACC + c0, r);
      tmem_ld_wait();
      float x[32], f[32];
      load_row32(smem + BwdSmem::QK + 8192, 16384, t, c0, x);
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = rkt * (__uint_as_float(r[j]) - x[j] * coef);
      store_global32(dkrow + c0, f);
    }
    if (wg == 0) {
      const float bek = s_beta[t] * s_ec[t];
      const float dot_kb = s_dotkb[t] + s_dotkb[BC + t];
      s_dc[BC + t] = 2.f * (s_rowdgg[t] + s_rowdgg[BC + t] + bek * rkt * dot_kb) - rkt * bk;
      a.dbeta[(row0 + t) * a.H + h] =
          s_dbv[t] + s_dbv[BC + t] + s_ec[t] * rkt * dot_kb + s_dba[t] + s_dba[BC + t];
    }
  } else {
    const float rqt = s_rq[t];
    const float rq_ns = rqt / a.scale;
    const float aq = s_aq[t] + s_aq[BC + t];
    const float coef = rq_ns * rq_ns * aq;
    __nv_bfloat16* dqrow = a.dq + (row0 + t) * a.d_stride + h * BD;
#pragma unroll 1
    for (int c0 = wg * 32; c0 < BD; c0 += 64) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + TC_ACC + c0, r);
      tmem_ld_wait();
      float x[32], f[32];
      load_row32(smem + BwdSmem::QK, 16384, t, c0, x);
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = rqt * (__uint_as_float(r[j]) - x[j] * coef);
      store_global32(dqrow + c0, f);
    }
    if (wg == 0) s_dc[t] = rqt * aq;
  }
  tc_fence_before();
  __syncthreads();   // all reads of Q | K, of TMEM and of this item's scalars are done
  if (tid == 0 && item + gridDim.x < a.items) issue_loads(item + gridDim.x, false, true);
  if (tid < 32) {
    // dg = suffix sum of dc: lane l owns the reversed positions 2l and 2l+1
    const int l = tid;
    const int t0 = BC - 1 - 2 * l, t1 = t0 - 1;
    float v0 = s_dc[t0] + s_dc[BC + t0], v1 = s_dc[t1] + s_dc[BC + t1];
    if (l == 0) v0 += a.dgam[item];
    const float pair = v0 + v1;
    float incl = pair;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, incl, o);
      if (l >= o) incl += n;
    }
    const float excl = incl - pair;
    a.dg[(row0 + t0) * a.H + h] = excl + v0;
    a.dg[(row0 + t1) * a.H + h] = excl + pair;
  }
  }  // items
done:
  if (*abort_flag && tid == 0) {
    // a wait ran out: the next item's loads may still be in flight; give them a bounded time to land
    const long long t0 = clock64();
    while (clock64() - t0 < (1ll << 21)) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid < 32) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dgam[item] = <dS_next, S_next>: the state entering the next chunk (or the final state after the
// last one) against its gradient.  ST, dST: bf16 [BH, n, 128(dv), 128(dk)]; Sf: fp32 [BH, 128(dk), 128(dv)].
__global__ void __launch_bounds__(256)
gdn_state_dot_kernel(const __nv_bfloat16* __restrict__ ST, const __nv_bfloat16* __restrict__ dST,
                     const float* __restrict__ Sf, float* __restrict__ dgam, int n) {
  __shared__ float sh[8];
  const long long item = blockIdx.x;
  const int i = static_cast<int>(item % n);
  const long long bh = item / n;
  const __nv_bfloat16* ds = dST + item * BD * BD;
  float acc = 0.f;
  if (i + 1 < n) {
    const __nv_bfloat16* s = ST + (item + 1) * BD * BD;
    for (int e = threadIdx.x * 8; e < BD * BD; e += 256 * 8) {
      float x[8], y[8];
      unpack8(*reinterpret_cast<const uint4*>(s + e), x);
      unpack8(*reinterpret_cast<const uint4*>(ds + e), y);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += x[j] * y[j];
    }
  } else {
    const float* s = Sf + bh * BD * BD;  // [dk][dv]: transposed against dST
    for (int e = threadIdx.x; e < BD * BD; e += 256) {
      const int kk = e >> 7, vv = e & 127;
      acc += s[e] * __bfloat162float(ds[vv * BD + kk]);
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? sh[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) dgam[item] = r;
  }
}

}  // namespace cvb

using namespace cvb;

// q, k, v: bf16 views [B, T, H, 128] as for cvb_gdn_chunk_prep (common token stride `tok_stride`); dO: bf16
// [B, T, H, 128] contiguous; beta: fp32 [B, T, H]; Tm, aux: the prep kernel's outputs; Vn, dVn: bf16
// [BH, n, 64, 128]; ST, dST: bf16 [BH, n, 128, 128] (chunk-start state and dS_next, both transposed); Sf: fp32
// [BH, 128, 128] final state; dgam: fp32 [BH, n] scratch.  Outputs dq, dk, dv: bf16 [B, T, H, 128] whose rows lie
// `d_tok_stride` elements apart (0 = H * 128; a larger stride writes the three straight into their column ranges
// of one packed gradient buffer); dbeta, dg: fp32 [B, T, H].
extern "C" int cvb_gdn_chunk_bwd(const void* q, const void* k, const void* v, long long tok_stride, const void* dO,
                                 const float* beta, const float* Tm, const float* aux, const void* Vn, const void* dVn,
                                 const void* ST, const void* dST, const float* Sf, float* dgam, long long B, int T, int H,
                                 float scale, void* dq, void* dk, void* dv, long long d_tok_stride, float* dbeta,
                                 float* dg, int* status, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (d_tok_stride == 0) d_tok_stride = static_cast<long long>(H) * BD;
  if (T % BC != 0 || (tok_stride % 8) != 0 || (d_tok_stride % 8) != 0 || d_tok_stride < static_cast<long long>(H) * BD)
    return -1;
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15)
    return -1;  // the rows are written as 16-byte vectors
  const long long rows = B * T;
  const int n = T / BC;
  const long long items = B * H * n;
  if (rows > 0x7fffffffLL || items * BD > 0x7fffffffLL) return -2;
  CUtensorMap mq, mk, mv, mdo, mdvn, mvn, ms, mds;
  if (make_tensor_map_2d(&mq, q, 2, static_cast<uint64_t>(H) * BD, rows, tok_stride * 2, 64, 64) ||
      make_tensor_map_2d(&mk, k, 2, static_cast<uint64_t>(H) * BD, rows, tok_stride * 2, 64, 64) ||
      make_tensor_map_2d(&mv, v, 2, static_cast<uint64_t>(H) * BD, rows, tok_stride * 2, 64, 64) ||
      make_tensor_map_2d(&mdo, dO, 2, static_cast<uint64_t>(H) * BD, rows, static_cast<uint64_t>(H) * BD * 2, 64, 64) ||
      make_tensor_map_2d(&mdvn, dVn, 2, BD, items * BC, BD * 2, 64, 64) ||
      make_tensor_map_2d(&mvn, Vn, 2, BD, items * BC, BD * 2, 64, 64) ||
      make_tensor_map_2d(&ms, ST, 2, BD, items * BD, BD * 2, 64, 128) ||
      make_tensor_map_2d(&mds, dST, 2, BD, items * BD, BD * 2, 64, 128))
    return -10;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  gdn_state_dot_kernel<<<static_cast<unsigned>(items), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(ST), static_cast<const __nv_bfloat16*>(dST), Sf, dgam, n);
  BwdArgs a{};
  a.beta = beta; a.Tm = Tm; a.aux = aux; a.dgam = dgam;
  a.dq = static_cast<__nv_bfloat16*>(dq); a.dk = static_cast<__nv_bfloat16*>(dk); a.dv = static_cast<__nv_bfloat16*>(dv);
  a.d_stride = d_tok_stride;
  a.dbeta = dbeta; a.dg = dg; a.T = T; a.H = H; a.n_chunks = n; a.scale = scale; a.status = status;
  a.items = items;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_chunk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::BYTES) !=
        cudaSuccess)
      return -11;
    attr = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const unsigned grid = static_cast<unsigned>(items < sms ? items : sms);  // persistent: one CTA per SM
  gdn_chunk_bwd_kernel<<<grid, BTHREADS, BwdSmem::BYTES, st>>>(mq, mk, mv, mdo, mdvn, mvn, ms, mds, a);
  return static_cast<int>(cudaGetLastError());
}
