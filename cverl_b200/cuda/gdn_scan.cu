// Gated-DeltaNet chunk-to-chunk state scans on tcgen05, state resident in TMEM.
//
// The chunked (WY / UT-transform) form of the gated delta rule leaves two
// sequential passes over the chunks of a sequence (C = 64 tokens, dk = dv = 128):
//
//   forward   Vn_i = U_i - W_i S_i ;            S_{i+1} = e^{g_i} S_i + Kd_i^T Vn_i
//   backward  dVn_i = P_i^T dO_i + Kd_i dS ;    dS <- e^{g_i} dS + Qd_i^T dO_i - W_i^T dVn_i
//
// One CTA owns one (batch, head) sequence.  The fp32 state is kept TRANSPOSED
// in tensor memory, S^T [dv = 128 lanes x dk = 128 columns], so that every
// product has M = 128:  (W S)^T = S^T W^T,  S^T += Vn^T Kd.  Per chunk the CTA
//   1. reads S^T from TMEM, stores it (bf16) for the chunk-local kernels and for
//      the backward pass, refreshes the bf16 smem copy used as MMA operand A, and
//      writes e^{g} S^T back;
//   2. issues MMA 1 (operand B = the TMA-loaded W / Kd tile, K-major);
//   3. forms Vn^T (or dVn^T) in registers, stores it, and writes it to smem as
//      the K-major A operand of the state update;
//   4. issues the accumulating state-update MMA(s) (B = Kd / Qd / W tile read
//      MN-major from the very same TMA box layout).
// Tiles are fetched by TMA with 128-byte swizzle; the next chunk's tiles are
// requested as soon as their buffer is free.  All waits are bounded.
//
// The reference runs this recurrence token by token in scalar SIMT kernels
// (cuda/qwen_linear_attention_cuda.cu:139-210 forward, :465-586 backward).
#include "ptx.cuh"
#include "gemm_tcgen05.h"

namespace cvb {

constexpr int GC = 64;    // chunk length
constexpr int GD = 128;   // dk = dv
constexpr int GTHREADS = 128;

// byte offset of 16-byte chunk `chunk` of row `row` in a 128-byte-swizzled tile with 128-byte rows
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}
// element (t, v) of a [64 x 128] bf16 tile loaded as two {64 cols, 64 rows} swizzled boxes
__device__ __forceinline__ float tile_elem(const uint8_t* tile, int t, int v) {
  const uint32_t off = static_cast<uint32_t>(v >> 6) * 8192u + sw128(t, (v & 63) >> 3) + (v & 7) * 2u;
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(tile + off));
}

struct ScanSmem {
  // offsets inside the 1024-aligned dynamic shared memory
  static constexpr int S_OP = 0;                 // S^T bf16, K-major A, 2 k-blocks x 16 KB
  static constexpr int T0 = 32768;               // tile 0 (W fwd / Kd bwd), 16 KB
  static constexpr int T1 = T0 + 16384;          // tile 1 (Kd fwd / Qd bwd)
  static constexpr int T2 = T1 + 16384;          // tile 2 (U fwd / W bwd)
  static constexpr int A2 = T2 + 16384;          // Vn^T (fwd) or -dVn^T (bwd), K-major A, 16 KB
  static constexpr int BARS_FWD = A2 + 16384;
  // backward: the -dVn^T operand reuses the Kd tile (dead after MMA 1), which keeps two CTAs per SM
  static constexpr int B_KD = 32768;             // Kd, then -dVn^T
  static constexpr int B_QD = B_KD + 16384;
  static constexpr int B_W = B_QD + 16384;
  static constexpr int B_DO = B_W + 16384;       // dO tile, read MN-major as dO^T
  static constexpr int B_P = B_DO + 16384;       // P tile [64 x 64], 8 KB
  static constexpr int BARS_BWD = B_P + 8192;
  static constexpr int BYTES_FWD = BARS_FWD + 128 + 1024;
  static constexpr int BYTES_BWD = BARS_BWD + 128 + 1024;
};

struct ScanArgs {
  int n_chunks;
  const float* egam;          // [BH, n]
  const float* s_init;        // [BH, dk, dv] fp32 or nullptr (zero)
  float* s_final;             // [BH, dk, dv] fp32
  __nv_bfloat16* out_v;       // Vn / dVn  [BH, n, C, dv]
  __nv_bfloat16* out_s;       // per-chunk state (transposed) [BH, n, dv, dk]
  int* status;
  int do_heads;               // backward: 0 = dO is [BH, n, C, dv]; H > 0 = dO is [B, n*C, H, dv] (token-major)
};

// issue the two 64x64 boxes of a [64 x 128] tile
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row0) {
  mbar_arrive_expect_tx(bar, 16384);
  tma_load_2d(dst, m, bar, 0, row0);
  tma_load_2d(dst + 8192, m, bar, 64, row0);
}

// S^T (or dS^T) round trip: TMEM -> (global bf16, smem bf16 operand) -> scaled -> TMEM
__device__ __forceinline__ void state_round_trip(uint32_t t_state, uint8_t* s_op, __nv_bfloat16* g_row,
                                                 float scale, int v) {
#pragma unroll 1
  for (int c0 = 0; c0 < GD; c0 += 32) {
    uint32_t r[32];
    tmem_ld_32x32(t_state + c0, r);
    tmem_ld_wait();
    uint32_t packed[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 q = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      if (g_row) *reinterpret_cast<uint4*>(g_row + c0 + 8 * j) = q;
      const int k = c0 + 8 * j;  // first dk index of this 16-byte chunk
      *reinterpret_cast<uint4*>(s_op + (k >> 6) * 16384 + sw128(v, (k & 63) >> 3)) = q;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * scale);
    tmem_st_32x32(t_state + c0, r);
  }
  tmem_st_wait();
}

__device__ __forceinline__ void issue_mma_state_times_tile(uint32_t t_d, uint32_t s_op, uint32_t tile) {
  // D[128 x 64] = S^T(bf16, K-major, K = 128) * tile^T  (tile [64 rows x 128] K-major)
  constexpr uint32_t idesc = umma_idesc(128, GC, 1, 0, 0);
#pragma unroll
  for (int k = 0; k < GD / 16; ++k) {
    const uint32_t kb = k >> 2, ks = (k & 3) * 32;
    const uint64_t ad = umma_smem_desc(s_op + kb * 16384 + ks, 16, 1024);
    const uint64_t bd = umma_smem_desc(tile + kb * 8192 + ks, 16, 1024);
    umma_bf16(t_d, ad, bd, idesc, k > 0 ? 1u : 0u);
  }
}
__device__ __forceinline__ void issue_mma_update(uint32_t t_state, uint32_t a_op, uint32_t tile) {
  // S^T[128 x 128] += A[128 x 64] (K-major, K = 64) * tile ([64 k-rows x 128 n] read MN-major)
  constexpr uint32_t idesc = umma_idesc(128, GD, 1, 0, 1);
#pragma unroll
  for (int k = 0; k < GC / 16; ++k) {
    const uint64_t ad = umma_smem_desc(a_op + k * 32, 16, 1024);
    const uint64_t bd = umma_smem_desc(tile + k * 2048, 8192, 1024);
    umma_bf16(t_state, ad, bd, idesc, 1u);
  }
}

#define SCAN_FAIL(code)                           \
  do {                                            \
    if (!*abort_flag) atomicCAS(a.status, 0, code); \
    *abort_flag = 1;                              \
  } while (0)

// ---------------------------------------------------------------------------
// forward scan
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(GTHREADS, 2)
gdn_scan_fwd_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmU, const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ScanSmem::BARS_FWD);
  uint64_t *bar_w = bars, *bar_k = bars + 1, *bar_u = bars + 2, *bar_m1 = bars + 3, *bar_m2 = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int v = threadIdx.x;
  const int warp = v >> 5;
  const long long bh = blockIdx.x;
  const int n = a.n_chunks;

  if (v == 0) {
    mbar_init(bar_w, 1); mbar_init(bar_k, 1); mbar_init(bar_u, 1); mbar_init(bar_m1, 1); mbar_init(bar_m2, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmU);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t t_d1 = tmem;          // columns [0, 64)
  const uint32_t t_state = tmem + 128;  // columns [128, 256)
  uint8_t* s_op = smem + ScanSmem::S_OP;
  uint8_t* s_w = smem + ScanSmem::T0;
  uint8_t* s_k = smem + ScanSmem::T1;
  uint8_t* s_u = smem + ScanSmem::T2;
  uint8_t* s_a2 = smem + ScanSmem::A2;
  const long long row_base = bh * n * GC;  // first row of this sequence in the [rows, 128] tensors

  if (v == 0 && n > 0) {
    load_tile(s_w, &tmW, bar_w, static_cast<int>(row_base));
    load_tile(s_u, &tmU, bar_u, static_cast<int>(row_base));
    load_tile(s_k, &tmK, bar_k, static_cast<int>(row_base));
  }
  // initial state: S^T[v][k] = s_init[k][v]
#pragma unroll 1
  for (int c0 = 0; c0 < GD; c0 += 32) {
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j)
      r[j] = a.s_init ? __float_as_uint(a.s_init[(bh * GD + (c0 + j)) * GD + v]) : 0u;
    tmem_st_32x32(t_state + c0, r);
  }
  tmem_st_wait();

  uint32_t phase = 0;
  bool ok = true;
  for (int i = 0; i < n && ok; ++i) {
    const float eg = a.egam[bh * n + i];
    // 1. state round trip
    state_round_trip(t_state, s_op, a.out_s + ((bh * n + i) * GD + v) * GD, eg, v);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // 2. D1 = S^T W^T
    if (v == 0) {
      if (mbar_wait_bounded(bar_w, phase, abort_flag)) {
        tc_fence_after();
        issue_mma_state_times_tile(t_d1, smem_u32(s_op), smem_u32(s_w));
        umma_commit(bar_m1);
      } else {
        SCAN_FAIL(ERR_WAIT_FULL);
      }
    }
    if (!mbar_wait_bounded(bar_m1, phase, abort_flag)) SCAN_FAIL(ERR_WAIT_TMEM_FULL);
    if (!mbar_wait_bounded(bar_u, phase, abort_flag)) SCAN_FAIL(ERR_WAIT_FULL);
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    if (v == 0 && i + 1 < n) load_tile(s_w, &tmW, bar_w, static_cast<int>(row_base + (i + 1) * GC));
    // 3. Vn^T = U^T - D1
    __nv_bfloat16* g_v = a.out_v + (bh * n + i) * GC * GD + v;
#pragma unroll 1
    for (int c0 = 0; c0 < GC; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(t_d1 + c0, r);
      tmem_ld_wait();
      uint32_t packed[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float x0 = tile_elem(s_u, c0 + j, v) - __uint_as_float(r[j]);
        const float x1 = tile_elem(s_u, c0 + j + 1, v) - __uint_as_float(r[j + 1]);
        const __nv_bfloat16 b0 = __float2bfloat16_rn(x0), b1 = __float2bfloat16_rn(x1);
        g_v[(c0 + j) * GD] = b0;
        g_v[(c0 + j + 1) * GD] = b1;
        packed[j >> 1] = pack_bf16x2(x0, x1);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(s_a2 + sw128(v, (c0 >> 3) + j)) =
            make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // 4. S^T += Vn^T Kd
    if (v == 0) {
      if (i + 1 < n) load_tile(s_u, &tmU, bar_u, static_cast<int>(row_base + (i + 1) * GC));
      if (mbar_wait_bounded(bar_k, phase, abort_flag)) {
        tc_fence_after();
        issue_mma_update(t_state, smem_u32(s_a2), smem_u32(s_k));
        umma_commit(bar_m2);
      } else {
        SCAN_FAIL(ERR_WAIT_FULL);
      }
    }
    if (!mbar_wait_bounded(bar_m2, phase, abort_flag)) SCAN_FAIL(ERR_WAIT_TMEM_FULL);
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    if (v == 0 && i + 1 < n) load_tile(s_k, &tmK, bar_k, static_cast<int>(row_base + (i + 1) * GC));
    phase ^= 1;
  }
  if (!ok && v == 0) {  // leave no copy in flight
    int dummy = 0;
    mbar_wait_bounded(bar_w, phase, &dummy);
    mbar_wait_bounded(bar_u, phase, &dummy);
    mbar_wait_bounded(bar_k, phase, &dummy);
  }
  // final state: s_final[k][v] = S^T[v][k]
  if (ok) {
#pragma unroll 1
    for (int c0 = 0; c0 < GD; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(t_state + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) a.s_final[(bh * GD + (c0 + j)) * GD + v] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(*tmem_slot, 256);
  }
}

// ---------------------------------------------------------------------------
// backward scan (chunks in descending order)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(GTHREADS, 2)
gdn_scan_bwd_kernel(const __grid_constant__ CUtensorMap tmKd, const __grid_constant__ CUtensorMap tmQd,
                    const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmP, const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ScanSmem::BARS_BWD);
  uint64_t *bar_a = bars, *bar_b = bars + 1, *bar_m1 = bars + 2, *bar_m2 = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int v = threadIdx.x;
  const int warp = v >> 5;
  const long long bh = blockIdx.x;
  const int n = a.n_chunks;

  if (v == 0) {
    mbar_init(bar_a, 1); mbar_init(bar_b, 1); mbar_init(bar_m1, 1); mbar_init(bar_m2, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t t_d1 = tmem;
  const uint32_t t_state = tmem + 128;
  uint8_t* s_op = smem + ScanSmem::S_OP;
  uint8_t* s_kd = smem + ScanSmem::B_KD;   // also -dVn^T
  uint8_t* s_qd = smem + ScanSmem::B_QD;
  uint8_t* s_w = smem + ScanSmem::B_W;
  uint8_t* s_do = smem + ScanSmem::B_DO;
  uint8_t* s_p = smem + ScanSmem::B_P;
  const long long row_base = bh * n * GC;

  // all five tiles of one chunk: {Kd, dO, P} complete bar_a, {Qd, W} complete bar_b
  auto load_chunk = [&](int i) {
    const int r0 = static_cast<int>(row_base + static_cast<long long>(i) * GC);
    mbar_arrive_expect_tx(bar_a, 16384 + 16384 + 8192);
    tma_load_2d(s_kd, &tmKd, bar_a, 0, r0);
    tma_load_2d(s_kd + 8192, &tmKd, bar_a, 64, r0);
    if (a.do_heads > 0) {  // straight from the [tokens, H * dv] gradient of the layer output
      const long long b = bh / a.do_heads;
      const int x0 = static_cast<int>(bh % a.do_heads) * GD;
      const int tr = static_cast<int>((b * n + i) * GC);
      tma_load_2d(s_do, &tmDO, bar_a, x0, tr);
      tma_load_2d(s_do + 8192, &tmDO, bar_a, x0 + 64, tr);
    } else {
      tma_load_2d(s_do, &tmDO, bar_a, 0, r0);
      tma_load_2d(s_do + 8192, &tmDO, bar_a, 64, r0);
    }
    tma_load_2d(s_p, &tmP, bar_a, 0, r0);
    mbar_arrive_expect_tx(bar_b, 32768);
    tma_load_2d(s_qd, &tmQd, bar_b, 0, r0);
    tma_load_2d(s_qd + 8192, &tmQd, bar_b, 64, r0);
    tma_load_2d(s_w, &tmW, bar_b, 0, r0);
    tma_load_2d(s_w + 8192, &tmW, bar_b, 64, r0);
  };
  if (v == 0 && n > 0) load_chunk(n - 1);
  // dS^T[v][k] = s_init[k][v]  (gradient of the final state, or zero)
#pragma unroll 1
  for (int c0 = 0; c0 < GD; c0 += 32) {
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j)
      r[j] = a.s_init ? __float_as_uint(a.s_init[(bh * GD + (c0 + j)) * GD + v]) : 0u;
    tmem_st_32x32(t_state + c0, r);
  }
  tmem_st_wait();

  uint32_t phase = 0;
  bool ok = true;
  for (int i = n - 1; i >= 0 && ok; --i) {
    const float eg = a.egam[bh * n + i];
    // 1. dS round trip: stores dS_{i+1} (the gradient of the state AFTER chunk i)
    state_round_trip(t_state, s_op, a.out_s + ((bh * n + i) * GD + v) * GD, eg, v);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // 2. D1 = dS^T Kd^T + dO^T P   (= dVn^T; dO^T is the dO tile read MN-major, P^T dO never leaves the SM)
    if (v == 0) {
      if (mbar_wait_bounded(bar_a, phase, abort_flag)) {
        tc_fence_after();
        issue_mma_state_times_tile(t_d1, smem_u32(s_op), smem_u32(s_kd));
        constexpr uint32_t idesc = umma_idesc(128, GC, 1, 1, 1);
#pragma unroll
        for (int k = 0; k < GC / 16; ++k)
          umma_bf16(t_d1, umma_smem_desc(smem_u32(s_do) + k * 2048, 8192, 1024),
                    umma_smem_desc(smem_u32(s_p) + k * 2048, 8192, 1024), idesc, 1u);
        umma_commit(bar_m1);
      } else {
        SCAN_FAIL(ERR_WAIT_FULL);
      }
    }
    if (!mbar_wait_bounded(bar_m1, phase, abort_flag)) SCAN_FAIL(ERR_WAIT_TMEM_FULL);
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    // 3. store dVn; A2 = -dVn^T over the (now dead) Kd tile
    __nv_bfloat16* g_v = a.out_v + (bh * n + i) * GC * GD + v;
#pragma unroll 1
    for (int c0 = 0; c0 < GC; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(t_d1 + c0, r);
      tmem_ld_wait();
      uint32_t p2[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float x0 = __uint_as_float(r[j]), x1 = __uint_as_float(r[j + 1]);
        g_v[(c0 + j) * GD] = __float2bfloat16_rn(x0);
        g_v[(c0 + j + 1) * GD] = __float2bfloat16_rn(x1);
        p2[j >> 1] = pack_bf16x2(-x0, -x1);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(s_kd + sw128(v, (c0 >> 3) + j)) =
            make_uint4(p2[4 * j], p2[4 * j + 1], p2[4 * j + 2], p2[4 * j + 3]);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // 4. dS^T += dO^T Qd - dVn^T W
    if (v == 0) {
      if (mbar_wait_bounded(bar_b, phase, abort_flag)) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(128, GD, 1, 1, 1);
#pragma unroll
        for (int k = 0; k < GC / 16; ++k)
          umma_bf16(t_state, umma_smem_desc(smem_u32(s_do) + k * 2048, 8192, 1024),
                    umma_smem_desc(smem_u32(s_qd) + k * 2048, 8192, 1024), idesc, 1u);
        issue_mma_update(t_state, smem_u32(s_kd), smem_u32(s_w));
        umma_commit(bar_m2);
      } else {
        SCAN_FAIL(ERR_WAIT_FULL);
      }
    }
    if (!mbar_wait_bounded(bar_m2, phase, abort_flag)) SCAN_FAIL(ERR_WAIT_TMEM_FULL);
    __syncthreads();
    if (*abort_flag) { ok = false; break; }
    tc_fence_after();
    if (v == 0 && i > 0) load_chunk(i - 1);
    phase ^= 1;
  }
  if (!ok && v == 0) {  // leave no copy in flight
    int dummy = 0;
    mbar_wait_bounded(bar_a, phase, &dummy);
    mbar_wait_bounded(bar_b, phase, &dummy);
  }
  if (ok) {
#pragma unroll 1
    for (int c0 = 0; c0 < GD; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(t_state + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) a.s_final[(bh * GD + (c0 + j)) * GD + v] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(*tmem_slot, 256);
  }
}

static int make_rows128_map(CUtensorMap* m, const void* base, long long rows) {
  return make_tensor_map_2d(m, base, 2, GD, static_cast<uint64_t>(rows), GD * 2, 64, 64);
}

}  // namespace cvb

using namespace cvb;

// W, U, Kd: [BH, n, 64, 128] bf16.  egam [BH, n].  s_init / s_final [BH, 128, 128] fp32 (dk-major).
// out_v [BH, n, 64, 128] bf16 (Vn), out_s [BH, n, 128(dv), 128(dk)] bf16 (chunk-start states, transposed).
extern "C" int cvb_gdn_scan_fwd(const void* W, const void* U, const void* Kd, const float* egam, const float* s_init,
                                float* s_final, void* out_v, void* out_s, long long BH, int n_chunks, int* status,
                                void* stream) {
  if (BH <= 0 || n_chunks <= 0) return 0;
  if (BH * n_chunks * GC > 0x7fffffffLL) return -2;
  CUtensorMap mW, mU, mK;
  const long long rows = BH * n_chunks * GC;
  if (make_rows128_map(&mW, W, rows) || make_rows128_map(&mU, U, rows) || make_rows128_map(&mK, Kd, rows)) return -10;
  ScanArgs a{};
  a.n_chunks = n_chunks; a.egam = egam; a.s_init = s_init; a.s_final = s_final;
  a.out_v = static_cast<__nv_bfloat16*>(out_v); a.out_s = static_cast<__nv_bfloat16*>(out_s); a.status = status;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ScanSmem::BYTES_FWD) !=
        cudaSuccess)
      return -11;
    attr = true;
  }
  gdn_scan_fwd_kernel<<<static_cast<int>(BH), GTHREADS, ScanSmem::BYTES_FWD, static_cast<cudaStream_t>(stream)>>>(
      mW, mK, mU, a);
  return static_cast<int>(cudaGetLastError());
}

// P: [BH, n, 64, 64] bf16 (the chunk's decayed, masked Q K^T); dO, Kd, Qd, W: [BH, n, 64, 128] bf16.
// ds_final (may be null) / ds_init_out: [BH, 128, 128] fp32.
// out_dv: dVn = P^T dO + Kd dS.  out_ds: dS_{i+1} per chunk, transposed [BH, n, dv, dk] bf16.
extern "C" int cvb_gdn_scan_bwd(const void* P, const void* Kd, const void* Qd, const void* W, const void* dO,
                                const float* egam, const float* ds_final, float* ds_init_out, void* out_dv,
                                void* out_ds, long long BH, int n_chunks, int do_heads, int* status, void* stream) {
  if (BH <= 0 || n_chunks <= 0) return 0;
  if (BH * n_chunks * GC > 0x7fffffffLL) return -2;
  if (do_heads < 0 || (do_heads > 0 && BH % do_heads != 0)) return -1;
  CUtensorMap mK, mQ, mW, mO, mP;
  const long long rows = BH * n_chunks * GC;
  // dO: chunk-major [BH, n, 64, 128], or (do_heads = H > 0) the token-major [B, n*64, H, 128] gradient itself
  const int rc_do = do_heads > 0
                        ? make_tensor_map_2d(&mO, dO, 2, static_cast<uint64_t>(do_heads) * GD,
                                             static_cast<uint64_t>(rows / do_heads),
                                             static_cast<uint64_t>(do_heads) * GD * 2, 64, 64)
                        : make_rows128_map(&mO, dO, rows);
  if (make_rows128_map(&mK, Kd, rows) || make_rows128_map(&mQ, Qd, rows) || make_rows128_map(&mW, W, rows) || rc_do ||
      make_tensor_map_2d(&mP, P, 2, GC, static_cast<uint64_t>(rows), GC * 2, 64, 64))
    return -10;
  ScanArgs a{};
  a.n_chunks = n_chunks; a.egam = egam; a.s_init = ds_final; a.s_final = ds_init_out;
  a.out_v = static_cast<__nv_bfloat16*>(out_dv); a.out_s = static_cast<__nv_bfloat16*>(out_ds);
  a.status = status; a.do_heads = do_heads;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ScanSmem::BYTES_BWD) !=
        cudaSuccess)
      return -11;
    attr = true;
  }
  gdn_scan_bwd_kernel<<<static_cast<int>(BH), GTHREADS, ScanSmem::BYTES_BWD, static_cast<cudaStream_t>(stream)>>>(
      mK, mQ, mW, mO, mP, a);
  return static_cast<int>(cudaGetLastError());
}
