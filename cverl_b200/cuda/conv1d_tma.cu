// Backward of the depthwise causal conv1d + SiLU on channels-last activations, tiled through shared memory by TMA.
//
//   pre[s,c] = sum_t w[c,t] x[s-(K-1)+t, c]        y = silu(pre)
//   dpre     = dy * sig(pre) * (1 + pre (1 - sig(pre)))
//   dx[p,c]  = sum_t w[c,t] dpre[p+(K-1)-t, c]     dw[c,t] += sum_s dpre[s,c] x[s-(K-1)+t, c]
//
// One CTA of 256 threads owns a tile of 64 sequence positions x 256 channels: thread 0 issues eight TMA box
// loads (four 64-channel boxes of x with the K-1 rows of history and of look-ahead it needs, four of dy); two
// warps per box then walk 32 positions each out of shared memory, two channels per thread in packed fp32x2
// arithmetic, keeping the K-row windows of x and dpre in registers.  Nothing waits on global loads inside the
// walk, and three CTAs (24 warps) per SM overlap one tile's load with the others' arithmetic.  The 128-byte
// swizzle of the boxes keeps a warp's row read on 32 distinct banks.  dw is accumulated per thread and added with one atomic per (channel, tap).
//
// Reference behaviour: src/model/qwen3_5_text.cc:1241-1243 (conv1d + SiLU inside the linear-attention block);
// the reference differentiates it through its autograd graph op by op.
#include "ptx.cuh"
#include "gemm_tcgen05.h"
#include <type_traits>

namespace cvb {

constexpr int CVT_SEG = 64;        // sequence positions per tile
constexpr int CVT_ROWS = 72;       // rows per TMA box: SEG + 2 (K-1) <= 70, rounded so a box is 9 KB (1 KB multiple)
constexpr int CVT_BOX_CH = 64;     // channels per box = 128 bytes = one swizzle row
constexpr int CVT_BOXES = 4;
constexpr int CVT_SPLIT = 2;       // warps per box: each walks SEG / SPLIT positions (plus K-1 recomputed rows)
constexpr int CVT_SUB = CVT_SEG / CVT_SPLIT;
constexpr int CVT_THREADS = 32 * CVT_BOXES * CVT_SPLIT;
constexpr int CVT_BOX_BYTES = CVT_ROWS * 128;
constexpr int CVT_SMEM_X = 0;
constexpr int CVT_SMEM_DY = CVT_BOXES * CVT_BOX_BYTES;
constexpr int CVT_SMEM_BAR = 2 * CVT_BOXES * CVT_BOX_BYTES;
constexpr int CVT_SMEM_BYTES = CVT_SMEM_BAR + 64 + 1024;

__device__ __forceinline__ float2 cvt_ld2(const uint8_t* box, int row, int lane) {
  const uint32_t off = row * 128u + ((((lane >> 2) ^ (row & 7)) << 4) | ((lane & 3) << 2));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(box + off));
}
// sigmoid = 1/2 + 1/2 tanh(v/2): one special-function instruction per value instead of an exponential and a
// reciprocal (relative error of tanh.approx about 2^-11, below the bf16 rounding of the outputs)
__device__ __forceinline__ float cvt_tanh(float v) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

template <int KW>
__global__ void __launch_bounds__(CVT_THREADS, 3)
conv1d_silu_bwd_tma_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ dx,
                           float* __restrict__ dw, int S, int C, long long dx_stride, int segs, int ch_tiles,
                           int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + CVT_SMEM_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);
  const int tid = threadIdx.x, lane = tid & 31, box = (tid >> 5) % CVT_BOXES, part = tid / (32 * CVT_BOXES);
  const long long item = blockIdx.x;
  const int ct = static_cast<int>(item % ch_tiles);
  const long long bs = item / ch_tiles;
  const int seg = static_cast<int>(bs % segs);
  const long long b = bs / segs;
  const int s_begin = seg * CVT_SEG;
  const int s_end = min(S, s_begin + CVT_SEG);
  const long long row0 = b * S + s_begin;
  const int c0 = ct * (CVT_BOXES * CVT_BOX_CH);
  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    mbar_arrive_expect_tx(bar, 2 * CVT_BOXES * CVT_BOX_BYTES);
#pragma unroll
    for (int q = 0; q < CVT_BOXES; ++q) {
      // a box that starts past the last channel or row is filled with zeros and still counts its bytes
      tma_load_2d(smem + CVT_SMEM_X + q * CVT_BOX_BYTES, &tmX, bar, c0 + q * CVT_BOX_CH,
                  static_cast<int>(row0) - (KW - 1));
      tma_load_2d(smem + CVT_SMEM_DY + q * CVT_BOX_BYTES, &tmDY, bar, c0 + q * CVT_BOX_CH, static_cast<int>(row0));
    }
  }
  const int c = c0 + box * CVT_BOX_CH + 2 * lane;
  const bool live = c < C;
  float2 wv[KW], dwa[KW];
#pragma unroll
  for (int t = 0; t < KW; ++t) {
    wv[t] = live ? make_float2(__bfloat162float(w[c * KW + t]), __bfloat162float(w[(c + 1) * KW + t]))
                 : make_float2(0.f, 0.f);
    dwa[t] = make_float2(0.f, 0.f);
  }
  __syncthreads();
  if (!mbar_wait_bounded(bar, 0, abort_flag)) {
    if (!*abort_flag) atomicCAS(status, 0, ERR_WAIT_FULL);
    *abort_flag = 1;
    return;
  }
  const uint8_t* xb = smem + CVT_SMEM_X + box * CVT_BOX_BYTES;    // row r holds x[s_begin - (KW-1) + r]
  const uint8_t* db = smem + CVT_SMEM_DY + box * CVT_BOX_BYTES;   // row r holds dy[s_begin + r]
  // this warp's positions [sub_begin, sub_end) of the tile; dpre of the K-1 positions after them is recomputed
  const int off = part * CVT_SUB;
  const int sub_begin = s_begin + off;
  const int sub_end = min(s_end, sub_begin + CVT_SUB);
  if (sub_end <= sub_begin) return;
  // windows: x_win[k] = x[s - k], dpre_win[k] = dpre[s - k]; positions before the sequence start read as zero
  float2 x_win[KW], dpre_win[KW];
#pragma unroll
  for (int k = 0; k < KW; ++k) x_win[k] = make_float2(0.f, 0.f), dpre_win[k] = make_float2(0.f, 0.f);
#pragma unroll
  for (int k = 1; k < KW; ++k)
    if (sub_begin - k >= 0) x_win[k - 1] = cvt_ld2(xb, off + KW - 1 - k, lane);
  if (!live) return;
  const int n_main = sub_end - sub_begin;  // rows that are positions of this warp: they feed dw
  __nv_bfloat16* dxp = dx + (row0 + off) * dx_stride + c;
  const float2 one = make_float2(1.f, 1.f), neg = make_float2(-1.f, -1.f), half = make_float2(0.5f, 0.5f);
  // One row of the walk.  MAIN rows (KW-1 <= i < n_main) need no test at all: the position is inside the
  // sequence, feeds dw, and completes a dx.  The K-1 rows before and after them go through the guarded form.
  auto row = [&](int i, auto main_tag) {
    constexpr bool MAIN = decltype(main_tag)::value;
#pragma unroll
    for (int k = KW - 1; k > 0; --k) dpre_win[k] = dpre_win[k - 1], x_win[k] = x_win[k - 1];
    x_win[0] = cvt_ld2(xb, off + i + (KW - 1), lane);
    float2 d = cvt_ld2(db, off + i, lane);
    if (!MAIN && sub_begin + i >= S) {  // past the sequence end (the tile holds the next sequence there)
      d = make_float2(0.f, 0.f);
      x_win[0] = d;
    }
    float2 pre = make_float2(0.f, 0.f);
#pragma unroll
    for (int t = 0; t < KW; ++t) pre = __ffma2_rn(wv[t], x_win[KW - 1 - t], pre);
    const float2 hp = __fmul2_rn(pre, half);
    const float2 sg = __ffma2_rn(make_float2(cvt_tanh(hp.x), cvt_tanh(hp.y)), half, half);
    const float2 om = __ffma2_rn(sg, neg, one);                                  // 1 - sig
    dpre_win[0] = __fmul2_rn(__fmul2_rn(d, sg), __ffma2_rn(pre, om, one));      // dy sig (1 + pre (1 - sig))
    if (MAIN || i < n_main) {
#pragma unroll
      for (int t = 0; t < KW; ++t) dwa[t] = __ffma2_rn(dpre_win[0], x_win[KW - 1 - t], dwa[t]);
    }
    // dx at p = i - (KW-1): sum_t w[t] dpre[p + (KW-1) - t] = sum_t w[t] dpre_win[t]
    const int p = i - (KW - 1);
    if (MAIN || (p >= 0 && p < n_main)) {
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int t = 0; t < KW; ++t) acc = __ffma2_rn(wv[t], dpre_win[t], acc);
      *reinterpret_cast<uint32_t*>(dxp + p * dx_stride) = pack_bf16x2(acc.x, acc.y);
    }
  };
  const int head = min(KW - 1, n_main);
  for (int i = 0; i < head; ++i) row(i, std::false_type{});
#pragma unroll 4
  for (int i = head; i < n_main; ++i) row(i, std::true_type{});
  for (int i = n_main; i < n_main + (KW - 1); ++i) row(i, std::false_type{});
#pragma unroll
  for (int t = 0; t < KW; ++t) {
    atomicAdd(dw + c * KW + t, dwa[t].x);
    atomicAdd(dw + (c + 1) * KW + t, dwa[t].y);
  }
}

template <int KW>
static int launch_conv_bwd_tma(const CUtensorMap& tx, const CUtensorMap& tdy, const void* w, void* dx, float* dw,
                               long long B, int S, int C, long long dx_stride, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(conv1d_silu_bwd_tma_kernel<KW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             CVT_SMEM_BYTES) != cudaSuccess)
      return -3;
    configured = true;
  }
  const int segs = (S + CVT_SEG - 1) / CVT_SEG;
  const int ch_tiles = (C + CVT_BOXES * CVT_BOX_CH - 1) / (CVT_BOXES * CVT_BOX_CH);
  const long long items = B * segs * ch_tiles;
  conv1d_silu_bwd_tma_kernel<KW><<<static_cast<unsigned>(items), CVT_THREADS, CVT_SMEM_BYTES, stream>>>(
      tx, tdy, static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(dx), dw, S, C, dx_stride, segs,
      ch_tiles, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace cvb

// Returns -2 when the operands do not meet the TMA layout rules (the caller then uses the plain kernel):
// 16-byte aligned bases, row strides that are multiples of 16 bytes, C a multiple of 64, fewer than 2^31 rows.
extern "C" int cvb_conv1d_silu_bwd_tma(const void* dy, const void* x, const void* w, void* dx, float* dw, long long B,
                                       int S, int C, int KW, long long x_stride, long long dx_stride, int* status,
                                       void* stream) {
  using namespace cvb;
  if (B <= 0) return 0;
  if (KW < 2 || KW > 4 || C % CVT_BOX_CH || x_stride % 8 || dx_stride % 2 || B * S >= (1ll << 31) - 128 ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15) ||
      (reinterpret_cast<uintptr_t>(dx) & 3) || !status)
    return -2;
  const long long items = B * ((S + CVT_SEG - 1) / CVT_SEG) * ((C + 255) / 256);
  if (items >= (1ll << 31)) return -2;
  CUtensorMap tx, tdy;
  if (make_tensor_map_2d(&tx, x, 2, C, B * S, x_stride * 2, CVT_BOX_CH, CVT_ROWS)) return -2;
  if (make_tensor_map_2d(&tdy, dy, 2, C, B * S, static_cast<uint64_t>(C) * 2, CVT_BOX_CH, CVT_ROWS)) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (KW == 4) return launch_conv_bwd_tma<4>(tx, tdy, w, dx, dw, B, S, C, dx_stride, status, st);
  if (KW == 3) return launch_conv_bwd_tma<3>(tx, tdy, w, dx, dw, B, S, C, dx_stride, status, st);
  return launch_conv_bwd_tma<2>(tx, tdy, w, dx, dw, B, S, C, dx_stride, status, st);
}
