// Gated-DeltaNet chunk-local forward kernels on tcgen05 (C = 64 tokens, dk = dv = 128).
//
// gdn_chunk_prep: one CTA per (batch, head, chunk).  From the raw q, k, v tiles (TMA, straight
// out of the convolution output), beta and g it produces everything the state scan and the
// output kernel consume:
//     rq, rk      l2-norm factors            c        cumulative log-decay inside the chunk
//     A[t,u]    = beta_t e^{c_t-c_u} <k^_t,k^_u> (u<t)      T = (I + A)^-1   (blocked triangular inverse, fp32)
//     W  = T diag(beta e^c) K^     U = T diag(beta) V       (pseudo keys / values, WY form)
//     P[t,u]    = e^{c_t-c_u} <q~_t,k^_u> (u<=t)            Kd = e^{c_C-c} K^      Qd = e^{c} Q~
// All products run with M = 128 on the tensor cores: [K;Q] K^T stacks the two 64-row tiles, and
// W^T = K^T T'^T, U^T = V^T T''^T read the TMA tiles MN-major, with the normalisation and decay
// factors folded into the small T' / T'' operands instead of the big ones.
//
// gdn_chunk_out: O^T = S^T Qd^T + Vn^T P^T per (batch, head, chunk), S being the chunk-start
// state written by the scan kernel.
//
// The reference has no chunked form: it walks the tokens one by one
// (src/model/qwen3_5_text.cc:207-262, cuda/qwen_linear_attention_cuda.cu:139-210).
#include "ptx.cuh"
#include "gemm_tcgen05.h"

namespace cvb {

constexpr int CC = 64;
constexpr int CD = 128;
constexpr int CTHREADS = 128;

__device__ __forceinline__ uint32_t csw128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

struct PrepArgs {
  const float* beta;   // [B, T, H]
  const float* g;      // [B, T, H]
  int T, H, n_chunks;
  float scale, eps;
  __nv_bfloat16 *W, *U, *Kd, *Qd;  // [BH, n, 64, 128]
  __nv_bfloat16* P;                // [BH, n, 64, 64]
  float* egam;                     // [BH, n]
  float* Tm;                       // [BH, n, 64, 64] or nullptr
  float* aux;                      // [BH, n, 3, 64]: c, rq, rk  (or nullptr)
  int* status;
};

struct PrepSmem {
  static constexpr int KQ = 0;            // K box0 | Q box0 | K box1 | Q box1   (4 x 8 KB)
  static constexpr int V = 32768;         // V box0 | V box1
  static constexpr int AM = 49152;        // fp32 [64][64]; dead after the substitution, then reused as:
  static constexpr int TP = 49152;        // T'  bf16 [64 x 64]
  static constexpr int TPP = 57344;       // T'' bf16 [64 x 64]
  static constexpr int SC = 65536;        // scalars: c, beta, rk, rq, partial sums
  static constexpr int XS = SC + 2048;     // fp32 [3][16][16]: block products of the triangular inverse
  static constexpr int BARS = XS + 3072;
  static constexpr int BYTES = BARS + 128 + 1024;
};

// Three CTAs per SM (168 registers, 71 KB of shared memory, 128 TMEM columns each): every CTA is one serial
// chain load -> MMA -> triangular inverse -> MMA -> store, so the SM is kept busy by the other CTAs' phases.
__global__ void __launch_bounds__(CTHREADS, 3)
gdn_chunk_prep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const PrepArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PrepSmem::BARS);
  uint64_t *bar_load = bars, *bar_m1 = bars + 1, *bar_m2 = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_c = reinterpret_cast<float*>(smem + PrepSmem::SC);  // [64]
  float* s_beta = s_c + 64;
  float* s_rk = s_c + 128;
  float* s_rq = s_c + 192;
  float* s_pk = s_c + 256;  // [2][64] partial sums of squares
  float* s_pq = s_c + 384;
  float* Am = reinterpret_cast<float*>(smem + PrepSmem::AM);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const long long item = blockIdx.x;  // bh * n + i
  const int i = static_cast<int>(item % a.n_chunks);
  const long long bh = item / a.n_chunks;
  const int h = static_cast<int>(bh % a.H);
  const long long b = bh / a.H;
  const long long row0 = b * a.T + static_cast<long long>(i) * CC;  // first token row of this chunk

  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_m1, 1); mbar_init(bar_m2, 1);
    *abort_flag = 0;
    mbar_fence_init();
    mbar_arrive_expect_tx(bar_load, 49152);
    const int col = h * CD;
    tma_load_2d(smem + PrepSmem::KQ, &tmK, bar_load, col, static_cast<int>(row0));
    tma_load_2d(smem + PrepSmem::KQ + 16384, &tmK, bar_load, col + 64, static_cast<int>(row0));
    tma_load_2d(smem + PrepSmem::KQ + 8192, &tmQ, bar_load, col, static_cast<int>(row0));
    tma_load_2d(smem + PrepSmem::KQ + 24576, &tmQ, bar_load, col + 64, static_cast<int>(row0));
    tma_load_2d(smem + PrepSmem::V, &tmV, bar_load, col, static_cast<int>(row0));
    tma_load_2d(smem + PrepSmem::V + 8192, &tmV, bar_load, col + 64, static_cast<int>(row0));
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, 128);  // columns 0-63: D1, then W^T; 64-127: U^T
    tmem_relinquish();
  }
  if (tid < CC) {
    const long long e = (row0 + tid) * a.H + h;
    s_beta[tid] = a.beta[e];
    s_c[tid] = a.g[e];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  if (tid == 0) {  // inclusive scan of g
    float acc = 0.f;
    for (int t = 0; t < CC; ++t) {
      acc += s_c[t];
      s_c[t] = acc;
    }
  }
  bool ok = mbar_wait_bounded(bar_load, 0, abort_flag);
  if (!ok) {
    if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_FULL);
    *abort_flag = 1;
  }
  __syncthreads();
  if (*abort_flag) goto done;
  // 1. D1 = [K;Q] K^T  (M = 128, N = 64, K = 128)
  if (tid == 0) {
    constexpr uint32_t idesc = umma_idesc(128, CC, 1, 0, 0);
    const uint32_t kq = smem_u32(smem + PrepSmem::KQ);
#pragma unroll
    for (int k = 0; k < CD / 16; ++k) {
      const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
      umma_bf16(tmem_base, umma_smem_desc(kq + off, 16, 1024), umma_smem_desc(kq + off, 16, 1024), idesc, k > 0);
    }
    umma_commit(bar_m1);
  }
  {  // row norms while the MMA runs: thread -> (row, half)
    const int t = tid & 63, half = tid >> 6;
    const uint8_t* kb = smem + PrepSmem::KQ + half * 16384 + t * 128;
    const uint8_t* qb = kb + 8192;
    float sk = 0.f, sq = 0.f;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const uint4 ku = *reinterpret_cast<const uint4*>(kb + ch * 16);
      const uint4 qu = *reinterpret_cast<const uint4*>(qb + ch * 16);
      const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&ku);
      const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qu);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 kf = __bfloat1622float2(kp[j]), qf = __bfloat1622float2(qp[j]);
        sk += kf.x * kf.x + kf.y * kf.y;
        sq += qf.x * qf.x + qf.y * qf.y;
      }
    }
    s_pk[half * 64 + t] = sk;
    s_pq[half * 64 + t] = sq;
  }
  __syncthreads();
  if (tid < CC) {
    s_rk[tid] = rsqrtf(s_pk[tid] + s_pk[64 + tid] + a.eps);
    s_rq[tid] = rsqrtf(s_pq[tid] + s_pq[64 + tid] + a.eps) * a.scale;
  }
  ok = mbar_wait_bounded(bar_m1, 0, abort_flag);
  if (!ok) {
    if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
    *abort_flag = 1;
  }
  __syncthreads();
  if (*abort_flag) goto done;
  tc_fence_after();
  {
    // 2. rows 0-63: A (fp32, smem); rows 64-127: P (bf16, global)
    const int t = tid & 63;
    const float ct = s_c[t];
#pragma unroll 1
    for (int c0 = 0; c0 < CC; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + c0, r);
      tmem_ld_wait();
      if (tid < CC) {
        const float bt = s_beta[t] * s_rk[t];
        // Row t as 16 float4 whose positions are XOR-ed with (t & 15): the threads of a quarter-warp (rows 256
        // bytes apart) then hit different banks; scalar stores in row order would be a 32-way conflict.
        float4* arow_w = reinterpret_cast<float4*>(Am + t * CC);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float f[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = 4 * q + e, u = c0 + j;
            f[e] = (u < t) ? bt * __expf(ct - s_c[u]) * s_rk[u] * __uint_as_float(r[j]) : 0.f;
          }
          arow_w[((c0 >> 2) + q) ^ (t & 15)] = make_float4(f[0], f[1], f[2], f[3]);
        }
      } else {
        const float qt = s_rq[t];
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int u = c0 + j;
          const float p0 = (u <= t) ? qt * __expf(ct - s_c[u]) * s_rk[u] * __uint_as_float(r[j]) : 0.f;
          const float p1 = (u + 1 <= t) ? qt * __expf(ct - s_c[u + 1]) * s_rk[u + 1] * __uint_as_float(r[j + 1]) : 0.f;
          pk[j >> 1] = pack_bf16x2(p0, p1);
        }
        __nv_bfloat16* dst = a.P + (item * CC + t) * CC + c0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
      }
    }
  }
  __syncthreads();
  {
    // 3. T = (I + A)^-1 by 16 x 16 blocks, in place over A (fp32 rows, float4 positions XOR-ed with row & 15).
    //    Diagonal blocks: forward substitution inside the block, one column per thread.  Then block row by block
    //    row: X_ij = sum_{k=j..i-1} A_ik T_kj and T_ij = -T_ii X_ij for j < i.  A column-by-column substitution
    //    over all 64 rows is a chain of 2,016 dependent FMAs per thread; here every dot product is independent.
    auto am = [&](int r, int c) -> float& { return Am[r * CC + ((((c >> 2) ^ (r & 15)) << 2) | (c & 3))]; };
    float* Xs = reinterpret_cast<float*>(smem + PrepSmem::XS);
    if (tid < CC) {
      const int b0 = (tid >> 4) * 16, jc = tid & 15;
      float dcol[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        float acc = (r == jc) ? 1.f : 0.f;
#pragma unroll
        for (int m = 0; m < r; ++m) acc -= am(b0 + r, b0 + m) * dcol[m];
        dcol[r] = acc;
      }
      __syncwarp();   // a block's 16 columns sit in one warp: all have read A_bb before anyone overwrites it
#pragma unroll
      for (int r = 0; r < 16; ++r) am(b0 + r, b0 + jc) = dcol[r];
    }
    __syncthreads();
#pragma unroll 1
    for (int i = 1; i < 4; ++i) {
      for (int e = tid; e < i * 256; e += CTHREADS) {
        const int jb = e >> 8, r = (e >> 4) & 15, c = e & 15;
        float acc0 = 0.f, acc1 = 0.f;
        for (int k = jb; k < i; ++k) {
#pragma unroll
          for (int m = 0; m < 16; m += 2) {
            acc0 += am(16 * i + r, 16 * k + m) * am(16 * k + m, 16 * jb + c);
            acc1 += am(16 * i + r, 16 * k + m + 1) * am(16 * k + m + 1, 16 * jb + c);
          }
        }
        Xs[e] = acc0 + acc1;
      }
      __syncthreads();
      for (int e = tid; e < i * 256; e += CTHREADS) {
        const int jb = e >> 8, r = (e >> 4) & 15, c = e & 15;
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int m = 0; m < 16; m += 2) {   // T_ii is lower triangular: its upper entries are stored zeros
          acc0 += am(16 * i + r, 16 * i + m) * Xs[(jb << 8) + (m << 4) + c];
          acc1 += am(16 * i + r, 16 * i + m + 1) * Xs[(jb << 8) + ((m + 1) << 4) + c];
        }
        am(16 * i + r, 16 * jb + c) = -(acc0 + acc1);
      }
      __syncthreads();
    }
  }
  if (tid < CC) {
    // column j of T into registers, then the scaled bf16 operand tiles (they overwrite A) and the fp32 copy
    const int j = tid;
    float col[CC];
#pragma unroll
    for (int r = 0; r < CC; ++r)
      col[r] = Am[r * CC + ((((j >> 2) ^ (r & 15)) << 2) | (j & 3))];
    const float fj = s_beta[j];
    const float fk = fj * __expf(s_c[j]) * s_rk[j];
    // T' and T'' overwrite A: wait until both substitution warps have read their last row of it
    asm volatile("bar.sync 1, 64;" ::: "memory");
    uint8_t* tp = smem + PrepSmem::TP;
    uint8_t* tpp = smem + PrepSmem::TPP;
#pragma unroll
    for (int r = 0; r < CC; ++r) {
      const uint32_t off = csw128(r, j >> 3) + (j & 7) * 2;
      *reinterpret_cast<__nv_bfloat16*>(tp + off) = __float2bfloat16_rn(col[r] * fk);
      *reinterpret_cast<__nv_bfloat16*>(tpp + off) = __float2bfloat16_rn(col[r] * fj);
    }
    if (a.Tm) {
#pragma unroll
      for (int r = 0; r < CC; ++r) a.Tm[(item * CC + r) * CC + j] = col[r];
    }
  } else {
    // 4. Kd = e^{c_C - c_t} rk_t k_t and Qd = e^{c_t} rq_t q_t, one row per thread
    const int t = tid - CC;
    const float fk = __expf(s_c[CC - 1] - s_c[t]) * s_rk[t];
    const float fq = __expf(s_c[t]) * s_rq[t];
    __nv_bfloat16* kd = a.Kd + (item * CC + t) * CD;
    __nv_bfloat16* qd = a.Qd + (item * CC + t) * CD;
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {
      const uint8_t* kb = smem + PrepSmem::KQ + hb * 16384;
      const uint8_t* qb = kb + 8192;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 ku = *reinterpret_cast<const uint4*>(kb + csw128(t, ch));
        const uint4 qu = *reinterpret_cast<const uint4*>(qb + csw128(t, ch));
        const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&ku);
        const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qu);
        uint32_t ko[4], qo[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const float2 kf = __bfloat1622float2(kp[jj]), qf = __bfloat1622float2(qp[jj]);
          ko[jj] = pack_bf16x2(kf.x * fk, kf.y * fk);
          qo[jj] = pack_bf16x2(qf.x * fq, qf.y * fq);
        }
        *reinterpret_cast<uint4*>(kd + hb * 64 + ch * 8) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
        *reinterpret_cast<uint4*>(qd + hb * 64 + ch * 8) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
      }
    }
    if (t == 0) a.egam[item] = __expf(s_c[CC - 1]);
    if (a.aux) {
      float* ax = a.aux + item * 3 * CC;
      ax[t] = s_c[t];
      ax[CC + t] = s_rq[t];
      ax[2 * CC + t] = s_rk[t];
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // 5. W^T = K^T T'^T,  U^T = V^T T''^T   (A read MN-major from the TMA tiles)
  if (tid == 0) {
    constexpr uint32_t idesc = umma_idesc(128, CC, 1, 1, 0);
    const uint32_t kq = smem_u32(smem + PrepSmem::KQ), vv = smem_u32(smem + PrepSmem::V);
    const uint32_t tp = smem_u32(smem + PrepSmem::TP), tpp = smem_u32(smem + PrepSmem::TPP);
#pragma unroll
    for (int k = 0; k < CC / 16; ++k) {
      umma_bf16(tmem_base, umma_smem_desc(kq + k * 2048, 16384, 1024), umma_smem_desc(tp + k * 32, 16, 1024),
                idesc, k > 0);
    }
#pragma unroll
    for (int k = 0; k < CC / 16; ++k) {
      umma_bf16(tmem_base + 64, umma_smem_desc(vv + k * 2048, 8192, 1024), umma_smem_desc(tpp + k * 32, 16, 1024),
                idesc, k > 0);
    }
    umma_commit(bar_m2);
  }
  ok = mbar_wait_bounded(bar_m2, 0, abort_flag);
  if (!ok) {
    if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
    *abort_flag = 1;
  }
  __syncthreads();
  if (*abort_flag) goto done;
  tc_fence_after();
  {
    // 6. transpose W^T / U^T through smem (the K/Q/V tiles are dead now) and store 16-byte rows
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + PrepSmem::KQ);  // [64][128]
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
#pragma unroll 1
      for (int c0 = 0; c0 < CC; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + which * 64 + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[(c0 + j) * CD + tid] = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
      __syncthreads();
      __nv_bfloat16* dst = (which == 0 ? a.W : a.U) + item * CC * CD;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const int idx = v * CTHREADS + tid;  // 16-byte vector index
        *reinterpret_cast<uint4*>(dst + idx * 8) = *reinterpret_cast<const uint4*>(stage + idx * 8);
      }
      __syncthreads();
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

// ---------------------------------------------------------------------------------------------
// output kernel: O^T[dv x C] = S^T Qd^T + Vn^T P^T
// ---------------------------------------------------------------------------------------------
struct OutArgs {
  __nv_bfloat16* out;  // [B, T, H, dv]
  int T, H, n_chunks;
  int* status;
};
struct OutSmem {
  static constexpr int S = 0;          // S^T: 2 k-blocks [128 x 64] = 32 KB (reused as output staging)
  static constexpr int QD = 32768;     // 16 KB
  static constexpr int VN = 49152;     // 16 KB
  static constexpr int PT = 65536;     // 8 KB
  static constexpr int BARS = 73728;
  static constexpr int BYTES = BARS + 128 + 1024;
};

__global__ void __launch_bounds__(CTHREADS, 2)
gdn_chunk_out_kernel(const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmQd,
                     const __grid_constant__ CUtensorMap tmVn, const __grid_constant__ CUtensorMap tmP,
                     const OutArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OutSmem::BARS);
  uint64_t *bar_load = bars, *bar_m = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const long long item = blockIdx.x;
  const int i = static_cast<int>(item % a.n_chunks);
  const long long bh = item / a.n_chunks;
  const int h = static_cast<int>(bh % a.H);
  const long long b = bh / a.H;

  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_m, 1);
    *abort_flag = 0;
    mbar_fence_init();
    mbar_arrive_expect_tx(bar_load, 32768 + 16384 + 16384 + 8192);
    const int srow = static_cast<int>(item * CD), crow = static_cast<int>(item * CC);
    tma_load_2d(smem + OutSmem::S, &tmS, bar_load, 0, srow);
    tma_load_2d(smem + OutSmem::S + 16384, &tmS, bar_load, 64, srow);
    tma_load_2d(smem + OutSmem::QD, &tmQd, bar_load, 0, crow);
    tma_load_2d(smem + OutSmem::QD + 8192, &tmQd, bar_load, 64, crow);
    tma_load_2d(smem + OutSmem::VN, &tmVn, bar_load, 0, crow);
    tma_load_2d(smem + OutSmem::VN + 8192, &tmVn, bar_load, 64, crow);
    tma_load_2d(smem + OutSmem::PT, &tmP, bar_load, 0, crow);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  if (tid == 0) {
    if (mbar_wait_bounded(bar_load, 0, abort_flag)) {
      tc_fence_after();
      const uint32_t s = smem_u32(smem + OutSmem::S), qd = smem_u32(smem + OutSmem::QD);
      const uint32_t vn = smem_u32(smem + OutSmem::VN), pt = smem_u32(smem + OutSmem::PT);
      constexpr uint32_t id1 = umma_idesc(128, CC, 1, 0, 0);
#pragma unroll
      for (int k = 0; k < CD / 16; ++k) {
        const uint32_t kb = k >> 2, ks = (k & 3) * 32;
        umma_bf16(tmem_base, umma_smem_desc(s + kb * 16384 + ks, 16, 1024),
                  umma_smem_desc(qd + kb * 8192 + ks, 16, 1024), id1, k > 0);
      }
      constexpr uint32_t id2 = umma_idesc(128, CC, 1, 1, 0);
#pragma unroll
      for (int k = 0; k < CC / 16; ++k)
        umma_bf16(tmem_base, umma_smem_desc(vn + k * 2048, 8192, 1024), umma_smem_desc(pt + k * 32, 16, 1024), id2, 1u);
      umma_commit(bar_m);
    } else {
      if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_FULL);
      *abort_flag = 1;
    }
  }
  if (!mbar_wait_bounded(bar_m, 0, abort_flag)) {
    if (!*abort_flag) atomicCAS(a.status, 0, ERR_WAIT_TMEM_FULL);
    *abort_flag = 1;
  }
  __syncthreads();
  if (!*abort_flag) {
    tc_fence_after();
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + OutSmem::S);  // [64][128]
#pragma unroll 1
    for (int c0 = 0; c0 < CC; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) stage[(c0 + j) * CD + tid] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
    __syncthreads();
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const int idx = v * CTHREADS + tid;
      const int t = idx >> 4, ch = idx & 15;
      __nv_bfloat16* dst = a.out + (((b * a.T + static_cast<long long>(i) * CC + t) * a.H + h) * CD) + ch * 8;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(stage + idx * 8);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace cvb

using namespace cvb;

// q, k, v: bf16 views [B, T, H, 128] with unit inner stride, head stride 128 and a common token stride
// `tok_stride` (elements); batch stride = T * tok_stride.  beta, g: fp32 [B, T, H] contiguous.
// Outputs as documented in PrepArgs.  T must be a multiple of 64.
extern "C" int cvb_gdn_chunk_prep(const void* q, const void* k, const void* v, long long tok_stride, const float* beta,
                                  const float* g, long long B, int T, int H, float scale, float eps, void* W, void* U,
                                  void* Kd, void* Qd, void* P, float* egam, float* Tm, float* aux, int* status,
                                  void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (T % CC != 0 || (tok_stride % 8) != 0) return -1;
  const long long rows = B * T;
  if (rows > 0x7fffffffLL) return -2;
  CUtensorMap mq, mk, mv;
  if (make_tensor_map_2d(&mq, q, 2, static_cast<uint64_t>(H) * CD, rows, tok_stride * 2, 64, 64) ||
      make_tensor_map_2d(&mk, k, 2, static_cast<uint64_t>(H) * CD, rows, tok_stride * 2, 64, 64) ||
      make_tensor_map_2d(&mv, v, 2, static_cast<uint64_t>(H) * CD, rows, tok_stride * 2, 64, 64))
    return -10;
  PrepArgs a{};
  a.beta = beta; a.g = g; a.T = T; a.H = H; a.n_chunks = T / CC; a.scale = scale; a.eps = eps;
  a.W = static_cast<__nv_bfloat16*>(W); a.U = static_cast<__nv_bfloat16*>(U);
  a.Kd = static_cast<__nv_bfloat16*>(Kd); a.Qd = static_cast<__nv_bfloat16*>(Qd);
  a.P = static_cast<__nv_bfloat16*>(P); a.egam = egam; a.Tm = Tm; a.aux = aux; a.status = status;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PrepSmem::BYTES) !=
        cudaSuccess)
      return -11;
    attr = true;
  }
  const long long items = B * H * a.n_chunks;
  gdn_chunk_prep_kernel<<<static_cast<unsigned>(items), CTHREADS, PrepSmem::BYTES, static_cast<cudaStream_t>(stream)>>>(
      mq, mk, mv, a);
  return static_cast<int>(cudaGetLastError());
}

// ST: [BH, n, 128(dv), 128(dk)] bf16 chunk-start states (transposed); Qd, Vn: [BH, n, 64, 128]; P: [BH, n, 64, 64].
// out: bf16 [B, T, H, 128] contiguous.
extern "C" int cvb_gdn_chunk_out(const void* ST, const void* Qd, const void* Vn, const void* P, void* out, long long B,
                                 int T, int H, int* status, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (T % CC != 0) return -1;
  const int n = T / CC;
  const long long items = B * H * n;
  if (items * CD > 0x7fffffffLL) return -2;
  CUtensorMap ms, mq, mv, mp;
  if (make_tensor_map_2d(&ms, ST, 2, CD, items * CD, CD * 2, 64, 128) ||
      make_tensor_map_2d(&mq, Qd, 2, CD, items * CC, CD * 2, 64, 64) ||
      make_tensor_map_2d(&mv, Vn, 2, CD, items * CC, CD * 2, 64, 64) ||
      make_tensor_map_2d(&mp, P, 2, CC, items * CC, CC * 2, 64, 64))
    return -10;
  OutArgs a{};
  a.out = static_cast<__nv_bfloat16*>(out); a.T = T; a.H = H; a.n_chunks = n; a.status = status;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, OutSmem::BYTES) !=
        cudaSuccess)
      return -11;
    attr = true;
  }
  gdn_chunk_out_kernel<<<static_cast<unsigned>(items), CTHREADS, OutSmem::BYTES, static_cast<cudaStream_t>(stream)>>>(
      ms, mq, mv, mp, a);
  return static_cast<int>(cudaGetLastError());
}
