// C interface of the tcgen05 GEMM (see gemm_tcgen05.cu).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum CvbGemmEpilogue {
  EPI_STORE_BF16 = 0,    // C(bf16)  = alpha * acc
  EPI_STORE_F32 = 1,     // C(fp32)  = alpha * acc
  EPI_ATOMIC_F32 = 2,    // C(fp32) += alpha * acc  (red.global.add; split-K and grad accumulation)
  EPI_LSE_PARTIAL = 3,   // per (row, N tile): running max and sum-exp; target logit gather
  EPI_SOFTMAX_GRAD = 4,  // C(bf16)  = g[row] * (onehot(target) - exp(acc - lse[row]))
};

// Arguments of one GEMM launch.  All pointers are device pointers.
//   a_mn = 0: A is [M, K] row-major with row stride lda (elements)
//   a_mn = 1: A is [K, M] row-major with row stride lda
//   b_mn = 0: B is [N, K] row-major with row stride ldb      (C = A * B^T)
//   b_mn = 1: B is [K, N] row-major with row stride ldb      (C = A * B)
typedef struct CvbGemmArgs {
  const void* A;
  const void* B;
  void* C;
  int64_t lda, ldb, ldc;
  int32_t M, N, K;
  int32_t a_mn, b_mn;
  int32_t epi;
  float alpha;
  int32_t split_k;   // 0 = automatic
  int32_t block_n;   // 0 / 256 / 128
  int32_t group_m;   // 0 = default rasterisation band
  int32_t max_ctas;  // 0 = one per SM
  // grouped (MoE) modes
  const int32_t* tile_group;       // [ceil(M/128)] expert of each M tile, -1 = skip
  int64_t b_group_rows;            // row offset into B per group
  int64_t b_total_rows;            // total rows of the stacked B (0 = single matrix)
  const int32_t* k_group_offsets;  // [num_groups+1] K range per group (multiples of 64)
  int32_t num_groups;
  int64_t c_group_stride;          // element offset into C per group
  // LM-head epilogues
  const long long* targets;  // [M] int64
  float* part_max;         // [n_tiles, M]
  float* part_sum;         // [n_tiles, M]
  float* tgt_logit;        // [M]
  const float* lse;        // [M]
  const float* gscale;     // [M]
  int32_t* status;         // device status word (0 = OK), required
  // EPI_STORE_BF16 only: the same tile is also stored at the same offsets into these buffers, e.g. peer
  // GPUs' mapped copies of C (plain stores over NVLink from the epilogue warps, tile by tile)
  void* mirror[7];
  int32_t n_mirror;
  // EPI_STORE_BF16, scatter_rows > 0 (a multiple of 128): row block `row / scatter_rows` of the output is stored
  // ONLY at scatter_base[block] + row * ldc + col, and C is not written - the reduce-scatter of a tensor-parallel
  // partial product: every row block goes straight to the rank that owns those rows (its own memory or a peer's,
  // over NVLink).  The caller folds the owner's row origin into each base pointer.
  void* scatter_base[8];
  int32_t scatter_rows;
  // EPI_STORE_BF16 with row_addr != nullptr: output row r is stored ONLY at byte address row_addr[r] (+ 2 * col),
  // rows with address 0 are dropped, C is not written.  The combine of expert-parallel MoE rides on the down
  // projection's epilogue this way: every expert output row goes straight back into the buffer of the rank its
  // token came from (own memory or a peer's, over NVLink).  Addresses must be 16-byte aligned; N % 64 == 0.
  const long long* row_addr;
} CvbGemmArgs;

// Launches on `stream` (a cudaStream_t).  Returns 0 or a negative/CUDA error.
int cvb_gemm_bf16(const CvbGemmArgs* args, void* stream);

#ifdef __cplusplus
}

#include <cuda.h>
namespace cvb {
struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  float alpha;
  int epi;
  int split_k, kb_per_split;
  int m_tiles, n_tiles, kblocks, total_items;
  int group_m;
  const int* tile_group;
  long long b_group_rows;
  const int* k_group_offsets;
  long long c_group_stride;
  const long long* targets;
  float* part_max;
  float* part_sum;
  float* tgt_logit;
  const float* lse;
  const float* gscale;
  int* status;
  void* mirror[7];
  int n_mirror;
  void* scatter_base[8];
  int scatter_rows;
  const long long* row_addr;
  int staged_store;  // bf16 epilogue through shared memory (coalesced 128-byte segments)
};
int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);
}  // namespace cvb
#endif
