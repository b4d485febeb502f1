// Kernels that use the NVSwitch multicast path (NVLS): one address that the switch maps onto the same buffer of
// every GPU bound to a multicast object.
//
//  * multimem_broadcast_store   trainer -> rollout weight push as ONE store per 16 bytes: `multimem.st` hands the
//                               data to the switch once and the switch writes it into every bound GPU's buffer,
//                               so the sender's links carry the payload once instead of once per receiver
//  * multimem_reduce_scatter    ZeRO gradient reduce-scatter: `multimem.ld_reduce.add` returns the sum over all
//                               GPUs' copies, reduced in the switch, so this GPU's inbound links carry its shard
//                               once instead of once per peer; accumulates into the shard gradient and adds the
//                               shard's squared norm
//  * multimem_allreduce_rows    sum of bf16 partial results over all GPUs, written back to every GPU:
//                               `ld_reduce` + `multimem.st` (the one-shot all-reduce of a tensor-parallel block)
//
// The multicast address comes from the framework's symmetric-memory allocator (parallel/nvls.py); these kernels
// never synchronise ranks themselves: the caller brackets them with flag barriers (symm_ops.cu) whose waits are
// bounded.  The reference does these with ncclBroadcast / ncclReduceScatter / ncclAllReduce
// (src/distributed/weight_sync.cc:140-189, src/distributed/optimizer_sharding.cc:463-585).
#include "ptx.cuh"

namespace cvb {

constexpr int NV_THREADS = 256;

__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_add_f32x4(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.weak.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
// eight bf16 values per call, summed over the GPUs with fp32 accumulation inside the switch
__device__ __forceinline__ uint4 multimem_ld_reduce_add_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.weak.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

__global__ void __launch_bounds__(NV_THREADS)
multimem_broadcast_store_kernel(const uint4* __restrict__ src, uint4* mc_dst, long long n16) {
  // four independent 16-byte loads in flight per thread before the first multicast store
  const long long stride = static_cast<long long>(gridDim.x) * NV_THREADS;
  long long i = static_cast<long long>(blockIdx.x) * NV_THREADS + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    multimem_st_v4(mc_dst + i, a);
    multimem_st_v4(mc_dst + i + stride, b);
    multimem_st_v4(mc_dst + i + 2 * stride, c);
    multimem_st_v4(mc_dst + i + 3 * stride, d);
  }
  for (; i < n16; i += stride) multimem_st_v4(mc_dst + i, src[i]);
}

// out[i] (+)= scale * sum over GPUs of buf[begin + i];  sq += sum of the new out[i]^2 when sq != nullptr
__global__ void __launch_bounds__(NV_THREADS)
multimem_reduce_scatter_kernel(const float* mc_src, long long begin, long long n, float scale, float* __restrict__ out,
                               int accumulate, float* __restrict__ sq) {
  __shared__ float sh[NV_THREADS / 32];
  float acc = 0.f;
  const long long nv = n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * NV_THREADS;
  auto finish = [&](float4 s, long long i) {
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    if (accumulate) {
      const float4 o = *reinterpret_cast<const float4*>(out + i * 4);
      s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
    }
    *reinterpret_cast<float4*>(out + i * 4) = s;
    acc += (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w);
  };
  long long i = static_cast<long long>(blockIdx.x) * NV_THREADS + threadIdx.x;
  for (; i + 3 * stride < nv; i += 4 * stride) {      // four reducing loads in flight per thread
    const float4 a = multimem_ld_reduce_add_f32x4(mc_src + begin + i * 4);
    const float4 b = multimem_ld_reduce_add_f32x4(mc_src + begin + (i + stride) * 4);
    const float4 c = multimem_ld_reduce_add_f32x4(mc_src + begin + (i + 2 * stride) * 4);
    const float4 d = multimem_ld_reduce_add_f32x4(mc_src + begin + (i + 3 * stride) * 4);
    finish(a, i); finish(b, i + stride); finish(c, i + 2 * stride); finish(d, i + 3 * stride);
  }
  for (; i < nv; i += stride) finish(multimem_ld_reduce_add_f32x4(mc_src + begin + i * 4), i);
  if (sq == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < NV_THREADS / 32 ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (threadIdx.x == 0) atomicAdd(sq, r);
  }
}

// this rank's slice [begin, begin + n) of a bf16 buffer: every GPU's copy becomes the sum over GPUs
__global__ void __launch_bounds__(NV_THREADS)
multimem_allreduce_bf16_kernel(__nv_bfloat16* mc_buf, long long begin, long long n) {
  const long long nv = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * NV_THREADS + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * NV_THREADS) {
    __nv_bfloat16* a = mc_buf + begin + i * 8;
    const uint4 s = multimem_ld_reduce_add_bf16x8(a);
    multimem_st_v4(a, s);
  }
}

static int nv_grid(long long nvec, int max_blocks) {
  long long b = (nvec + NV_THREADS - 1) / NV_THREADS;
  const long long cap = max_blocks > 0 ? max_blocks : 148 * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : static_cast<int>(b);
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_multimem_broadcast_store(const void* src, void* mc_dst, long long nbytes, int max_blocks,
                                            void* stream) {
  if (nbytes % 16 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(mc_dst)) & 15) || !mc_dst)
    return -1;
  if (nbytes == 0) return 0;
  multimem_broadcast_store_kernel<<<nv_grid(nbytes / 16, max_blocks), NV_THREADS, 0,
                                    static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src),
                                                                         static_cast<uint4*>(mc_dst), nbytes / 16);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_multimem_reduce_scatter(const void* mc_src, long long begin, long long n, float scale, float* out,
                                           int accumulate, float* sq, int max_blocks, void* stream) {
  if (n % 4 || begin % 4 || !mc_src ||
      ((reinterpret_cast<uintptr_t>(mc_src) | reinterpret_cast<uintptr_t>(out)) & 15))
    return -1;
  if (n == 0) return 0;
  multimem_reduce_scatter_kernel<<<nv_grid(n / 4, max_blocks), NV_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(mc_src), begin, n, scale, out, accumulate, sq);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cvb_multimem_allreduce_bf16(void* mc_buf, long long begin, long long n, int max_blocks, void* stream) {
  if (n % 8 || begin % 8 || !mc_buf || (reinterpret_cast<uintptr_t>(mc_buf) & 15)) return -1;
  if (n == 0) return 0;
  multimem_allreduce_bf16_kernel<<<nv_grid(n / 8, max_blocks), NV_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(mc_buf), begin, n);
  return static_cast<int>(cudaGetLastError());
}
