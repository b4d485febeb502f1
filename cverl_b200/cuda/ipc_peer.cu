// CUDA IPC handle export / import for same-node tensor hand-off between processes, and
// peer-access helpers used by the symmetric-memory kernels.
// Reference: src/rollout/gpu_ipc_rollout_batch.cc:30-139 (cudaIpcGetMemHandle on the data
// pointer, cudaIpcOpenMemHandle with lazy peer access, close on release).
#include <cuda_runtime.h>
#include <cstring>
#include <stdint.h>

extern "C" {

// Writes the 64-byte handle of the allocation containing `ptr` and the byte offset of `ptr` in it.
int cvb_ipc_get_handle(const void* ptr, unsigned char* handle64, long long* offset_bytes) {
  cudaIpcMemHandle_t h;
  // the handle names a whole allocation: find its base with the driver's address-range query
  typedef int (*RangeFn)(unsigned long long*, size_t*, unsigned long long);
  static RangeFn range_fn = nullptr;
  if (!range_fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      range_fn = reinterpret_cast<RangeFn>(sym);
  }
  void* base = const_cast<void*>(ptr);
  if (range_fn) {
    unsigned long long b = 0;
    size_t size = 0;
    if (range_fn(&b, &size, reinterpret_cast<unsigned long long>(ptr)) == 0) base = reinterpret_cast<void*>(b);
  }
  cudaError_t e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  std::memcpy(handle64, &h, 64);
  *offset_bytes = static_cast<long long>(static_cast<const char*>(ptr) - static_cast<const char*>(base));
  return 0;
}

// Maps a peer process's allocation; *out_base is the mapped base address.
int cvb_ipc_open_handle(const unsigned char* handle64, void** out_base) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(out_base, h, cudaIpcMemLazyEnablePeerAccess));
}

int cvb_ipc_close_handle(void* base) { return static_cast<int>(cudaIpcCloseMemHandle(base)); }

// cudaMalloc / cudaFree for buffers that must be IPC-exportable (outside the caching allocator).
int cvb_device_malloc(void** out, long long bytes) { return static_cast<int>(cudaMalloc(out, static_cast<size_t>(bytes))); }
int cvb_device_free(void* p) { return static_cast<int>(cudaFree(p)); }
int cvb_device_memset(void* p, int value, long long bytes, void* stream) {
  return static_cast<int>(cudaMemsetAsync(p, value, static_cast<size_t>(bytes), static_cast<cudaStream_t>(stream)));
}
// Device-to-device copy on `stream`; either side may be a peer-mapped address (the copy engines move the bytes
// over NVLink without occupying an SM).
int cvb_device_memcpy_async(void* dst, const void* src, long long bytes, void* stream) {
  return static_cast<int>(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice,
                                          static_cast<cudaStream_t>(stream)));
}
int cvb_can_access_peer(int device, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, device, peer) != cudaSuccess) return 0;
  return ok;
}
}
