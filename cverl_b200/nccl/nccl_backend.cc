// Native NCCL communicator: one ncclComm_t with a dedicated non-blocking CUDA stream, hand-off to the caller's
// stream by events, sub-communicators by ncclCommSplit, and rendezvous through a file holding the unique id.
//
// What the reference does (src/distributed/nccl_collectives.cc): rank 0 of a communicator writes the 128-byte
// ncclUniqueId atomically (tmp + rename) and the others poll for it (:156-196); every communicator owns a
// non-blocking stream (:211-213); before an operation that stream waits for the caller's current stream through
// a throw-away event (:136-143); afterwards either the host synchronises (default) or, in "async" mode, an event
// makes the caller's stream wait and the tensors are kept alive in a list (:278-312); sub-groups are split once
// per rank list (:252-276); all-to-all and send+recv are grouped ncclSend / ncclRecv pairs (:412-492).
//
// Here the C layer works on raw device pointers and cudaStream_t handles and keeps two events per communicator
// instead of creating one per call; tensor lifetime is the Python wrapper's business (it tells the caching
// allocator about the communicator stream instead of holding references).  Every entry point returns 0 or a
// negative code and leaves a message for cvn_last_error().
#include <cuda_runtime.h>
#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>

namespace {

thread_local std::string g_err;

int fail(const std::string& what) {
  g_err = what;
  return -1;
}

struct Comm {
  ncclComm_t comm = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ready = nullptr;   // caller's stream -> communicator stream
  cudaEvent_t done = nullptr;    // communicator stream -> caller's stream
  int rank = 0, world = 1, device = 0;
  bool sync_after_op = true;
  bool owns_stream = true;       // false: the stream was lent by the caller and outlives the communicator
};

#define CVN_CUDA(expr)                                                            \
  do {                                                                            \
    cudaError_t e_ = (expr);                                                      \
    if (e_ != cudaSuccess) return fail(std::string(#expr) + ": " + cudaGetErrorString(e_)); \
  } while (0)
#define CVN_NCCL(expr)                                                            \
  do {                                                                            \
    ncclResult_t r_ = (expr);                                                     \
    if (r_ != ncclSuccess) return fail(std::string(#expr) + ": " + ncclGetErrorString(r_)); \
  } while (0)

bool dtype_of(int code, ncclDataType_t* out, size_t* bytes) {
  switch (code) {  // 0 f32, 1 f16, 2 bf16, 3 i32, 4 i64, 5 u8
    case 0: *out = ncclFloat32; *bytes = 4; return true;
    case 1: *out = ncclFloat16; *bytes = 2; return true;
    case 2: *out = ncclBfloat16; *bytes = 2; return true;
    case 3: *out = ncclInt32; *bytes = 4; return true;
    case 4: *out = ncclInt64; *bytes = 8; return true;
    case 5: *out = ncclUint8; *bytes = 1; return true;
  }
  return false;
}

bool op_of(int code, ncclRedOp_t* out) {
  switch (code) {  // 0 sum, 1 max, 2 min, 3 prod, 4 avg
    case 0: *out = ncclSum; return true;
    case 1: *out = ncclMax; return true;
    case 2: *out = ncclMin; return true;
    case 3: *out = ncclProd; return true;
    case 4: *out = ncclAvg; return true;
  }
  return false;
}

// communicator stream waits for everything the caller has enqueued so far
int enter(Comm* c, cudaStream_t caller) {
  CVN_CUDA(cudaSetDevice(c->device));
  CVN_CUDA(cudaEventRecord(c->ready, caller));
  CVN_CUDA(cudaStreamWaitEvent(c->stream, c->ready, 0));
  return 0;
}

// the caller's stream (or the host) waits for the operation
int leave(Comm* c, cudaStream_t caller) {
  if (c->sync_after_op) {
    CVN_CUDA(cudaStreamSynchronize(c->stream));
    return 0;
  }
  CVN_CUDA(cudaEventRecord(c->done, c->stream));
  CVN_CUDA(cudaStreamWaitEvent(caller, c->done, 0));
  return 0;
}

Comm* finish_create(ncclComm_t comm, int rank, int world, int device, bool sync_after_op, cudaStream_t lent) {
  Comm* c = new Comm;
  c->stream = lent;
  c->owns_stream = lent == nullptr;
  c->comm = comm;
  c->rank = rank;
  c->world = world;
  c->device = device;
  c->sync_after_op = sync_after_op;
  if ((c->owns_stream && cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) ||
      cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess) {
    g_err = "cannot create the communicator's stream / events";
    ncclCommAbort(comm);
    delete c;
    return nullptr;
  }
  return c;
}

}  // namespace

extern "C" {

const char* cvn_last_error() { return g_err.c_str(); }

int cvn_unique_id_bytes() { return static_cast<int>(sizeof(ncclUniqueId)); }

int cvn_unique_id_create(unsigned char* id128) {
  ncclUniqueId id;
  CVN_NCCL(ncclGetUniqueId(&id));
  std::memcpy(id128, &id, sizeof(id));
  return 0;
}

// Atomic publish: write `path.tmp`, then rename.
int cvn_unique_id_write_file(const char* path, const unsigned char* id128) {
  const std::string tmp = std::string(path) + ".tmp";
  FILE* f = std::fopen(tmp.c_str(), "wb");
  if (!f) return fail("cannot open " + tmp);
  const size_t n = std::fwrite(id128, 1, sizeof(ncclUniqueId), f);
  std::fclose(f);
  if (n != sizeof(ncclUniqueId)) return fail("short write to " + tmp);
  if (std::rename(tmp.c_str(), path) != 0) return fail(std::string("cannot rename to ") + path);
  return 0;
}

// Polls for the file (`polls` tries, `poll_ms` apart); -2 when it never appears with the full size.
int cvn_unique_id_read_file(const char* path, unsigned char* id128, int polls, int poll_ms) {
  for (int i = 0; i < (polls > 0 ? polls : 1); ++i) {
    FILE* f = std::fopen(path, "rb");
    if (f) {
      const size_t n = std::fread(id128, 1, sizeof(ncclUniqueId), f);
      std::fclose(f);
      if (n == sizeof(ncclUniqueId)) return 0;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(poll_ms > 0 ? poll_ms : 25));
  }
  g_err = std::string("timed out waiting for NCCL id file ") + path;
  return -2;
}

// `stream`: a non-blocking stream lent by the caller for the communicator's lifetime and longer (a framework's
// pooled stream, which an allocator may still touch after the communicator is gone), or null to own one.
void* cvn_comm_create(int rank, int world, int device, const unsigned char* id128, int sync_after_op, void* stream) {
  if (rank < 0 || world <= 0 || rank >= world) {
    g_err = "rank out of range";
    return nullptr;
  }
  if (cudaSetDevice(device) != cudaSuccess) {
    g_err = "cudaSetDevice failed";
    return nullptr;
  }
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  ncclComm_t comm;
  ncclResult_t r = ncclCommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess) {
    g_err = std::string("ncclCommInitRank: ") + ncclGetErrorString(r);
    return nullptr;
  }
  return finish_create(comm, rank, world, device, sync_after_op != 0, static_cast<cudaStream_t>(stream));
}

// Collective over the parent: members of one sub-group pass the same `color` (>= 0) and their index as `key`;
// a rank outside every group passes color -1 and gets a null handle.
void* cvn_comm_split(void* parent, int color, int key, int new_world, void* stream) {
  Comm* p = static_cast<Comm*>(parent);
  if (!p) return nullptr;
  cudaSetDevice(p->device);
  ncclComm_t sub = nullptr;
  ncclResult_t r = ncclCommSplit(p->comm, color < 0 ? NCCL_SPLIT_NOCOLOR : color, key, &sub, nullptr);
  if (r != ncclSuccess) {
    g_err = std::string("ncclCommSplit: ") + ncclGetErrorString(r);
    return nullptr;
  }
  if (color < 0 || sub == nullptr) return nullptr;
  return finish_create(sub, key, new_world, p->device, p->sync_after_op, static_cast<cudaStream_t>(stream));
}

int cvn_comm_destroy(void* h) {
  Comm* c = static_cast<Comm*>(h);
  if (!c) return 0;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  ncclCommDestroy(c->comm);
  cudaEventDestroy(c->ready);
  cudaEventDestroy(c->done);
  if (c->owns_stream) cudaStreamDestroy(c->stream);
  delete c;
  return 0;
}

void* cvn_comm_stream(void* h) { return h ? static_cast<Comm*>(h)->stream : nullptr; }
int cvn_comm_rank(void* h) { return h ? static_cast<Comm*>(h)->rank : -1; }
int cvn_comm_world(void* h) { return h ? static_cast<Comm*>(h)->world : 0; }

int cvn_all_reduce(void* h, const void* send, void* recv, long long count, int dtype, int op, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  ncclRedOp_t ro;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz) || !op_of(op, &ro)) return fail("all_reduce: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclAllReduce(send, recv, static_cast<size_t>(count), dt, ro, c->comm, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

int cvn_broadcast(void* h, const void* send, void* recv, long long count, int dtype, int root, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz) || root < 0 || root >= c->world) return fail("broadcast: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclBroadcast(send, recv, static_cast<size_t>(count), dt, root, c->comm, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

// recv holds world * count elements
int cvn_all_gather(void* h, const void* send, void* recv, long long count, int dtype, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz)) return fail("all_gather: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclAllGather(send, recv, static_cast<size_t>(count), dt, c->comm, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

// send holds world * count elements, recv count
int cvn_reduce_scatter(void* h, const void* send, void* recv, long long count, int dtype, int op, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  ncclRedOp_t ro;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz) || !op_of(op, &ro)) return fail("reduce_scatter: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclReduceScatter(send, recv, static_cast<size_t>(count), dt, ro, c->comm, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

// equal split on dim 0: chunk p of `send` goes to rank p, chunk p of `recv` comes from rank p
int cvn_all_to_all(void* h, const void* send, void* recv, long long count_per_rank, int dtype, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz)) return fail("all_to_all: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  const char* s = static_cast<const char*>(send);
  char* r = static_cast<char*>(recv);
  const size_t chunk = static_cast<size_t>(count_per_rank) * esz;
  CVN_NCCL(ncclGroupStart());
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank) continue;
    ncclSend(s + p * chunk, static_cast<size_t>(count_per_rank), dt, p, c->comm, c->stream);
    ncclRecv(r + p * chunk, static_cast<size_t>(count_per_rank), dt, p, c->comm, c->stream);
  }
  CVN_NCCL(ncclGroupEnd());
  CVN_CUDA(cudaMemcpyAsync(r + c->rank * chunk, s + c->rank * chunk, chunk, cudaMemcpyDeviceToDevice, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

int cvn_send(void* h, const void* send, long long count, int dtype, int peer, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz) || peer < 0 || peer >= c->world || peer == c->rank)
    return fail("send: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclSend(send, static_cast<size_t>(count), dt, peer, c->comm, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

int cvn_recv(void* h, void* recv, long long count, int dtype, int peer, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz) || peer < 0 || peer >= c->world || peer == c->rank)
    return fail("recv: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclRecv(recv, static_cast<size_t>(count), dt, peer, c->comm, c->stream));
  return leave(c, static_cast<cudaStream_t>(caller));
}

// one grouped send + recv (a ring hop): cannot deadlock whatever the order of the peers' calls
int cvn_send_recv(void* h, const void* send, long long send_count, int dst, void* recv, long long recv_count,
                  int src, int dtype, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  ncclDataType_t dt;
  size_t esz;
  if (!c || !dtype_of(dtype, &dt, &esz) || dst < 0 || dst >= c->world || src < 0 || src >= c->world)
    return fail("send_recv: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclGroupStart());
  ncclSend(send, static_cast<size_t>(send_count), dt, dst, c->comm, c->stream);
  ncclRecv(recv, static_cast<size_t>(recv_count), dt, src, c->comm, c->stream);
  CVN_NCCL(ncclGroupEnd());
  return leave(c, static_cast<cudaStream_t>(caller));
}

// 1-float all-reduce on `scratch` (a device float), then a host wait on the communicator stream
int cvn_barrier(void* h, float* scratch, void* caller) {
  Comm* c = static_cast<Comm*>(h);
  if (!c || !scratch) return fail("barrier: bad argument");
  if (enter(c, static_cast<cudaStream_t>(caller))) return -1;
  CVN_NCCL(ncclAllReduce(scratch, scratch, 1, ncclFloat32, ncclSum, c->comm, c->stream));
  CVN_CUDA(cudaStreamSynchronize(c->stream));
  return 0;
}

}  // extern "C"
