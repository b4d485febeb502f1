// Shared-memory region and the single-slot request/response transport built on it.
//
// One POSIX shm region holds a header and one payload area; two named semaphores
// ("/<name>.req", "/<name>.resp") hand the slot back and forth.  Header fields: magic
// 'CVST', version, payload capacity, request size, response size, request id, response
// status (0 ok, 1 handler error, 2 response too large).  Both sides wait with
// sem_timedwait; a timeout is reported to the caller instead of blocking forever.
// Payloads are opaque byte strings here; the Python layer serialises RolloutRequest /
// RolloutResponse with little-endian length-prefixed fields.
// Reference: src/rollout/shared_memory.cc:29-110, src/rollout/shared_memory_transport.cc:
// 23-38,202-335,373-518.
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <fcntl.h>
#include <semaphore.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

constexpr uint32_t kMagic = 0x54535643u;  // 'CVST' little endian
constexpr uint32_t kVersion = 1;

struct Header {
  uint32_t magic;
  uint32_t version;
  uint64_t payload_capacity;
  uint64_t request_size;
  uint64_t response_size;
  uint64_t request_id;
  uint32_t response_status;
  uint32_t reserved;
};

struct Region {
  std::string name;
  int fd = -1;
  void* addr = nullptr;
  size_t size = 0;
  bool owner = false;
};

struct Transport {
  Region region;
  sem_t* req = SEM_FAILED;
  sem_t* resp = SEM_FAILED;
  std::string req_name, resp_name;
  bool owner = false;
  uint64_t next_id = 1;
  Header* header() { return static_cast<Header*>(region.addr); }
  uint8_t* payload() { return static_cast<uint8_t*>(region.addr) + sizeof(Header); }
};

bool open_region(Region& r, const std::string& name, size_t size, bool create) {
  r.name = name;
  r.owner = create;
  r.size = size;
  if (create) shm_unlink(name.c_str());
  r.fd = shm_open(name.c_str(), create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
  if (r.fd < 0) return false;
  if (create && ftruncate(r.fd, static_cast<off_t>(size)) != 0) return false;
  if (!create) {
    struct stat st;
    if (fstat(r.fd, &st) != 0) return false;
    r.size = static_cast<size_t>(st.st_size);
  }
  r.addr = mmap(nullptr, r.size, PROT_READ | PROT_WRITE, MAP_SHARED, r.fd, 0);
  if (r.addr == MAP_FAILED) {
    r.addr = nullptr;
    return false;
  }
  return true;
}

void close_region(Region& r) {
  if (r.addr) munmap(r.addr, r.size);
  if (r.fd >= 0) close(r.fd);
  if (r.owner) shm_unlink(r.name.c_str());
  r.addr = nullptr;
  r.fd = -1;
}

// 0 = acquired, 1 = timed out, 2 = error
int timed_wait(sem_t* s, int64_t timeout_ms) {
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  ts.tv_sec += timeout_ms / 1000;
  ts.tv_nsec += (timeout_ms % 1000) * 1000000L;
  if (ts.tv_nsec >= 1000000000L) {
    ts.tv_sec += 1;
    ts.tv_nsec -= 1000000000L;
  }
  for (;;) {
    if (sem_timedwait(s, &ts) == 0) return 0;
    if (errno == EINTR) continue;
    return errno == ETIMEDOUT ? 1 : 2;
  }
}

}  // namespace

extern "C" {

// ---- plain region (RAII in the Python wrapper) -------------------------------------------------
void* cverl_shm_region_open(const char* name, int64_t size, int create) {
  auto* r = new Region();
  if (!open_region(*r, name, static_cast<size_t>(size), create != 0)) {
    close_region(*r);
    delete r;
    return nullptr;
  }
  return r;
}
void* cverl_shm_region_addr(void* h) { return static_cast<Region*>(h)->addr; }
int64_t cverl_shm_region_size(void* h) { return static_cast<int64_t>(static_cast<Region*>(h)->size); }
void cverl_shm_region_close(void* h) {
  auto* r = static_cast<Region*>(h);
  close_region(*r);
  delete r;
}

// ---- transport -----------------------------------------------------------------------------------
void* cverl_shm_transport_open(const char* name, int64_t payload_capacity, int create) {
  auto* t = new Transport();
  t->owner = create != 0;
  t->req_name = std::string(name) + ".req";
  t->resp_name = std::string(name) + ".resp";
  const size_t size = sizeof(Header) + static_cast<size_t>(payload_capacity);
  bool ok = open_region(t->region, name, size, t->owner);
  if (ok && t->owner) {
    sem_unlink(t->req_name.c_str());
    sem_unlink(t->resp_name.c_str());
    std::memset(t->region.addr, 0, sizeof(Header));
    Header* h = t->header();
    h->magic = kMagic;
    h->version = kVersion;
    h->payload_capacity = static_cast<uint64_t>(payload_capacity);
  }
  if (ok) {
    t->req = sem_open(t->req_name.c_str(), t->owner ? O_CREAT : 0, 0600, 0);
    t->resp = sem_open(t->resp_name.c_str(), t->owner ? O_CREAT : 0, 0600, 0);
    ok = t->req != SEM_FAILED && t->resp != SEM_FAILED;
  }
  if (ok && !t->owner) ok = t->header()->magic == kMagic && t->header()->version == kVersion;
  if (!ok) {
    if (t->req != SEM_FAILED) sem_close(t->req);
    if (t->resp != SEM_FAILED) sem_close(t->resp);
    close_region(t->region);
    delete t;
    return nullptr;
  }
  return t;
}

void cverl_shm_transport_close(void* h) {
  auto* t = static_cast<Transport*>(h);
  if (t->req != SEM_FAILED) sem_close(t->req);
  if (t->resp != SEM_FAILED) sem_close(t->resp);
  if (t->owner) {
    sem_unlink(t->req_name.c_str());
    sem_unlink(t->resp_name.c_str());
  }
  close_region(t->region);
  delete t;
}

int64_t cverl_shm_transport_capacity(void* h) {
  return static_cast<int64_t>(static_cast<Transport*>(h)->header()->payload_capacity);
}

// Client: post a request and wait for the response.
// Returns >= 0 response size; -1 request too large; -2 timeout; -3 semaphore error;
// -4 server reported a handler error; -5 server response did not fit; -6 request id mismatch.
int64_t cverl_shm_client_call(void* h, const void* request, int64_t request_size, void* response,
                              int64_t response_capacity, int64_t timeout_ms) {
  auto* t = static_cast<Transport*>(h);
  Header* hd = t->header();
  if (request_size < 0 || static_cast<uint64_t>(request_size) > hd->payload_capacity) return -1;
  const uint64_t id = t->next_id++;
  std::memcpy(t->payload(), request, static_cast<size_t>(request_size));
  hd->request_size = static_cast<uint64_t>(request_size);
  hd->response_size = 0;
  hd->request_id = id;
  hd->response_status = 0;
  __sync_synchronize();
  if (sem_post(t->req) != 0) return -3;
  const int w = timed_wait(t->resp, timeout_ms);
  if (w == 1) return -2;
  if (w != 0) return -3;
  __sync_synchronize();
  if (hd->request_id != id) return -6;
  if (hd->response_status == 1) return -4;
  if (hd->response_status == 2) return -5;
  const int64_t n = static_cast<int64_t>(hd->response_size);
  if (n > response_capacity) return -5;
  std::memcpy(response, t->payload(), static_cast<size_t>(n));
  return n;
}

// Server: wait for a request.  Returns its size, -2 on timeout, -3 on error.
int64_t cverl_shm_server_wait(void* h, void* request, int64_t capacity, int64_t timeout_ms) {
  auto* t = static_cast<Transport*>(h);
  const int w = timed_wait(t->req, timeout_ms);
  if (w == 1) return -2;
  if (w != 0) return -3;
  __sync_synchronize();
  const int64_t n = static_cast<int64_t>(t->header()->request_size);
  if (n > capacity) return -3;
  std::memcpy(request, t->payload(), static_cast<size_t>(n));
  return n;
}

// Server: publish the response (status 0) or an error status (1 handler error, 2 oversize).
int cverl_shm_server_reply(void* h, const void* response, int64_t size, int status) {
  auto* t = static_cast<Transport*>(h);
  Header* hd = t->header();
  if (status == 0 && (size < 0 || static_cast<uint64_t>(size) > hd->payload_capacity)) {
    status = 2;
    size = 0;
  }
  if (status == 0) std::memcpy(t->payload(), response, static_cast<size_t>(size));
  hd->response_size = status == 0 ? static_cast<uint64_t>(size) : 0;
  hd->response_status = static_cast<uint32_t>(status);
  __sync_synchronize();
  return sem_post(t->resp) == 0 ? 0 : 1;
}
}
