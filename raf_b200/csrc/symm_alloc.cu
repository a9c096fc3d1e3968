// Symmetric device memory for the library's own collectives: one allocation per rank that
// every rank of the node has mapped, plus (where the GPUs offer it) one NVSwitch multicast
// address bound to all of them.  The reference has no counterpart: every collective buffer
// of src/op/dialect/nccl/nccl.cc comes from its memory pool and is only ever touched by NCCL.
//
// Per rank: cuMemCreate with a shareable (file descriptor) handle, descriptors handed to the
// peers over abstract unix sockets (SCM_RIGHTS), cuMemImportFromShareableHandle + cuMemMap of
// every peer's memory; rank 0 creates the multicast object, every rank adds its device, and -
// after a barrier over the same sockets, because binding needs all devices added - binds its
// memory and maps the multicast address.  Every wait has the caller's deadline.  The driver
// entry points are looked up at run time (cudaGetDriverEntryPoint), so the library itself
// does not link libcuda and still loads on a machine without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "common.h"

namespace rafb200 {
namespace {

using Clock = std::chrono::steady_clock;

struct Driver {
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExport = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImport = nullptr;
  decltype(&cuMemAddressReserve) AddressReserve = nullptr;
  decltype(&cuMemAddressFree) AddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGranularity = nullptr;
  decltype(&cuMulticastCreate) McCreate = nullptr;
  decltype(&cuMulticastAddDevice) McAddDevice = nullptr;
  decltype(&cuMulticastBindMem) McBindMem = nullptr;
  decltype(&cuMulticastUnbind) McUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) McGranularity = nullptr;
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  bool ok = false;
};

template <typename F>
bool entry(const char* name, F* fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  *fn = reinterpret_cast<F>(p);
  return true;
}

const Driver& driver() {
  static Driver d = [] {
    Driver x;
    x.ok = entry("cuMemCreate", &x.MemCreate) && entry("cuMemRelease", &x.MemRelease) &&
           entry("cuMemExportToShareableHandle", &x.MemExport) &&
           entry("cuMemImportFromShareableHandle", &x.MemImport) &&
           entry("cuMemAddressReserve", &x.AddressReserve) && entry("cuMemAddressFree", &x.AddressFree) &&
           entry("cuMemMap", &x.MemMap) && entry("cuMemUnmap", &x.MemUnmap) &&
           entry("cuMemSetAccess", &x.MemSetAccess) &&
           entry("cuMemGetAllocationGranularity", &x.MemGranularity) && entry("cuDeviceGet", &x.DeviceGet) &&
           entry("cuDeviceGetAttribute", &x.DeviceGetAttribute) && entry("cuGetErrorString", &x.GetErrorString);
    // the multicast calls may be missing on an old driver: then there is simply no multicast address
    entry("cuMulticastCreate", &x.McCreate);
    entry("cuMulticastAddDevice", &x.McAddDevice);
    entry("cuMulticastBindMem", &x.McBindMem);
    entry("cuMulticastUnbind", &x.McUnbind);
    entry("cuMulticastGetGranularity", &x.McGranularity);
    return x;
  }();
  return d;
}

int cu_fail(CUresult r, const char* what) {
  const char* msg = nullptr;
  if (driver().GetErrorString) driver().GetErrorString(r, &msg);
  return set_error(RAFB200_CUDA_ERROR, "%s: %s", what, msg ? msg : "driver error");
}
#define RAFB200_CU(expr)                               \
  do {                                                 \
    CUresult r__ = (expr);                             \
    if (r__ != CUDA_SUCCESS) return cu_fail(r__, #expr); \
  } while (0)

// ---- descriptors between the ranks of a node --------------------------------------------
// Rank r listens on the abstract unix socket "\0rafb200.<key>.<r>".  A peer connects, sends one
// request byte and gets the answer: 'm' this rank's memory descriptor, 'c' the multicast
// descriptor (rank 0 only), 'b' a barrier: rank 0 answers when every other rank has asked.
sockaddr_un address_of(const std::string& key, int rank, socklen_t* len) {
  sockaddr_un a;
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  const std::string name = "rafb200." + key + "." + std::to_string(rank);
  const size_t n = name.size() < sizeof(a.sun_path) - 2 ? name.size() : sizeof(a.sun_path) - 2;
  memcpy(a.sun_path + 1, name.data(), n);  // sun_path[0] = 0: abstract name, nothing in the file system
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
  return a;
}

bool send_fd(int sock, int fd) {
  char byte = 'k';
  iovec io{&byte, 1};
  char ctl[CMSG_SPACE(sizeof(int))];
  memset(ctl, 0, sizeof(ctl));
  msghdr msg{};
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  if (fd >= 0) {
    msg.msg_control = ctl;
    msg.msg_controllen = sizeof(ctl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  return ::sendmsg(sock, &msg, MSG_NOSIGNAL) == 1;
}

// -> 0 and *fd (or -1 when none came with the byte), or -1 on error / timeout
int recv_fd(int sock, int* fd, int timeout_ms) {
  pollfd p{sock, POLLIN, 0};
  if (::poll(&p, 1, timeout_ms) <= 0) return -1;
  char byte = 0;
  iovec io{&byte, 1};
  char ctl[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  msg.msg_control = ctl;
  msg.msg_controllen = sizeof(ctl);
  if (::recvmsg(sock, &msg, 0) != 1) return -1;
  *fd = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c))
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(fd, CMSG_DATA(c), sizeof(int));
  return 0;
}

struct Server {
  int listen_fd = -1;
  int world = 1, rank = 0;
  std::atomic<int> mem_fd{-1}, mc_fd{-1};
  std::atomic<bool> stop{false};
  std::thread thread;
  std::vector<int> waiting;  // rank 0: connections parked at the barrier
  std::atomic<int> root_gen{0}, done_gen{0};  // rank 0's own arrivals / barriers released

  void run() {
    while (!stop.load()) {
      release_barrier();
      pollfd p{listen_fd, POLLIN, 0};
      if (::poll(&p, 1, 5) <= 0) continue;
      int c = ::accept(listen_fd, nullptr, nullptr);
      if (c < 0) continue;
      pollfd q{c, POLLIN, 0};
      char req = 0;
      if (::poll(&q, 1, 2000) <= 0 || ::recv(c, &req, 1, 0) != 1) {
        ::close(c);
        continue;
      }
      if (req == 'b') {
        waiting.push_back(c);
        continue;
      }
      // a descriptor that is not there yet: the peer asks again
      const int fd = req == 'm' ? mem_fd.load() : mc_fd.load();
      if (fd >= 0) send_fd(c, fd);
      ::close(c);
    }
    for (int w : waiting) ::close(w);
  }

  // everybody else has asked and rank 0 itself has arrived: let them go
  void release_barrier() {
    if ((int)waiting.size() < world - 1 || root_gen.load() == done_gen.load()) return;
    for (int i = 0; i < world - 1; ++i) {
      send_fd(waiting[i], -1);
      ::close(waiting[i]);
    }
    waiting.erase(waiting.begin(), waiting.begin() + (world - 1));
    done_gen.fetch_add(1);
  }

  int start(const std::string& key, int world_, int rank_) {
    world = world_;
    rank = rank_;
    listen_fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (listen_fd < 0) return set_error(RAFB200_IO_ERROR, "socket: %s", strerror(errno));
    socklen_t len = 0;
    sockaddr_un a = address_of(key, rank, &len);
    if (::bind(listen_fd, reinterpret_cast<sockaddr*>(&a), len) != 0 || ::listen(listen_fd, 64) != 0) {
      const int e = errno;
      ::close(listen_fd);
      listen_fd = -1;
      return set_error(RAFB200_IO_ERROR, "cannot listen for the peers (key %s): %s", key.c_str(), strerror(e));
    }
    thread = std::thread([this] { run(); });
    return RAFB200_OK;
  }

  void finish() {
    stop.store(true);
    if (thread.joinable()) thread.join();
    if (listen_fd >= 0) ::close(listen_fd);
    listen_fd = -1;
  }
};

// Asks rank `peer` for `what` until the deadline; -> RAFB200_OK (and *fd when a descriptor came)
int ask(const std::string& key, int peer, char what, int* fd, Clock::time_point deadline, int timeout_ms) {
  while (true) {
    int s = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) return set_error(RAFB200_IO_ERROR, "socket: %s", strerror(errno));
    socklen_t len = 0;
    sockaddr_un a = address_of(key, peer, &len);
    if (::connect(s, reinterpret_cast<sockaddr*>(&a), len) == 0 && ::send(s, &what, 1, MSG_NOSIGNAL) == 1) {
      const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
      int got = -1;
      const int rc = recv_fd(s, &got, left > 0 ? (int)left : 0);
      ::close(s);
      if (rc == 0 && (what == 'b' || got >= 0)) {
        if (fd) *fd = got;
        return RAFB200_OK;
      }
    } else {
      ::close(s);
    }
    if (Clock::now() > deadline)
      return set_error(RAFB200_TIMEOUT, "rafb200_symm_alloc: rank %d did not answer within %d ms", peer, timeout_ms);
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

int barrier(Server& srv, const std::string& key, Clock::time_point deadline, int timeout_ms) {
  if (srv.world == 1) return RAFB200_OK;
  if (srv.rank != 0) return ask(key, 0, 'b', nullptr, deadline, timeout_ms);
  const int gen = srv.root_gen.fetch_add(1) + 1;
  while (srv.done_gen.load() < gen) {
    if (Clock::now() > deadline)
      return set_error(RAFB200_TIMEOUT, "rafb200_symm_alloc: not every rank reached the barrier within %d ms", timeout_ms);
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  return RAFB200_OK;
}

std::atomic<int> g_symm_seq{0};

}  // namespace
}  // namespace rafb200

struct rafb200_symm_s {
  int world = 1, rank = 0, device = 0;
  size_t bytes = 0;  // mapped size (the request rounded up to the granularity)
  CUmemGenericAllocationHandle mem = 0, mc = 0;
  std::vector<CUmemGenericAllocationHandle> imported;  // peers' memory (0 at [rank])
  std::vector<void*> peer;                             // where each rank's memory is mapped here
  void* mc_ptr = nullptr;
  bool bound = false;
};

using namespace rafb200;

static int map_here(const Driver& d, CUmemGenericAllocationHandle h, size_t bytes, size_t gran, int device, void** out) {
  CUdeviceptr va = 0;
  RAFB200_CU(d.AddressReserve(&va, bytes, gran, 0, 0));
  CUresult r = d.MemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    d.AddressFree(va, bytes);
    return cu_fail(r, "cuMemMap");
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.MemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap(va, bytes);
    d.AddressFree(va, bytes);
    return cu_fail(r, "cuMemSetAccess");
  }
  *out = reinterpret_cast<void*>(va);
  return RAFB200_OK;
}

extern "C" {

int rafb200_symm_free(rafb200_symm_t s) {
  if (!s) return RAFB200_OK;
  const Driver& d = driver();
  cudaDeviceSynchronize();
  if (s->mc_ptr) {
    d.MemUnmap(reinterpret_cast<CUdeviceptr>(s->mc_ptr), s->bytes);
    d.AddressFree(reinterpret_cast<CUdeviceptr>(s->mc_ptr), s->bytes);
  }
  if (s->bound && d.McUnbind) {
    CUdevice dev = 0;
    d.DeviceGet(&dev, s->device);
    d.McUnbind(s->mc, dev, 0, s->bytes);
  }
  if (s->mc) d.MemRelease(s->mc);
  for (int q = 0; q < (int)s->peer.size(); ++q) {
    if (!s->peer[q]) continue;
    d.MemUnmap(reinterpret_cast<CUdeviceptr>(s->peer[q]), s->bytes);
    d.AddressFree(reinterpret_cast<CUdeviceptr>(s->peer[q]), s->bytes);
    if (q != s->rank && s->imported[q]) d.MemRelease(s->imported[q]);
  }
  if (s->mem) d.MemRelease(s->mem);
  delete s;
  return RAFB200_OK;
}

int rafb200_symm_alloc(int world, int rank, int device, size_t bytes, const char* key, int want_multicast,
                       int timeout_ms, rafb200_symm_t* out) {
  RAFB200_REQUIRE(out, "rafb200_symm_alloc: NULL result pointer");
  *out = nullptr;
  RAFB200_REQUIRE(world >= 1 && rank >= 0 && rank < world && bytes > 0 && timeout_ms > 0 && key,
                  "rafb200_symm_alloc: bad arguments");
  RAFB200_CUDA(cudaSetDevice(device));
  RAFB200_CUDA(cudaFree(nullptr));  // the device's context exists from here on
  const Driver& d = driver();
  if (!d.ok) return set_error(RAFB200_CUDA_ERROR, "rafb200_symm_alloc: the driver lacks the virtual memory calls");
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  const std::string k = std::string(key) + "." + std::to_string(++g_symm_seq);  // same order on every rank

  CUdevice dev = 0;
  RAFB200_CU(d.DeviceGet(&dev, device));
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  RAFB200_CU(d.MemGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  int mc_ok = 0;
  if (want_multicast && world > 1 && d.McCreate && d.McAddDevice && d.McBindMem && d.McGranularity)
    d.DeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  CUmulticastObjectProp mprop{};
  mprop.numDevices = (unsigned)world;
  mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  if (mc_ok) {
    // the multicast object has a granularity of its own; every rank computes the same size
    size_t mgran = 0;
    mprop.size = bytes;
    if (d.McGranularity(&mgran, &mprop, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mgran > gran) gran = mgran;
  }
  const size_t size = (bytes + gran - 1) / gran * gran;
  mprop.size = size;

  auto* s = new rafb200_symm_s();
  s->world = world;
  s->rank = rank;
  s->device = device;
  s->bytes = size;
  s->imported.assign((size_t)world, 0);
  s->peer.assign((size_t)world, nullptr);
  Server srv;
  int my_fd = -1, mc_fd = -1;
  int rc = RAFB200_OK;
  auto fail = [&](int code) {
    srv.finish();
    if (my_fd >= 0) ::close(my_fd);
    if (mc_fd >= 0) ::close(mc_fd);
    rafb200_symm_free(s);
    return code;
  };
  {
    CUresult r = d.MemCreate(&s->mem, size, &prop, 0);
    if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMemCreate"));
  }
  rc = map_here(d, s->mem, size, gran, device, &s->peer[(size_t)rank]);
  if (rc != RAFB200_OK) return fail(rc);
  if (world == 1) {
    *out = s;
    return RAFB200_OK;
  }
  {
    CUresult r = d.MemExport(&my_fd, s->mem, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMemExportToShareableHandle"));
  }
  rc = srv.start(k, world, rank);
  if (rc != RAFB200_OK) return fail(rc);
  srv.mem_fd.store(my_fd);

  // every peer's memory, mapped here
  for (int q = 0; q < world; ++q) {
    if (q == rank) continue;
    int fd = -1;
    rc = ask(k, q, 'm', &fd, deadline, timeout_ms);
    if (rc != RAFB200_OK) return fail(rc);
    CUresult r = d.MemImport(&s->imported[(size_t)q], reinterpret_cast<void*>((uintptr_t)fd),
                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMemImportFromShareableHandle"));
    rc = map_here(d, s->imported[(size_t)q], size, gran, device, &s->peer[(size_t)q]);
    if (rc != RAFB200_OK) return fail(rc);
  }

  if (mc_ok) {
    // rank 0 creates the object, everybody adds its device, and only then may anybody bind
    if (rank == 0) {
      CUresult r = d.McCreate(&s->mc, &mprop);
      if (r == CUDA_SUCCESS) r = d.MemExport(&mc_fd, s->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMulticastCreate"));
      srv.mc_fd.store(mc_fd);
    } else {
      int fd = -1;
      rc = ask(k, 0, 'c', &fd, deadline, timeout_ms);
      if (rc != RAFB200_OK) return fail(rc);
      CUresult r = d.MemImport(&s->mc, reinterpret_cast<void*>((uintptr_t)fd), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMemImportFromShareableHandle (multicast)"));
    }
    CUresult r = d.McAddDevice(s->mc, dev);
    if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMulticastAddDevice"));
    rc = barrier(srv, k, deadline, timeout_ms);
    if (rc != RAFB200_OK) return fail(rc);
    r = d.McBindMem(s->mc, 0, s->mem, 0, size, 0);
    if (r != CUDA_SUCCESS) return fail(cu_fail(r, "cuMulticastBindMem"));
    s->bound = true;
    rc = map_here(d, s->mc, size, gran, device, &s->mc_ptr);
    if (rc != RAFB200_OK) return fail(rc);
  }
  // nobody leaves (and stops answering) before everybody has what it asked for
  rc = barrier(srv, k, deadline, timeout_ms);
  if (rc != RAFB200_OK) return fail(rc);
  srv.finish();
  ::close(my_fd);
  if (mc_fd >= 0) ::close(mc_fd);
  *out = s;
  return RAFB200_OK;
}

size_t rafb200_symm_bytes(rafb200_symm_t s) { return s ? s->bytes : 0; }

int rafb200_symm_pointers(rafb200_symm_t s, void** peer, void** multicast) {
  RAFB200_REQUIRE(s && peer, "rafb200_symm_pointers: NULL argument");
  for (int q = 0; q < s->world; ++q) peer[q] = s->peer[(size_t)q];
  if (multicast) *multicast = s->mc_ptr;
  return RAFB200_OK;
}

}  // extern "C"
