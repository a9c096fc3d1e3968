// Communicator lifecycle and the collective entry points.
//
// One process per GPU.  The global communicator is an NCCL communicator whose
// 128-byte id is published by rank 0 through a file store, as the reference
// does when no MPI is present (src/distributed/cuda/nccl_communicator.cc:20-69),
// or handed in by the caller.  Differences from the reference, all on the
// failure path: the id exchange and ncclCommInitRank have a host-side deadline
// (the latter runs on a helper thread that is abandoned when the deadline
// passes), errors are returned instead of exit(), and rafb200_comm_check polls
// NCCL's asynchronous error state.
#include <nccl.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <thread>

#include "common.h"

struct rafb200_comm_s {
  int size = 1;
  int rank = 0;
  int device = 0;
  bool is_void = true;  // world of one: no NCCL underneath
  ncclComm_t nccl = nullptr;
  bool borrowed = false;   // adopted from the caller: never destroyed here
  // buffers from rafb200_comm_alloc: pointer -> (registration handle or NULL, from ncclMemAlloc?)
  struct Reg {
    void* handle;
    bool nccl_mem;
  };
  std::map<void*, Reg> regs;
  std::string store_file;  // file this rank published (removed on destroy)
  // sub-communicators by rank list (the reference's CommunicatorPool,
  // include/raf/communicator.h:104-147), owned by the global communicator
  std::map<std::vector<int>, rafb200_comm_s*> subs;
  int timeout_ms = 60000;
};

namespace rafb200 {

using Clock = std::chrono::steady_clock;

static int nccl_fail(ncclResult_t r, const char* what) {
  return set_error(RAFB200_NCCL_ERROR, "%s: %s", what, ncclGetErrorString(r));
}

// The communicators are non-blocking (their creation has a deadline, see init_rank), so a call
// may answer ncclInProgress: the work is then being queued by NCCL's own thread, and nothing
// that relies on it being on the stream may follow before ncclCommGetAsyncError reports
// ncclSuccess.  Every entry point therefore waits for that (bounded by the communicator's
// timeout) before it returns; inside a group only the closing ncclGroupEnd does.
static int finish_call(rafb200_comm_s* c, ncclResult_t r, const char* what);
#define RAFB200_NCCL(comm, expr)                            \
  do {                                                      \
    int rc__ = finish_call((comm), (expr), #expr);          \
    if (rc__ != RAFB200_OK) return rc__;                    \
  } while (0)

// src/op/dialect/nccl/communication_utils.h:31-48 (int8, int64, uint8, f16, f32, f64), plus bf16
static int to_nccl_dtype(int dtype, ncclDataType_t* out) {
  switch (dtype) {
    case RAFB200_F32: *out = ncclFloat32; return RAFB200_OK;
    case RAFB200_F16: *out = ncclFloat16; return RAFB200_OK;
    case RAFB200_BF16: *out = ncclBfloat16; return RAFB200_OK;
    case RAFB200_F64: *out = ncclFloat64; return RAFB200_OK;
    case RAFB200_I8: *out = ncclInt8; return RAFB200_OK;
    case RAFB200_U8: *out = ncclUint8; return RAFB200_OK;
    case RAFB200_I64: *out = ncclInt64; return RAFB200_OK;
  }
  return set_error(RAFB200_INVALID_ARGUMENT, "NotImplementedError: no NCCL type for dtype %d", dtype);
}
static size_t comm_dtype_size(int dtype) {
  switch (dtype) {
    case RAFB200_F16: case RAFB200_BF16: return 2;
    case RAFB200_F64: case RAFB200_I64: return 8;
    case RAFB200_I8: case RAFB200_U8: return 1;
    default: return 4;
  }
}

// "sum" | "prod" | "min" | "max" | "avg"  (src/op/dialect/nccl/nccl.cc:57-72)
static int to_nccl_op(const char* computation, ncclRedOp_t* out) {
  if (!computation) return set_error(RAFB200_INVALID_ARGUMENT, "NULL computation");
  if (!strcmp(computation, "sum")) *out = ncclSum;
  else if (!strcmp(computation, "prod")) *out = ncclProd;
  else if (!strcmp(computation, "min")) *out = ncclMin;
  else if (!strcmp(computation, "max")) *out = ncclMax;
  else if (!strcmp(computation, "avg")) *out = ncclAvg;
  else return set_error(RAFB200_INVALID_ARGUMENT, "Invalid computation %s", computation);
  return RAFB200_OK;
}

// ---- file store ---------------------------------------------------------------
static std::atomic<int> g_store_seq{0};

static std::string store_dir(const char* store_path) {
  if (store_path && *store_path) return store_path;
  const char* env = getenv("RAF_FILE_STORE_PATH");
  if (env && *env) return env;
  return "/tmp/.raf_file_store";
}

static int store_publish(const std::string& file, const void* data, size_t n) {
  const std::string tmp = file + ".tmp." + std::to_string((long)getpid());
  int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return set_error(RAFB200_IO_ERROR, "cannot create %s: %s", tmp.c_str(), strerror(errno));
  ssize_t w = ::write(fd, data, n);
  ::close(fd);
  if (w != (ssize_t)n) {
    ::unlink(tmp.c_str());
    return set_error(RAFB200_IO_ERROR, "short write to %s", tmp.c_str());
  }
  if (::rename(tmp.c_str(), file.c_str()) != 0) {  // atomic: readers see nothing or all of it
    ::unlink(tmp.c_str());
    return set_error(RAFB200_IO_ERROR, "cannot publish %s: %s", file.c_str(), strerror(errno));
  }
  return RAFB200_OK;
}

static int store_fetch(const std::string& file, void* data, size_t n, int timeout_ms) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  while (true) {
    int fd = ::open(file.c_str(), O_RDONLY);
    if (fd >= 0) {
      ssize_t r = ::read(fd, data, n);
      ::close(fd);
      if (r == (ssize_t)n) return RAFB200_OK;
    }
    if (Clock::now() > deadline)
      return set_error(RAFB200_TIMEOUT, "no communicator id at %s after %d ms", file.c_str(),
                       timeout_ms);
    std::this_thread::sleep_for(std::chrono::milliseconds(10));  // nccl_utils.h:247
  }
}

// Communicator creation with a deadline: a non-blocking communicator
// (ncclCommInitRankConfig, blocking = 0) is polled with ncclCommGetAsyncError until
// it is ready; a peer that never arrives costs `timeout_ms`, after which the
// half-built communicator is released with ncclCommAbort and the caller gets
// RAFB200_TIMEOUT.  (The reference calls the blocking ncclCommInitRank and waits forever,
// src/distributed/cuda/nccl_communicator.cc:113.)
static int wait_ready(ncclComm_t comm, int timeout_ms, const char* what) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  while (true) {
    ncclResult_t st = ncclSuccess;
    ncclResult_t r = ncclCommGetAsyncError(comm, &st);
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommGetAsyncError");
    if (st == ncclSuccess) return RAFB200_OK;
    if (st != ncclInProgress) return nccl_fail(st, what);
    if (Clock::now() > deadline) return set_error(RAFB200_TIMEOUT, "%s: not every rank joined within %d ms", what, timeout_ms);
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
}

static int finish_call(rafb200_comm_s* c, ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return RAFB200_OK;
  if (r != ncclInProgress || !c || !c->nccl) return nccl_fail(r, what);
  const auto deadline = Clock::now() + std::chrono::milliseconds(c->timeout_ms > 0 ? c->timeout_ms : 60000);
  while (true) {
    ncclResult_t st = ncclSuccess;
    ncclResult_t q = ncclCommGetAsyncError(c->nccl, &st);
    if (q != ncclSuccess) return nccl_fail(q, "ncclCommGetAsyncError");
    if (st == ncclSuccess) return RAFB200_OK;
    if (st != ncclInProgress) return nccl_fail(st, what);
    if (Clock::now() > deadline) return set_error(RAFB200_TIMEOUT, "%s: still in progress after %d ms", what, c->timeout_ms);
    std::this_thread::yield();
  }
}

static int init_rank(rafb200_comm_s* c, const ncclUniqueId& id, int timeout_ms) {
  RAFB200_CUDA(cudaSetDevice(c->device));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  ncclComm_t comm = nullptr;
  ncclResult_t r = ncclCommInitRankConfig(&comm, c->size, id, c->rank, &cfg);
  if (r != ncclSuccess && r != ncclInProgress) return nccl_fail(r, "ncclCommInitRankConfig");
  int rc = wait_ready(comm, timeout_ms, "ncclCommInitRankConfig");
  if (rc != RAFB200_OK) {
    if (comm) ncclCommAbort(comm);
    return rc;
  }
  c->nccl = comm;
  return RAFB200_OK;
}

}  // namespace rafb200

using namespace rafb200;

extern "C" {

int rafb200_unique_id(void* id128) {
  RAFB200_REQUIRE(id128, "rafb200_unique_id: NULL buffer");
  static_assert(sizeof(ncclUniqueId) == 128, "NCCL id is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = ncclGetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  memcpy(id128, &id, sizeof(id));
  return RAFB200_OK;
}

int rafb200_comm_create_with_id(int world_size, int rank, int device, const void* id128,
                                int timeout_ms, rafb200_comm_t* comm) {
  RAFB200_REQUIRE(comm, "rafb200_comm_create: NULL result pointer");
  *comm = nullptr;
  RAFB200_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size,
                  "rafb200_comm_create: rank %d outside world of %d", rank, world_size);
  RAFB200_REQUIRE(timeout_ms > 0, "rafb200_comm_create: timeout must be positive");
  RAFB200_CUDA(cudaSetDevice(device));
  auto* c = new rafb200_comm_s();
  c->size = world_size;
  c->rank = rank;
  c->device = device;
  if (world_size > 1) {
    if (!id128) {
      delete c;
      return set_error(RAFB200_INVALID_ARGUMENT, "rafb200_comm_create: NULL id");
    }
    c->is_void = false;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    c->timeout_ms = timeout_ms;
    int rc = init_rank(c, id, timeout_ms);
    if (rc != RAFB200_OK) {
      delete c;
      return rc;
    }
  }
  *comm = c;
  return RAFB200_OK;
}

int rafb200_store_exchange(int rank, const char* store_path, int key, void* data, size_t nbytes,
                           int timeout_ms) {
  RAFB200_REQUIRE(rank >= 0 && key >= 0 && data && nbytes > 0 && timeout_ms > 0,
                  "rafb200_store_exchange: bad argument");
  const std::string dir = store_dir(store_path);
  ::mkdir(dir.c_str(), 0777);  // nccl_communicator.cc:28-33; fine if it exists
  const std::string file = dir + "/" + std::to_string(key);
  if (rank == 0) return store_publish(file, data, nbytes);
  return store_fetch(file, data, nbytes, timeout_ms);
}

int rafb200_comm_adopt(void* nccl_comm, int world_size, int rank, rafb200_comm_t* comm) {
  RAFB200_REQUIRE(comm, "rafb200_comm_adopt: NULL result pointer");
  *comm = nullptr;
  RAFB200_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size,
                  "rafb200_comm_adopt: rank %d outside world of %d", rank, world_size);
  RAFB200_REQUIRE(world_size == 1 || nccl_comm, "rafb200_comm_adopt: NULL ncclComm_t");
  auto* c = new rafb200_comm_s();
  c->size = world_size;
  c->rank = rank;
  if (cudaGetDevice(&c->device) != cudaSuccess) c->device = 0;
  if (world_size > 1) {
    c->is_void = false;
    c->borrowed = true;
    c->nccl = static_cast<ncclComm_t>(nccl_comm);
    int n = 0, r = -1;
    if (ncclCommCount(c->nccl, &n) != ncclSuccess || ncclCommUserRank(c->nccl, &r) != ncclSuccess ||
        n != world_size || r != rank) {
      delete c;
      return set_error(RAFB200_INVALID_ARGUMENT,
                       "rafb200_comm_adopt: communicator reports rank %d of %d, caller said %d of %d",
                       r, n, rank, world_size);
    }
  }
  *comm = c;
  return RAFB200_OK;
}

int rafb200_comm_create(int world_size, int rank, int device, const char* store_path,
                        int timeout_ms, rafb200_comm_t* comm) {
  RAFB200_REQUIRE(comm, "rafb200_comm_create: NULL result pointer");
  *comm = nullptr;
  RAFB200_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size,
                  "rafb200_comm_create: rank %d outside world of %d", rank, world_size);
  RAFB200_REQUIRE(timeout_ms > 0, "rafb200_comm_create: timeout must be positive");
  if (world_size == 1) return rafb200_comm_create_with_id(1, 0, device, nullptr, timeout_ms, comm);

  const int seq = ++g_store_seq;  // every rank creates its communicators in the same order
  const std::string file = store_dir(store_path) + "/" + std::to_string(seq);
  ncclUniqueId id;
  if (rank == 0) {
    ncclResult_t r = ncclGetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  }
  {
    int rc = rafb200_store_exchange(rank, store_path, seq, &id, sizeof(id), timeout_ms);
    if (rc != RAFB200_OK) return rc;
  }
  int rc = rafb200_comm_create_with_id(world_size, rank, device, &id, timeout_ms, comm);
  if (rank == 0) {
    if (rc == RAFB200_OK) (*comm)->store_file = file;  // every rank has joined: safe to remove later
    else ::unlink(file.c_str());
  }
  return rc;
}

int rafb200_comm_destroy(rafb200_comm_t c) {
  if (!c) return RAFB200_OK;
  int rc = RAFB200_OK;
  // Buffers the caller forgot to hand back: deregister and free them with the communicator.
  while (!c->regs.empty()) rafb200_comm_free(c, c->regs.begin()->first);
  for (auto& kv : c->subs) rafb200_comm_destroy(kv.second);
  c->subs.clear();
  if (c->nccl && !c->borrowed) {
    // a non-blocking communicator is finalised first (that may still be in progress when the
    // call returns), then destroyed
    rc = finish_call(c, ncclCommFinalize(c->nccl), "ncclCommFinalize");
    ncclResult_t r = ncclCommDestroy(c->nccl);
    if (r != ncclSuccess && rc == RAFB200_OK) rc = nccl_fail(r, "ncclCommDestroy");
  }
  if (!c->store_file.empty()) ::unlink(c->store_file.c_str());
  delete c;
  return rc;
}

int rafb200_comm_alloc(rafb200_comm_t c, size_t bytes, void** ptr) {
  RAFB200_REQUIRE(c && ptr && bytes > 0, "rafb200_comm_alloc: bad arguments");
  *ptr = nullptr;
  const char* off = getenv("RAFB200_NCCL_REGISTER");
  const bool want = !c->is_void && !(off && off[0] == '0');
  rafb200_comm_s::Reg reg{nullptr, false};
  void* p = nullptr;
  if (want && ncclMemAlloc(&p, bytes) == ncclSuccess && p) {
    reg.nccl_mem = true;
    if (finish_call(c, ncclCommRegister(c->nccl, p, bytes, &reg.handle), "ncclCommRegister") != RAFB200_OK)
      reg.handle = nullptr;
  } else {
    p = nullptr;
    RAFB200_CUDA(cudaMalloc(&p, bytes));
  }
  c->regs[p] = reg;
  *ptr = p;
  return RAFB200_OK;
}

int rafb200_comm_free(rafb200_comm_t c, void* ptr) {
  if (!c || !ptr) return RAFB200_OK;
  auto it = c->regs.find(ptr);
  RAFB200_REQUIRE(it != c->regs.end(), "rafb200_comm_free: pointer was not allocated by rafb200_comm_alloc");
  int rc = RAFB200_OK;
  if (it->second.handle) rc = finish_call(c, ncclCommDeregister(c->nccl, it->second.handle), "ncclCommDeregister");
  if (it->second.nccl_mem) {
    if (ncclMemFree(ptr) != ncclSuccess) rc = set_error(RAFB200_NCCL_ERROR, "ncclMemFree failed");
  } else {
    cudaFree(ptr);
  }
  c->regs.erase(it);
  return rc;
}

int rafb200_comm_sub(rafb200_comm_t c, int n_groups, const int* group_sizes, const int* ranks,
                     rafb200_comm_t* sub) {
  RAFB200_REQUIRE(c && sub, "rafb200_comm_sub: NULL argument");
  *sub = nullptr;
  if (n_groups == 0) {  // no rank_list: the global communicator itself
    *sub = c;
    return RAFB200_OK;
  }
  RAFB200_REQUIRE(n_groups > 0 && group_sizes && ranks, "rafb200_comm_sub: bad rank list");
  // key of the pool: the rank list, flattened with separators
  std::vector<int> key;
  int total = 0, my_group = -1, my_rank = -1;
  for (int g = 0; g < n_groups; ++g) {
    RAFB200_REQUIRE(group_sizes[g] > 0, "rafb200_comm_sub: empty group %d", g);
    for (int i = 0; i < group_sizes[g]; ++i) {
      const int r = ranks[total + i];
      RAFB200_REQUIRE(r >= 0 && r < c->size, "rafb200_comm_sub: rank %d outside the communicator of %d", r, c->size);
      if (r == c->rank && my_group < 0) {  // communicator.cc:38-46: the first group that names this rank
        my_group = g;
        my_rank = i;
      }
      key.push_back(r);
    }
    key.push_back(-1);
    total += group_sizes[g];
  }
  auto it = c->subs.find(key);
  if (it != c->subs.end()) {
    *sub = it->second;
    return RAFB200_OK;
  }
  auto* s = new rafb200_comm_s();
  s->device = c->device;
  s->timeout_ms = c->timeout_ms;
  if (my_group >= 0) {
    s->size = group_sizes[my_group];
    s->rank = my_rank;
  }  // else: a world of one (communicator.cc:48-58)
  bool any_group = false;  // a group of two or more ranks: only then is NCCL needed at all
  for (int g = 0; g < n_groups; ++g) any_group = any_group || group_sizes[g] > 1;
  if (!c->is_void && any_group) {
    // As the reference does (nccl_communicator.cc:115-158), every group gets a communicator of
    // its own from an id that its first rank draws.  The ids travel over the parent: one
    // all-gather of a 128-byte record per rank, which every rank of the parent takes part in -
    // also those that no group names.  (No file store is needed, so this works for adopted
    // communicators too.)
    const int n = c->size;
    ncclUniqueId mine;
    memset(&mine, 0, sizeof(mine));
    const bool needs_nccl = my_group >= 0 && s->size > 1;
    if (needs_nccl && my_rank == 0) {
      ncclResult_t r = ncclGetUniqueId(&mine);
      if (r != ncclSuccess) {
        delete s;
        return nccl_fail(r, "ncclGetUniqueId");
      }
    }
    std::vector<ncclUniqueId> all((size_t)n);
    unsigned char* dbuf = nullptr;
    cudaStream_t xs = nullptr;
    cudaEvent_t done = nullptr;
    int rc = RAFB200_OK;
    auto cuda_ok = [&](cudaError_t e, const char* what) {
      if (e != cudaSuccess && rc == RAFB200_OK) rc = set_error(RAFB200_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
      return e == cudaSuccess;
    };
    if (cuda_ok(cudaMalloc(reinterpret_cast<void**>(&dbuf), sizeof(mine) * ((size_t)n + 1)), "cudaMalloc") &&
        cuda_ok(cudaStreamCreateWithFlags(&xs, cudaStreamNonBlocking), "cudaStreamCreate") &&
        cuda_ok(cudaEventCreateWithFlags(&done, cudaEventDisableTiming), "cudaEventCreate") &&
        cuda_ok(cudaMemcpyAsync(dbuf, &mine, sizeof(mine), cudaMemcpyHostToDevice, xs), "cudaMemcpyAsync")) {
      rc = finish_call(c, ncclAllGather(dbuf, dbuf + sizeof(mine), sizeof(mine), ncclUint8, c->nccl, xs), "ncclAllGather");
      if (rc == RAFB200_OK &&
          cuda_ok(cudaMemcpyAsync(all.data(), dbuf + sizeof(mine), sizeof(mine) * (size_t)n, cudaMemcpyDeviceToHost, xs),
                  "cudaMemcpyAsync") &&
          cuda_ok(cudaEventRecord(done, xs), "cudaEventRecord")) {
        // a rank of the parent that never makes this call must not hang the others for ever
        const auto deadline = Clock::now() + std::chrono::milliseconds(c->timeout_ms > 0 ? c->timeout_ms : 60000);
        while (true) {
          cudaError_t q = cudaEventQuery(done);
          if (q == cudaSuccess) break;
          if (q != cudaErrorNotReady) {
            cuda_ok(q, "cudaEventQuery");
            break;
          }
          if (Clock::now() > deadline) {
            rc = set_error(RAFB200_TIMEOUT, "rafb200_comm_sub: not every rank joined within %d ms", c->timeout_ms);
            break;
          }
          std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
      }
    }
    if (rc != RAFB200_TIMEOUT) {  // after a timeout the copy may still be pending: leak rather than fault
      if (done) cudaEventDestroy(done);
      if (xs) cudaStreamDestroy(xs);
      if (dbuf) cudaFree(dbuf);
    }
    if (rc == RAFB200_OK && needs_nccl) {
      const int* grp = ranks;
      for (int g = 0; g < my_group; ++g) grp += group_sizes[g];
      s->is_void = false;
      rc = init_rank(s, all[(size_t)grp[0]], c->timeout_ms);
    }
    if (rc != RAFB200_OK) {
      delete s;
      return rc;
    }
  }
  c->subs[key] = s;
  *sub = s;
  return RAFB200_OK;
}

// ---- DistConfig (include/raf/dist_config.h:17-48): one process-wide object ----------
static rafb200_dist_config g_dist_config = {0, 0, 0, 0, 0, 2, 4, 5000000000ll};

int rafb200_dist_config_get(rafb200_dist_config* out) {
  RAFB200_REQUIRE(out, "rafb200_dist_config_get: NULL argument");
  *out = g_dist_config;
  return RAFB200_OK;
}

int rafb200_dist_config_set(const rafb200_dist_config* in) {
  RAFB200_REQUIRE(in, "rafb200_dist_config_set: NULL argument");
  RAFB200_REQUIRE(in->zero_opt_level >= 0 && in->zero_opt_level <= 3, "rafb200_dist_config_set: zero_opt_level %d",
                  in->zero_opt_level);
  RAFB200_REQUIRE(in->group_bucket_size > 0, "rafb200_dist_config_set: group_bucket_size must be positive");
  g_dist_config = *in;
  return RAFB200_OK;
}

// ---- streams by tag (src/impl/stream_pool.cc:53-98) ---------------------------------
namespace {
struct StreamKey {
  int device, tag, index;
  bool operator<(const StreamKey& o) const {
    return device != o.device ? device < o.device : tag != o.tag ? tag < o.tag : index < o.index;
  }
};
std::mutex g_stream_mu;
std::map<StreamKey, cudaStream_t> g_streams;
}  // namespace

int rafb200_stream_get(int device, int tag, int index, void** stream) {
  RAFB200_REQUIRE(stream && device >= 0 && tag >= 1 && tag <= 6 && index >= 0,
                  "rafb200_stream_get: bad arguments (tags are 1 .. 6)");
  std::lock_guard<std::mutex> lk(g_stream_mu);
  const StreamKey key{device, tag, index};
  auto it = g_streams.find(key);
  if (it == g_streams.end()) {
    int prev = 0;
    RAFB200_CUDA(cudaGetDevice(&prev));
    RAFB200_CUDA(cudaSetDevice(device));
    cudaStream_t s = nullptr;
    cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    cudaSetDevice(prev);
    if (e != cudaSuccess) return set_error(RAFB200_CUDA_ERROR, "cudaStreamCreate: %s", cudaGetErrorString(e));
    it = g_streams.emplace(key, s).first;
  }
  *stream = it->second;
  return RAFB200_OK;
}

int rafb200_stream_release_all(void) {
  std::lock_guard<std::mutex> lk(g_stream_mu);
  for (auto& kv : g_streams) cudaStreamDestroy(kv.second);
  g_streams.clear();
  return RAFB200_OK;
}

int rafb200_comm_size(rafb200_comm_t c) { return c ? c->size : 0; }
int rafb200_comm_rank(rafb200_comm_t c) { return c ? c->rank : -1; }

int rafb200_comm_check(rafb200_comm_t c) {
  RAFB200_REQUIRE(c, "rafb200_comm_check: NULL communicator");
  if (c->is_void) return RAFB200_OK;
  ncclResult_t st = ncclSuccess;
  ncclResult_t r = ncclCommGetAsyncError(c->nccl, &st);
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommGetAsyncError");
  if (st != ncclSuccess) return nccl_fail(st, "asynchronous NCCL error");
  return RAFB200_OK;
}

static int local_copy(const void* src, void* dst, size_t bytes, cudaStream_t s) {
  if (src != dst && bytes)
    RAFB200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s));
  return RAFB200_OK;
}

int rafb200_allreduce(rafb200_comm_t c, const void* sendbuf, void* recvbuf, int64_t count,
                      int dtype, const char* computation, void* stream) {
  RAFB200_REQUIRE(c && count >= 0, "rafb200_allreduce: bad arguments");
  ncclDataType_t dt = ncclFloat32;
  ncclRedOp_t op = ncclSum;
  int rc = to_nccl_dtype(dtype, &dt);
  if (rc == RAFB200_OK) rc = to_nccl_op(computation, &op);
  if (rc != RAFB200_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (c->is_void) return local_copy(sendbuf, recvbuf, (size_t)count * comm_dtype_size(dtype), s);
  RAFB200_NCCL(c, ncclAllReduce(sendbuf, recvbuf, (size_t)count, dt, op, c->nccl, s));
  return RAFB200_OK;
}

int rafb200_group_reduce_scatter(rafb200_comm_t c, int k, const void* const* sendbuf,
                                 void* const* recvbuf, const int64_t* recvcount, int dtype,
                                 const char* computation, void* stream) {
  RAFB200_REQUIRE(c && k >= 0 && (k == 0 || (sendbuf && recvbuf && recvcount)),
                  "rafb200_group_reduce_scatter: bad arguments");
  ncclDataType_t dt = ncclFloat32;
  ncclRedOp_t op = ncclSum;
  int rc = to_nccl_dtype(dtype, &dt);
  if (rc == RAFB200_OK) rc = to_nccl_op(computation, &op);
  if (rc != RAFB200_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (c->is_void) {
    for (int i = 0; i < k; ++i) {
      rc = local_copy(sendbuf[i], recvbuf[i], (size_t)recvcount[i] * comm_dtype_size(dtype), s);
      if (rc != RAFB200_OK) return rc;
    }
    return RAFB200_OK;
  }
  if (k == 0) return RAFB200_OK;
  RAFB200_NCCL(c, ncclGroupStart());
  for (int i = 0; i < k; ++i) {
    ncclResult_t r = ncclReduceScatter(sendbuf[i], recvbuf[i], (size_t)recvcount[i], dt, op, c->nccl, s);
    if (r != ncclSuccess && r != ncclInProgress) {
      ncclGroupEnd();
      return nccl_fail(r, "ncclReduceScatter");
    }
  }
  RAFB200_NCCL(c, ncclGroupEnd());
  return RAFB200_OK;
}

int rafb200_reduce_scatter(rafb200_comm_t c, const void* sendbuf, void* recvbuf,
                           int64_t recvcount, int dtype, const char* computation, void* stream) {
  return rafb200_group_reduce_scatter(c, 1, &sendbuf, &recvbuf, &recvcount, dtype, computation,
                                      stream);
}

int rafb200_group_allgather(rafb200_comm_t c, int k, const void* const* sendbuf,
                            void* const* recvbuf, const int64_t* sendcount, int dtype,
                            void* stream) {
  RAFB200_REQUIRE(c && k >= 0 && (k == 0 || (sendbuf && recvbuf && sendcount)),
                  "rafb200_group_allgather: bad arguments");
  ncclDataType_t dt = ncclFloat32;
  int rc = to_nccl_dtype(dtype, &dt);
  if (rc != RAFB200_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (c->is_void) {
    for (int i = 0; i < k; ++i) {
      rc = local_copy(sendbuf[i], recvbuf[i], (size_t)sendcount[i] * comm_dtype_size(dtype), s);
      if (rc != RAFB200_OK) return rc;
    }
    return RAFB200_OK;
  }
  if (k == 0) return RAFB200_OK;
  RAFB200_NCCL(c, ncclGroupStart());
  for (int i = 0; i < k; ++i) {
    ncclResult_t r = ncclAllGather(sendbuf[i], recvbuf[i], (size_t)sendcount[i], dt, c->nccl, s);
    if (r != ncclSuccess && r != ncclInProgress) {
      ncclGroupEnd();
      return nccl_fail(r, "ncclAllGather");
    }
  }
  RAFB200_NCCL(c, ncclGroupEnd());
  return RAFB200_OK;
}

int rafb200_allgather(rafb200_comm_t c, const void* sendbuf, void* recvbuf, int64_t sendcount,
                      int dtype, void* stream) {
  return rafb200_group_allgather(c, 1, &sendbuf, &recvbuf, &sendcount, dtype, stream);
}

}  // extern "C"
