// ZeRO plan (shard geometry, buckets) and the step driver.  Per bucket:
//   pack (gradient row blocks -> rank-major flat buffer)  ->  ONE reduce-scatter
//   -> shard-local update (writes the parameter copy into the flat gather buffer)
//   -> ONE all-gather  ->  unpack (row blocks -> the caller's parameter tensors).
// Collectives run on the communication stream, kernels on the compute stream.
#include <algorithm>
#include <cstring>
#include <memory>

#include "common.h"
#include "symm.h"
#include "vec_io.cuh"

struct rafb200_plan_s {
  int k = 0, n = 1, rank = 0;
  int64_t bucket_elems = 0;
  std::vector<int64_t> dim0, row_elems, shard_rows, shard_elems, padded_elems, numel;
  std::vector<int> bucket_of;
  int nbuckets = 0;
  int64_t total = 0, total_padded = 0, total_shard = 0;
};

namespace rafb200 {

// One contiguous run of bytes moved by the pack / unpack kernel.
struct Seg {
  const char* src;
  char* dst;
  int64_t bytes;
  int64_t pad_;
};
constexpr int kSegChunkBytes = 32768;  // bytes per work item of the copy kernel

struct Bucket {
  std::vector<int> tensors;
  rafb200_tensor_list_t list = nullptr;
  void* lans_ws = nullptr;
  size_t lans_ws_bytes = 0;
  cudaEvent_t packed = nullptr, rs_done = nullptr, upd_done = nullptr, ag_done = nullptr;
  cudaEvent_t h2d_done = nullptr, out_ready = nullptr;  // host-buffer form of the step
  // n > 1: rank-major flat buffers.  Slot r of a buffer holds, for every tensor of the
  // bucket in order, row block r of that tensor at element offset `off[j]` (each offset a
  // multiple of 8 elements, so every block starts 16-byte aligned in either dtype).
  int64_t slot_elems = 0;          // elements per rank slot (sum of aligned shard sizes)
  std::vector<int64_t> off;        // element offset of tensor j inside a slot
  char* g_flat = nullptr;          // n * slot_elems gradients (reduce-scatter in place)
  char* p_flat = nullptr;          // n * slot_elems parameter copies (all-gather in place)
  Seg* dev_pack = nullptr;         // n * tensors segments each
  Seg* dev_unpack = nullptr;
  Item* dev_pack_items = nullptr;  // (segment, chunk) work items
  Item* dev_unpack_items = nullptr;
  uint32_t n_pack_items = 0, n_unpack_items = 0;
  // Symmetric mode lays a bucket out tensor-major instead: tensor j owns n row blocks of
  // align8(shard elements) each, starting n * off[j] elements into the bucket, i.e. the
  // padded tensor in its natural layout whenever its shard size is a multiple of 8
  // elements.  The collectives then work on one segment per tensor (this rank's block).
  int64_t base_elems = 0;          // first element of the bucket inside the flat buffers
  SymmSeg* dev_rs_segs = nullptr;
  SymmSeg* dev_ag_segs = nullptr;
  Item* dev_rs_items = nullptr;
  Item* dev_ag_items = nullptr;
  uint32_t n_rs_items = 0, n_ag_items = 0;
};

// Copies every segment; 16-byte accesses when both ends of a segment are aligned,
// element-sized (2 or 4 byte) accesses otherwise.
__global__ void __launch_bounds__(kBlockThreads)
    seg_copy_kernel(const Seg* __restrict__ segs, const Item* __restrict__ items, uint32_t nitems,
                    int elem_size) {
  Policies pol;
  pol.init();
  for (uint32_t it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item item = items[it];
    const Seg sg = segs[item.tensor_phase];
    const int64_t begin = (int64_t)item.chunk * kSegChunkBytes;
    int64_t n = sg.bytes - begin;
    if (n > kSegChunkBytes) n = kSegChunkBytes;
    const char* src = sg.src + begin;
    char* dst = sg.dst + begin;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
      const int nv = (int)(n >> 4);
      constexpr int kU = kSegChunkBytes / 16 / kBlockThreads;  // 8 vectors per thread
      uint4 r[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int i = threadIdx.x + u * kBlockThreads;
        if (i < nv) r[u] = ld16<kStream>(src + (size_t)i * 16, pol);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int i = threadIdx.x + u * kBlockThreads;
        if (i < nv) st16<kDefault>(dst + (size_t)i * 16, r[u], pol);
      }
      for (int64_t e = ((int64_t)nv << 4) + threadIdx.x; e < n; e += kBlockThreads) dst[e] = src[e];
    } else if (elem_size == 4) {
      for (int64_t e = threadIdx.x; e < (n >> 2); e += kBlockThreads)
        reinterpret_cast<uint32_t*>(dst)[e] = reinterpret_cast<const uint32_t*>(src)[e];
    } else {
      for (int64_t e = threadIdx.x; e < (n >> 1); e += kBlockThreads)
        reinterpret_cast<uint16_t*>(dst)[e] = reinterpret_cast<const uint16_t*>(src)[e];
    }
  }
}

static int launch_seg_copy(const Seg* segs, const Item* items, uint32_t nitems, int elem_size,
                           int sm_count, cudaStream_t s) {
  if (nitems == 0) return RAFB200_OK;
  int64_t grid = (int64_t)sm_count * 8;
  if (grid > (int64_t)nitems) grid = nitems;
  seg_copy_kernel<<<(unsigned)grid, kBlockThreads, 0, s>>>(segs, items, nitems, elem_size);
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

static int upload(const void* host, size_t bytes, void** dev) {
  if (*dev) {
    cudaFree(*dev);
    *dev = nullptr;
  }
  if (bytes == 0) return RAFB200_OK;
  RAFB200_CUDA(cudaMalloc(dev, bytes));
  RAFB200_CUDA(cudaMemcpy(*dev, host, bytes, cudaMemcpyHostToDevice));
  return RAFB200_OK;
}

static std::vector<Item> seg_items(const std::vector<Seg>& segs) {
  std::vector<Item> items;
  for (size_t i = 0; i < segs.size(); ++i) {
    const int64_t chunks = (segs[i].bytes + kSegChunkBytes - 1) / kSegChunkBytes;
    for (int64_t c = 0; c < chunks; ++c) items.push_back(Item{(uint32_t)i, (uint32_t)c});
  }
  return items;
}

}  // namespace rafb200

struct rafb200_zero_s {
  rafb200_plan_s plan;
  rafb200_comm_t comm = nullptr;
  int n = 1, rank = 0;
  int g_dtype = 0, param_dtype = 0, optimizer = 0;
  std::vector<rafb200::Bucket> buckets;
  // world of one, host-buffer form: one list per plan bucket so that the copy of bucket b+1
  // from the host, the update of bucket b and the copy of bucket b-1 to the host overlap
  std::vector<rafb200::Bucket> hbuckets;
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  cudaEvent_t ev_d2h_done = nullptr;
  char* g_flat = nullptr;  // all buckets' gradient buffers, one allocation (n > 1)
  char* p_flat = nullptr;  // all buckets' parameter-copy buffers
  int sm_count = 148;
  int64_t flat_elems = 0;  // elements of each flat buffer (all buckets, all slots)
  std::vector<void*> grads, params;
  std::vector<float*> p, m, v;
  bool bound = false;
  cudaEvent_t ev_start = nullptr, ev_done = nullptr;
  int max_update_blocks = 0;
  int stage_mask = 31;  // measurement aid: which of the five stages a step issues
  // symmetric-memory mode (rafb200_zero_attach_symmetric): the flat buffers live in memory
  // every rank has mapped; the collectives are this library's own kernels, not NCCL's
  bool symmetric = false;
  rafb200::SymmPeers g_peers{}, p_peers{}, sig_peers{};
  void* g_mc = nullptr;
  void* p_mc = nullptr;
  char* g_red = nullptr;             // this rank's reduced gradient blocks (plain local memory)
  unsigned int* dev_err = nullptr;   // first expired cross-GPU wait, 0 if none
  // The same word as the host sees it without synchronising: pinned, mapped memory that the
  // barrier kernel stores to when it gives up, read at the top of every step.
  volatile unsigned int* host_err = nullptr;
  unsigned int* host_err_dev = nullptr;  // device address of *host_err
  int device = 0;                        // the device current at creation
  uint64_t wait_limit_ns = 10000000000ull;
  int host_output = 0;               // 0: full parameters to the host, 1: this rank's row blocks
  std::vector<const void*> shard_g;  // per tensor: where the update reads its gradient block
  // ranges the caller declared to be single allocations: copies may be merged inside them
  std::vector<std::pair<const char*, size_t>> arenas;
  bool in_one_arena(const void* lo, const void* hi) const {  // [lo, hi) inside one declared range
    for (const auto& a : arenas)
      if (static_cast<const char*>(lo) >= a.first && static_cast<const char*>(hi) <= a.first + a.second) return true;
    return false;
  }
  uint32_t epoch[2] = {0, 0};        // barrier lanes: 0 before reduce-scatter, 1 after all-gather
  cudaStream_t gather_stream = nullptr;
  cudaEvent_t ev_gather = nullptr;
  int comm_blocks = 128;
  int kernels_per_step = 0, collectives_per_step = 0;
  // The collectives inside the update kernel (rafb200_zero_set_fused): one list over
  // all tensors, one launch per step, two cross-GPU barriers per step instead of two per bucket
  int fused = 0;  // 0 off, 1 reduce-scatter inside the kernel, 2 all-gather too, 3 = 2 with peer stores
  rafb200_tensor_list_t fused_list = nullptr;
  void* fused_ws = nullptr;
  size_t fused_ws_bytes = 0;
};

using namespace rafb200;

extern "C" {

int rafb200_plan_create(int k, const int64_t* dim0, const int64_t* row_elems, int n_ranks,
                        int rank, int64_t bucket_elems, rafb200_plan_t* plan) {
  RAFB200_REQUIRE(plan, "rafb200_plan_create: NULL result pointer");
  *plan = nullptr;
  RAFB200_REQUIRE(k >= 0 && (k == 0 || (dim0 && row_elems)), "rafb200_plan_create: bad tensor table");
  RAFB200_REQUIRE(n_ranks >= 1 && rank >= 0 && rank < n_ranks,
                  "rafb200_plan_create: rank %d outside %d partitions", rank, n_ranks);
  auto pl = std::make_unique<rafb200_plan_s>();
  pl->k = k;
  pl->n = n_ranks;
  pl->rank = rank;
  pl->bucket_elems = bucket_elems;
  pl->dim0.assign(dim0, dim0 + k);
  pl->row_elems.assign(row_elems, row_elems + k);
  pl->shard_rows.resize(k);
  pl->shard_elems.resize(k);
  pl->padded_elems.resize(k);
  pl->numel.resize(k);
  pl->bucket_of.resize(k);
  int b = 0, open = 0;
  int64_t curr = 0;
  for (int i = 0; i < k; ++i) {
    RAFB200_REQUIRE(dim0[i] >= 0 && row_elems[i] >= 0, "rafb200_plan_create: negative shape, tensor %d", i);
    // partition_gradient.cc:191-197: d0/n + 1 rows per part when d0 % n != 0
    const int64_t rows = (dim0[i] % n_ranks == 0) ? dim0[i] / n_ranks : dim0[i] / n_ranks + 1;
    pl->shard_rows[i] = rows;
    pl->shard_elems[i] = rows * row_elems[i];
    pl->padded_elems[i] = rows * n_ranks * row_elems[i];
    pl->numel[i] = dim0[i] * row_elems[i];
    pl->total += pl->numel[i];
    pl->total_padded += pl->padded_elems[i];
    pl->total_shard += pl->shard_elems[i];
    // partition_gradient.cc:289-300 / group_allgather.cc:110-145: join while curr + size < bucket
    if (curr + pl->numel[i] < bucket_elems) {
      curr += pl->numel[i];
      open++;
    } else {
      if (open > 0) b++;
      curr = pl->numel[i];
      open = 1;
    }
    pl->bucket_of[i] = b;
  }
  pl->nbuckets = k > 0 ? b + 1 : 0;
  *plan = pl.release();
  return RAFB200_OK;
}

int rafb200_plan_destroy(rafb200_plan_t plan) {
  delete plan;
  return RAFB200_OK;
}

int rafb200_plan_num_buckets(rafb200_plan_t plan) { return plan ? plan->nbuckets : 0; }

int rafb200_plan_query(rafb200_plan_t plan, int64_t* shard_rows, int64_t* shard_elems,
                       int64_t* padded_elems, int* bucket_of) {
  RAFB200_REQUIRE(plan, "rafb200_plan_query: NULL plan");
  for (int i = 0; i < plan->k; ++i) {
    if (shard_rows) shard_rows[i] = plan->shard_rows[i];
    if (shard_elems) shard_elems[i] = plan->shard_elems[i];
    if (padded_elems) padded_elems[i] = plan->padded_elems[i];
    if (bucket_of) bucket_of[i] = plan->bucket_of[i];
  }
  return RAFB200_OK;
}

int rafb200_plan_totals(rafb200_plan_t plan, int64_t* elems, int64_t* padded_elems,
                        int64_t* shard_elems) {
  RAFB200_REQUIRE(plan, "rafb200_plan_totals: NULL plan");
  if (elems) *elems = plan->total;
  if (padded_elems) *padded_elems = plan->total_padded;
  if (shard_elems) *shard_elems = plan->total_shard;
  return RAFB200_OK;
}

// ---- step driver ----------------------------------------------------------------

int rafb200_zero_destroy(rafb200_zero_t z) {
  if (!z) return RAFB200_OK;
  if (z->fused_list) rafb200_tensor_list_destroy(z->fused_list);
  if (z->fused_ws) cudaFree(z->fused_ws);
  for (auto* set : {&z->buckets, &z->hbuckets})
   for (auto& b : *set) {
    if (b.list) rafb200_tensor_list_destroy(b.list);
    if (b.lans_ws) cudaFree(b.lans_ws);
    for (cudaEvent_t e : {b.packed, b.rs_done, b.upd_done, b.ag_done, b.h2d_done, b.out_ready})
      if (e) cudaEventDestroy(e);
    for (void* ptr : {(void*)b.dev_pack, (void*)b.dev_unpack, (void*)b.dev_pack_items,
                      (void*)b.dev_unpack_items, (void*)b.dev_rs_segs, (void*)b.dev_ag_segs,
                      (void*)b.dev_rs_items, (void*)b.dev_ag_items})
      if (ptr) cudaFree(ptr);
  }
  if (z->g_flat && !z->symmetric) rafb200_comm_free(z->comm, z->g_flat);
  if (z->p_flat && !z->symmetric) rafb200_comm_free(z->comm, z->p_flat);
  if (z->dev_err) cudaFree(z->dev_err);
  if (z->host_err) cudaFreeHost(const_cast<unsigned int*>(z->host_err));
  if (z->g_red) cudaFree(z->g_red);
  if (z->gather_stream) cudaStreamDestroy(z->gather_stream);
  if (z->ev_gather) cudaEventDestroy(z->ev_gather);
  if (z->ev_start) cudaEventDestroy(z->ev_start);
  if (z->ev_done) cudaEventDestroy(z->ev_done);
  if (z->ev_d2h_done) cudaEventDestroy(z->ev_d2h_done);
  if (z->h2d_stream) cudaStreamDestroy(z->h2d_stream);
  if (z->d2h_stream) cudaStreamDestroy(z->d2h_stream);
  delete z;
  return RAFB200_OK;
}

int rafb200_zero_create(rafb200_plan_t plan, rafb200_comm_t comm, int g_dtype, int param_dtype,
                        int optimizer, rafb200_zero_t* zero) {
  RAFB200_REQUIRE(zero, "rafb200_zero_create: NULL result pointer");
  *zero = nullptr;
  RAFB200_REQUIRE(plan && comm, "rafb200_zero_create: NULL plan or communicator");
  RAFB200_REQUIRE(dtype_valid(g_dtype) && dtype_valid(param_dtype), "rafb200_zero_create: bad dtype");
  RAFB200_REQUIRE(optimizer >= RAFB200_OPT_SGD && optimizer <= RAFB200_OPT_LANS,
                  "rafb200_zero_create: unknown optimizer %d", optimizer);
  RAFB200_REQUIRE(plan->n == rafb200_comm_size(comm) && plan->rank == rafb200_comm_rank(comm),
                  "rafb200_zero_create: plan is for rank %d of %d, communicator is rank %d of %d",
                  plan->rank, plan->n, rafb200_comm_rank(comm), rafb200_comm_size(comm));
  auto* z = new rafb200_zero_s();
  z->plan = *plan;
  z->comm = comm;
  z->n = plan->n;
  z->rank = plan->rank;
  z->g_dtype = g_dtype;
  z->param_dtype = param_dtype;
  z->optimizer = optimizer;
  const int k = plan->k;
  int rc = RAFB200_OK;
  do {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&z->sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: no usable CUDA device");
      break;
    }
    z->device = dev;
    // With a single rank there is nothing to overlap: one bucket, one launch.
    const int nb = (z->n == 1) ? (k > 0 ? 1 : 0) : plan->nbuckets;
    z->buckets.resize(nb);
    for (int i = 0; i < k; ++i) z->buckets[z->n == 1 ? 0 : plan->bucket_of[i]].tensors.push_back(i);
    if (z->n == 1 && k > 1) {
      // Host-buffer form on one rank: groups of about 16 Mi elements (32-64 MB over PCIe, a
      // few ms each way), small enough that the first copy in and the last copy out, which
      // nothing overlaps, stay short.
      constexpr int64_t kHostGroupElems = 16ll << 20;
      int64_t run = 0;
      for (int i = 0; i < k; ++i) {
        if (z->hbuckets.empty() || (run > 0 && run + plan->numel[i] > kHostGroupElems)) {
          z->hbuckets.emplace_back();
          run = 0;
        }
        z->hbuckets.back().tensors.push_back(i);
        run += plan->numel[i];
      }
      if (z->hbuckets.size() < 2) z->hbuckets.clear();
    }
    int64_t flat_elems = 0;
    for (auto* set : {&z->buckets, &z->hbuckets}) {
      for (auto& b : *set) {
        std::vector<int64_t> numel;
        for (int i : b.tensors) {
          numel.push_back(plan->shard_elems[i]);
          b.off.push_back(b.slot_elems);
          b.slot_elems += (plan->shard_elems[i] + 7) & ~(int64_t)7;
        }
        if (set == &z->buckets) flat_elems += b.slot_elems * z->n;
        rc = rafb200_tensor_list_create((int)numel.size(), numel.data(), g_dtype, param_dtype, &b.list);
        if (rc != RAFB200_OK) break;
        if (optimizer == RAFB200_OPT_LANS) {
          b.lans_ws_bytes = rafb200_lans_workspace_bytes(b.list);
          if (cudaMalloc(&b.lans_ws, b.lans_ws_bytes) != cudaSuccess) {
            rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot allocate LANS workspace");
            break;
          }
        }
        for (cudaEvent_t* e : {&b.packed, &b.rs_done, &b.upd_done, &b.ag_done, &b.h2d_done, &b.out_ready})
          if (cudaEventCreateWithFlags(e, cudaEventDisableTiming) != cudaSuccess)
            rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot create events");
        if (rc != RAFB200_OK) break;
      }
      if (rc != RAFB200_OK) break;
    }
    if (rc != RAFB200_OK) break;
    if (cudaStreamCreateWithFlags(&z->h2d_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&z->d2h_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&z->ev_d2h_done, cudaEventDisableTiming) != cudaSuccess) {
      rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot create copy streams");
      break;
    }
    if (rc != RAFB200_OK) break;
    if (cudaEventCreateWithFlags(&z->ev_start, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&z->ev_done, cudaEventDisableTiming) != cudaSuccess) {
      rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot create events");
      break;
    }
    z->flat_elems = flat_elems;
    if (z->n > 1 && flat_elems > 0) {
      const size_t gbytes = (size_t)flat_elems * dtype_size(g_dtype);
      const size_t pbytes = (size_t)flat_elems * dtype_size(param_dtype);
      if ((rc = rafb200_comm_alloc(comm, gbytes, reinterpret_cast<void**>(&z->g_flat))) != RAFB200_OK ||
          (rc = rafb200_comm_alloc(comm, pbytes, reinterpret_cast<void**>(&z->p_flat))) != RAFB200_OK)
        break;
      // Zeroed once: the pack kernel never writes the padding rows or the alignment
      // gaps, and a reduce-scatter only ever adds zeros to them.
      if (cudaMemset(z->g_flat, 0, gbytes) != cudaSuccess || cudaMemset(z->p_flat, 0, pbytes) != cudaSuccess) {
        rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot clear the bucket buffers");
        break;
      }
      int64_t at = 0;
      for (auto& b : z->buckets) {
        b.base_elems = at;
        b.g_flat = z->g_flat + (size_t)at * dtype_size(g_dtype);
        b.p_flat = z->p_flat + (size_t)at * dtype_size(param_dtype);
        at += b.slot_elems * z->n;
      }
    }
  } while (false);
  if (rc != RAFB200_OK) {
    rafb200_zero_destroy(z);
    return rc;
  }
  *zero = z;
  return RAFB200_OK;
}

int rafb200_zero_bind(rafb200_zero_t z, void* const* grads, void* const* params, float* const* p,
                      float* const* m, float* const* v) {
  RAFB200_REQUIRE(z, "rafb200_zero_bind: NULL state");
  const int k = z->plan.k;
  RAFB200_REQUIRE(k == 0 || (grads && params && p && m), "rafb200_zero_bind: NULL pointer table");
  RAFB200_REQUIRE(z->optimizer == RAFB200_OPT_SGD || v, "rafb200_zero_bind: v is required");
  const bool same = z->bound && std::equal(grads, grads + k, z->grads.begin()) &&
                    std::equal(params, params + k, z->params.begin()) &&
                    std::equal(p, p + k, z->p.begin()) && std::equal(m, m + k, z->m.begin()) &&
                    (v ? (z->v.size() == (size_t)k && std::equal(v, v + k, z->v.begin())) : z->v.empty());
  if (same) return RAFB200_OK;
  z->grads.assign(grads, grads + k);
  z->params.assign(params, params + k);
  z->p.assign(p, p + k);
  z->m.assign(m, m + k);
  if (v) z->v.assign(v, v + k);
  else z->v.clear();
  const int gs = dtype_size(z->g_dtype), ps = dtype_size(z->param_dtype);
  z->kernels_per_step = 0;
  z->collectives_per_step = 0;
  // Tables that a kernel of an earlier step may still be reading are replaced below.
  RAFB200_CUDA(cudaDeviceSynchronize());
  // for the one-launch form (z->fused): every tensor's reduced-gradient block, its block of
  // the local parameter buffer and its byte offset inside the symmetric gradient buffer
  std::vector<const void*> fused_g((size_t)k, nullptr);
  std::vector<void*> fused_out((size_t)k, nullptr);
  std::vector<int64_t> fused_off((size_t)k, 0);
  for (auto* set : {&z->buckets, &z->hbuckets})
   for (auto& b : *set) {
    const bool counted = (set == &z->buckets);
    const size_t nt = b.tensors.size();
    std::vector<const void*> lg(nt);
    std::vector<float*> lp(nt), lm(nt), lv(nt);
    std::vector<void*> lo(nt);
    std::vector<Seg> pack, unpack;
    std::vector<SymmSeg> rs_segs, ag_segs;
    for (size_t j = 0; j < nt; ++j) {
      const int i = b.tensors[j];
      const int64_t se = z->plan.shard_elems[i];
      RAFB200_REQUIRE(se == 0 || (grads[i] && params[i] && p[i] && m[i]),
                      "rafb200_zero_bind: NULL buffer for tensor %d", i);
      lp[j] = p[i];
      lm[j] = m[i];
      lv[j] = v ? v[i] : nullptr;
      if (z->n == 1) {
        lg[j] = grads[i];
        // An fp32 model whose parameter IS the master copy (python/raf/optim/lans.py:218,
        // `weight = param`) gets no second write.
        lo[j] = (params[i] == static_cast<void*>(p[i])) ? nullptr : params[i];
        continue;
      }
      // This rank updates its own row block inside the flat buffers, in place.
      const int64_t bs = (se + 7) & ~(int64_t)7;  // block stride of the tensor-major layout
      const bool tm = z->symmetric;
      auto block = [&](int r) -> size_t {          // element offset of row block r of tensor j
        return tm ? (size_t)(z->n * b.off[j] + r * bs) : (size_t)(r * b.slot_elems + b.off[j]);
      };
      lg[j] = b.g_flat + block(z->rank) * gs;
      lo[j] = b.p_flat + block(z->rank) * ps;
      if (tm) {
        // The sum goes to a buffer of its own: the gradients in the symmetric buffer (which
        // may be the caller's tensors themselves) are inputs only.
        const size_t red = (size_t)(b.base_elems / z->n + b.off[j]) * gs;
        lg[j] = z->g_red + red;
        rs_segs.push_back(SymmSeg{(size_t)(b.g_flat - z->g_flat) + block(z->rank) * gs, red, bs * gs});
        if (counted) {
          fused_g[(size_t)i] = lg[j];
          fused_out[(size_t)i] = lo[j];
          fused_off[(size_t)i] = (int64_t)rs_segs.back().off;
        }
        ag_segs.push_back(SymmSeg{(size_t)(b.p_flat - z->p_flat) + block(z->rank) * ps, 0, bs * ps});
      }
      // A caller tensor that IS the tensor's region of the flat buffer needs no copy.
      const bool g_view = tm && bs == se && grads[i] == b.g_flat + block(0) * gs;
      const bool p_view = tm && bs == se && params[i] == b.p_flat + block(0) * ps;
      if (tm && bs == se) {  // natural layout: one contiguous copy per tensor
        if (!g_view && z->plan.numel[i] > 0)
          pack.push_back(Seg{static_cast<const char*>(grads[i]), b.g_flat + block(0) * gs,
                             z->plan.numel[i] * gs, 0});
        if (!p_view && z->plan.numel[i] > 0)
          unpack.push_back(Seg{b.p_flat + block(0) * ps, static_cast<char*>(params[i]),
                               z->plan.numel[i] * ps, 0});
        continue;
      }
      for (int r = 0; r < z->n; ++r) {
        // rows of block r that exist in the unpadded tensor (raf.op.pad / strided_slice)
        int64_t cnt = z->plan.numel[i] - (int64_t)r * se;
        cnt = cnt < 0 ? 0 : (cnt > se ? se : cnt);
        if (cnt == 0) continue;
        pack.push_back(Seg{static_cast<const char*>(grads[i]) + (size_t)r * se * gs,
                           b.g_flat + block(r) * gs, cnt * gs, 0});
        unpack.push_back(Seg{b.p_flat + block(r) * ps, static_cast<char*>(params[i]) + (size_t)r * se * ps,
                             cnt * ps, 0});
      }
    }
    if (counted) {
      z->shard_g.resize(k);
      for (size_t j = 0; j < nt; ++j) z->shard_g[b.tensors[j]] = lg[j];
    }
    int rc = rafb200_tensor_list_bind(b.list, lg.data(), lp.data(), lm.data(), v ? lv.data() : nullptr,
                                      lo.data(), nullptr);
    if (rc != RAFB200_OK) return rc;
    if (counted && rafb200_tensor_list_total_elems(b.list) > 0) z->kernels_per_step += 1;
    if (z->n > 1) {
      const std::vector<Item> pi = seg_items(pack), ui = seg_items(unpack);
      b.n_pack_items = (uint32_t)pi.size();
      b.n_unpack_items = (uint32_t)ui.size();
      if ((rc = upload(pack.data(), pack.size() * sizeof(Seg), reinterpret_cast<void**>(&b.dev_pack))) ||
          (rc = upload(unpack.data(), unpack.size() * sizeof(Seg), reinterpret_cast<void**>(&b.dev_unpack))) ||
          (rc = upload(pi.data(), pi.size() * sizeof(Item), reinterpret_cast<void**>(&b.dev_pack_items))) ||
          (rc = upload(ui.data(), ui.size() * sizeof(Item), reinterpret_cast<void**>(&b.dev_unpack_items))))
        return rc;
      if (z->symmetric) {
        auto chunks = [](const std::vector<SymmSeg>& segs) {
          std::vector<Item> items;
          for (size_t si = 0; si < segs.size(); ++si)
            for (int64_t c = 0; c * kSymmChunkBytes < segs[si].bytes; ++c)
              items.push_back(Item{(uint32_t)si, (uint32_t)c});
          return items;
        };
        const std::vector<Item> ri = chunks(rs_segs), ai = chunks(ag_segs);
        b.n_rs_items = (uint32_t)ri.size();
        b.n_ag_items = (uint32_t)ai.size();
        if ((rc = upload(rs_segs.data(), rs_segs.size() * sizeof(SymmSeg), reinterpret_cast<void**>(&b.dev_rs_segs))) ||
            (rc = upload(ag_segs.data(), ag_segs.size() * sizeof(SymmSeg), reinterpret_cast<void**>(&b.dev_ag_segs))) ||
            (rc = upload(ri.data(), ri.size() * sizeof(Item), reinterpret_cast<void**>(&b.dev_rs_items))) ||
            (rc = upload(ai.data(), ai.size() * sizeof(Item), reinterpret_cast<void**>(&b.dev_ag_items))))
          return rc;
      }
      z->kernels_per_step += (b.n_pack_items > 0) + (b.n_unpack_items > 0);
      if (z->symmetric) z->kernels_per_step += (b.n_rs_items > 0) + (b.n_ag_items > 0) + 2;  // + 2 barriers
      else if (b.slot_elems > 0) z->collectives_per_step += 2;  // NCCL calls
    }
  }
  if (z->fused && z->symmetric) {
    if (!z->fused_list) {
      int rc = rafb200_tensor_list_create(k, z->plan.shard_elems.data(), z->g_dtype, z->param_dtype, &z->fused_list);
      if (rc != RAFB200_OK) return rc;
      if (z->optimizer == RAFB200_OPT_LANS) {
        z->fused_ws_bytes = rafb200_lans_workspace_bytes(z->fused_list);
        RAFB200_CUDA(cudaMalloc(&z->fused_ws, z->fused_ws_bytes));
      }
    }
    LansFuse f;
    f.world = z->n;
    f.rank = z->rank;
    f.fuse_rs = 1;
    f.fuse_ag = z->fused >= 2 ? 1 : 0;
    f.g_mc = static_cast<const char*>(z->g_mc);
    f.p_mc = z->fused == 3 ? nullptr : static_cast<char*>(z->p_mc);  // 3: the copies go out as peer stores
    for (int q = 0; q < z->n; ++q) {
      f.g_peer[q] = static_cast<const char*>(z->g_peers.ptr[q]);
      f.p_peer[q] = static_cast<char*>(z->p_peers.ptr[q]);
    }
    int rc = tensor_list_set_fuse(z->fused_list, f, fused_off.data());
    if (rc != RAFB200_OK) return rc;
    rc = rafb200_tensor_list_bind(z->fused_list, fused_g.data(), z->p.data(), z->m.data(),
                                  z->v.empty() ? nullptr : z->v.data(), fused_out.data(), nullptr);
    if (rc != RAFB200_OK) return rc;
    // what such a step launches: pack / unpack where needed, two barriers, one update, and the
    // all-gather kernels unless they are inside the update too
    z->kernels_per_step = 3;
    for (auto& b : z->buckets)
      z->kernels_per_step += (b.n_pack_items > 0) + (b.n_unpack_items > 0) + ((z->fused < 2 && b.n_ag_items > 0) ? 1 : 0);
  }
  RAFB200_CUDA(cudaStreamSynchronize(nullptr));  // descriptor tables are in place
  z->bound = true;
  return RAFB200_OK;
}

int rafb200_zero_set_fused(rafb200_zero_t z, int mode) {
  RAFB200_REQUIRE(z && mode >= 0 && mode <= 3, "rafb200_zero_set_fused: mode must be 0 .. 3");
  RAFB200_REQUIRE(mode == 0 || z->symmetric, "rafb200_zero_set_fused: attach symmetric memory first");
  RAFB200_REQUIRE(!z->bound, "rafb200_zero_set_fused: call before rafb200_zero_bind");
  z->fused = mode;
  return RAFB200_OK;
}

int rafb200_zero_flat_bytes(rafb200_zero_t z, size_t* g_bytes, size_t* p_bytes, size_t* signal_bytes) {
  RAFB200_REQUIRE(z, "rafb200_zero_flat_bytes: NULL state");
  const int64_t e = z->n > 1 ? z->flat_elems : 0;
  if (g_bytes) *g_bytes = (size_t)e * dtype_size(z->g_dtype);
  if (p_bytes) *p_bytes = (size_t)e * dtype_size(z->param_dtype);
  if (signal_bytes) *signal_bytes = kSymmSignalBytes;
  return RAFB200_OK;
}

int rafb200_zero_attach_symmetric(rafb200_zero_t z, void* const* g_peer, void* g_mc, void* const* p_peer,
                                  void* p_mc, void* const* signal_peer, int comm_blocks) {
  RAFB200_REQUIRE(z && g_peer && p_peer && signal_peer, "rafb200_zero_attach_symmetric: NULL argument");
  RAFB200_REQUIRE(z->n > 1, "rafb200_zero_attach_symmetric: a world of one has no collectives");
  RAFB200_REQUIRE(z->n <= kSymmMaxWorld, "rafb200_zero_attach_symmetric: at most %d ranks", kSymmMaxWorld);
  RAFB200_REQUIRE(!z->bound, "rafb200_zero_attach_symmetric: attach before rafb200_zero_bind");
  RAFB200_REQUIRE(!z->symmetric, "rafb200_zero_attach_symmetric: already attached");
  RAFB200_REQUIRE((g_mc == nullptr) == (p_mc == nullptr),
                  "rafb200_zero_attach_symmetric: give both multicast addresses or neither");
  for (int q = 0; q < z->n; ++q) {
    RAFB200_REQUIRE(g_peer[q] && p_peer[q] && signal_peer[q],
                    "rafb200_zero_attach_symmetric: NULL mapping of rank %d", q);
    RAFB200_REQUIRE(((reinterpret_cast<uintptr_t>(g_peer[q]) | reinterpret_cast<uintptr_t>(p_peer[q])) & 15u) == 0,
                    "rafb200_zero_attach_symmetric: buffers must be 16-byte aligned");
    z->g_peers.ptr[q] = g_peer[q];
    z->p_peers.ptr[q] = p_peer[q];
    z->sig_peers.ptr[q] = signal_peer[q];
  }
  RAFB200_CUDA(cudaMalloc(reinterpret_cast<void**>(&z->dev_err), 16));
  RAFB200_CUDA(cudaMalloc(reinterpret_cast<void**>(&z->g_red),
                          (size_t)(z->flat_elems / z->n + 8) * dtype_size(z->g_dtype)));
  RAFB200_CUDA(cudaMemset(z->dev_err, 0, 16));
  {
    void* h = nullptr;
    RAFB200_CUDA(cudaHostAlloc(&h, 64, cudaHostAllocMapped));
    memset(h, 0, 64);
    z->host_err = static_cast<volatile unsigned int*>(h);
    void* d = nullptr;
    RAFB200_CUDA(cudaHostGetDevicePointer(&d, h, 0));
    z->host_err_dev = static_cast<unsigned int*>(d);
  }
  RAFB200_CUDA(cudaStreamCreateWithFlags(&z->gather_stream, cudaStreamNonBlocking));
  RAFB200_CUDA(cudaEventCreateWithFlags(&z->ev_gather, cudaEventDisableTiming));
  // The NCCL-registered buffers of rafb200_zero_create are not needed in this mode.
  if (z->g_flat) rafb200_comm_free(z->comm, z->g_flat);
  if (z->p_flat) rafb200_comm_free(z->comm, z->p_flat);
  z->g_flat = static_cast<char*>(g_peer[z->rank]);
  z->p_flat = static_cast<char*>(p_peer[z->rank]);
  z->g_mc = g_mc;
  z->p_mc = p_mc;
  z->symmetric = true;
  // Plain peer loads need more requests in flight than switch-side reductions do.
  z->comm_blocks = comm_blocks > 0 ? comm_blocks : (g_mc ? 128 : 4 * z->sm_count);
  int64_t at = 0;
  for (auto& b : z->buckets) {
    b.base_elems = at;
    b.g_flat = z->g_flat + (size_t)at * dtype_size(z->g_dtype);
    b.p_flat = z->p_flat + (size_t)at * dtype_size(z->param_dtype);
    at += b.slot_elems * z->n;
  }
  return RAFB200_OK;
}

int rafb200_zero_arena_offsets(rafb200_zero_t z, int64_t* elem_offset, int* natural) {
  RAFB200_REQUIRE(z && z->symmetric, "rafb200_zero_arena_offsets: attach symmetric memory first");
  for (auto& b : z->buckets)
    for (size_t j = 0; j < b.tensors.size(); ++j) {
      const int i = b.tensors[j];
      const int64_t se = z->plan.shard_elems[i];
      if (elem_offset) elem_offset[i] = b.base_elems + z->n * b.off[j];
      if (natural) natural[i] = (((se + 7) & ~(int64_t)7) == se) ? 1 : 0;
    }
  return RAFB200_OK;
}

static int wait_expired(unsigned int e) {
  return set_error(RAFB200_DEVICE_WAIT_EXPIRED,
                   "rafb200_zero_step: rank %u did not reach barrier lane %u within the limit; the "
                   "ranks are out of step, destroy this state on every rank and create it again",
                   e & 15u, (e >> 4) & 15u);
}

int rafb200_zero_status(rafb200_zero_t z) {
  RAFB200_REQUIRE(z, "rafb200_zero_status: NULL state");
  RAFB200_CUDA(cudaDeviceSynchronize());
  if (!z->dev_err) return RAFB200_OK;
  unsigned int e = 0;
  RAFB200_CUDA(cudaMemcpy(&e, z->dev_err, sizeof(e), cudaMemcpyDeviceToHost));
  if (e != 0) return wait_expired(e);
  return RAFB200_OK;
}

int rafb200_zero_set_wait_limit(rafb200_zero_t z, int limit_ms) {
  RAFB200_REQUIRE(z && limit_ms > 0, "rafb200_zero_set_wait_limit: bad arguments");
  z->wait_limit_ns = (uint64_t)limit_ms * 1000000ull;
  return RAFB200_OK;
}

int rafb200_zero_set_host_output(rafb200_zero_t z, int mode) {
  RAFB200_REQUIRE(z && (mode == 0 || mode == 1), "rafb200_zero_set_host_output: mode must be 0 or 1");
  z->host_output = mode;
  return RAFB200_OK;
}

int rafb200_zero_declare_arena(rafb200_zero_t z, const void* base, size_t bytes) {
  RAFB200_REQUIRE(z && base && bytes > 0, "rafb200_zero_declare_arena: bad arguments");
  z->arenas.emplace_back(static_cast<const char*>(base), bytes);
  return RAFB200_OK;
}

int rafb200_zero_shard_grad(rafb200_zero_t z, int tensor, const void** ptr) {
  RAFB200_REQUIRE(z && ptr, "rafb200_zero_shard_grad: NULL argument");
  RAFB200_REQUIRE(z->bound, "rafb200_zero_shard_grad: bind buffers first");
  RAFB200_REQUIRE(tensor >= 0 && tensor < z->plan.k, "rafb200_zero_shard_grad: no tensor %d", tensor);
  *ptr = z->shard_g[tensor];
  return RAFB200_OK;
}

int rafb200_zero_set_update_blocks(rafb200_zero_t z, int max_blocks) {
  RAFB200_REQUIRE(z && max_blocks >= 0, "rafb200_zero_set_update_blocks: bad arguments");
  z->max_update_blocks = max_blocks;
  for (auto& b : z->buckets) {
    int rc = rafb200_tensor_list_tune(b.list, b.list->lead_elems, b.list->gap_items, max_blocks);
    if (rc != RAFB200_OK) return rc;
  }
  return RAFB200_OK;
}

int rafb200_zero_set_stage_mask(rafb200_zero_t z, int mask) {
  RAFB200_REQUIRE(z && mask >= 0 && mask < 32, "rafb200_zero_set_stage_mask: bad arguments");
  z->stage_mask = mask;
  return RAFB200_OK;
}

int rafb200_zero_launch_counts(rafb200_zero_t z, int* kernels, int* collectives) {
  RAFB200_REQUIRE(z, "rafb200_zero_launch_counts: NULL state");
  if (kernels) *kernels = z->kernels_per_step;
  if (collectives) *collectives = z->collectives_per_step;
  return RAFB200_OK;
}

static int run_update(rafb200_zero_s* z, Bucket& b, const rafb200_hyper* h, int step, float gscale,
                      cudaStream_t s) {
  switch (z->optimizer) {
    case RAFB200_OPT_SGD:
      return rafb200_sgd_list(b.list, h->learning_rate, h->mu, h->weight_decay, gscale, s);
    case RAFB200_OPT_ADAM:
      return rafb200_adam(b.list, step, nullptr, h->learning_rate, h->beta1, h->beta2, h->eps,
                          h->bias_correction, h->weight_decay, h->mode, gscale, s);
    default:
      return rafb200_lans(b.list, step, nullptr, h->learning_rate, h->beta1, h->beta2, h->eps,
                          h->bias_correction, h->weight_decay, h->grad_averaging, h->mode,
                          h->normalize_grad, gscale, b.lans_ws, b.lans_ws_bytes, s);
  }
}

// One step.  grads_host / params_host are NULL for the device-buffer form; otherwise the
// gradients of bucket b arrive on the copy-in stream while earlier buckets are in flight and
// its parameters leave on the copy-out stream as soon as they are complete.
static int step_impl(rafb200_zero_t z, const rafb200_hyper* h, int step, void* compute_stream,
                     void* comm_stream, const void* const* grads_host, void* const* params_host) {
  RAFB200_REQUIRE(z && h, "rafb200_zero_step: NULL argument");
  RAFB200_REQUIRE(z->bound, "rafb200_zero_step: bind buffers first");
  RAFB200_REQUIRE(h->optimizer == z->optimizer, "rafb200_zero_step: optimizer differs from the one created");
  // A barrier of an earlier step gave up: the ranks are no longer in step and every later
  // barrier would pass without waiting.  Queue nothing more.
  if (z->host_err && *z->host_err != 0) return wait_expired(*z->host_err);
  cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
  cudaStream_t ms = static_cast<cudaStream_t>(comm_stream);
  // A mean over ranks is a sum on the wire and a 1/n folded into the update's
  // gradient scale (the `divide` of partition_gradient.cc:274-279, fused).
  const float gscale = h->grad_scale * ((h->average && z->n > 1) ? 1.0f / (float)z->n : 1.0f);
  const int gs = dtype_size(z->g_dtype), ps = dtype_size(z->param_dtype);
  const bool host = grads_host != nullptr;
  std::vector<Bucket>& bl = (z->n == 1 && host && !z->hbuckets.empty()) ? z->hbuckets : z->buckets;
  const int nb = (int)bl.size();
  if (host) {
    // Every copy from the host is queued up front, bucket by bucket, behind whatever the
    // compute stream still does with the gradient buffers.
    RAFB200_CUDA(cudaEventRecord(z->ev_start, cs));
    RAFB200_CUDA(cudaStreamWaitEvent(z->h2d_stream, z->ev_start, 0));
    RAFB200_CUDA(cudaStreamWaitEvent(z->d2h_stream, z->ev_start, 0));
    for (auto& b : bl) {
      // Tensors that follow one another in host AND device memory, inside ranges the caller
      // declared to be single allocations, travel as one copy: a caller that keeps its
      // gradients (parameters) in one arena per side pays one copy per bucket and direction
      // instead of one per tensor.  (A copy must not span two allocations, however close.)
      const char *run_src = nullptr;
      char* run_dst = nullptr;
      size_t run = 0;
      auto flush = [&]() -> int {
        if (run) RAFB200_CUDA(cudaMemcpyAsync(run_dst, run_src, run, cudaMemcpyHostToDevice, z->h2d_stream));
        run = 0;
        return RAFB200_OK;
      };
      for (int i : b.tensors) {
        const size_t bytes = (size_t)z->plan.numel[i] * gs;
        if (!bytes) continue;
        const char* src = static_cast<const char*>(grads_host[i]);
        char* dst = static_cast<char*>(z->grads[i]);
        if (run && src == run_src + run && dst == run_dst + run && z->in_one_arena(run_src, src + bytes) &&
            z->in_one_arena(run_dst, dst + bytes)) {
          run += bytes;
          continue;
        }
        if (int rc = flush()) return rc;
        run_src = src;
        run_dst = dst;
        run = bytes;
      }
      if (int rc = flush()) return rc;
      RAFB200_CUDA(cudaEventRecord(b.h2d_done, z->h2d_stream));
    }
  }
  auto copy_out = [&](Bucket& b) -> int {  // after the last kernel of bucket b on the compute stream
    if (!host) return RAFB200_OK;
    RAFB200_CUDA(cudaEventRecord(b.out_ready, cs));
    RAFB200_CUDA(cudaStreamWaitEvent(z->d2h_stream, b.out_ready, 0));
    const char* run_src = nullptr;
    char* run_dst = nullptr;
    size_t run = 0;
    auto flush = [&]() -> int {
      if (run) RAFB200_CUDA(cudaMemcpyAsync(run_dst, run_src, run, cudaMemcpyDeviceToHost, z->d2h_stream));
      run = 0;
      return RAFB200_OK;
    };
    for (int i : b.tensors) {
      // what leaves: the whole parameter, or (host_output 1) the rows this rank owns
      int64_t lo = 0, hi = z->plan.numel[i];
      if (z->host_output == 1 && z->n > 1) {
        lo = std::min<int64_t>(hi, (int64_t)z->rank * z->plan.shard_elems[i]);
        hi = std::min<int64_t>(hi, lo + z->plan.shard_elems[i]);
      }
      const size_t bytes = (size_t)(hi - lo) * ps;
      if (!bytes) continue;
      const char* src = static_cast<const char*>(z->params[i]) + (size_t)lo * ps;
      char* dst = static_cast<char*>(params_host[i]) + (size_t)lo * ps;
      if (run && src == run_src + run && dst == run_dst + run && z->in_one_arena(run_src, src + bytes) &&
          z->in_one_arena(run_dst, dst + bytes)) {
        run += bytes;
        continue;
      }
      if (int rc = flush()) return rc;
      run_src = src;
      run_dst = dst;
      run = bytes;
    }
    return flush();
  };
  auto finish = [&]() -> int {  // the compute stream ends the step for the caller
    if (!host) return RAFB200_OK;
    RAFB200_CUDA(cudaEventRecord(z->ev_d2h_done, z->d2h_stream));
    RAFB200_CUDA(cudaStreamWaitEvent(cs, z->ev_d2h_done, 0));
    return RAFB200_OK;
  };
  if (z->n == 1) {
    for (auto& b : bl) {
      if (host) RAFB200_CUDA(cudaStreamWaitEvent(cs, b.h2d_done, 0));
      int rc = run_update(z, b, h, step, gscale, cs);
      if (rc != RAFB200_OK) return rc;
      if ((rc = copy_out(b)) != RAFB200_OK) return rc;
    }
    return finish();
  }
  // (the host-buffer form keeps the bucketed pipeline: there the copies from and to the host
  // bound the step, and they overlap with the buckets' kernels)
  if (z->fused && !host && z->symmetric && (z->optimizer != RAFB200_OPT_LANS || h->normalize_grad) && z->stage_mask == 31) {
    // The step as one update launch: pack -> every rank's gradients are in place (barrier) ->
    // the LANS kernel, whose gradient-norm items read the sum over ranks through the switch
    // and, with z->fused == 2, whose stage 2 stores the model-dtype copy into every rank's
    // buffer -> (otherwise the all-gather kernels) -> everything has landed (barrier) -> unpack.
    // All on the compute stream; link-bound and memory-bound items interleave inside the kernel.
    for (auto& b : z->buckets) {
      int rc = launch_seg_copy(b.dev_pack, b.dev_pack_items, b.n_pack_items, gs, z->sm_count, cs);
      if (rc != RAFB200_OK) return rc;
    }
    int rc = symm_barrier(z->sig_peers, z->n, z->rank, 0, ++z->epoch[0], z->wait_limit_ns, z->dev_err,
                          z->host_err_dev, cs);
    if (rc != RAFB200_OK) return rc;
    if (z->optimizer == RAFB200_OPT_SGD)
      rc = rafb200_sgd_list(z->fused_list, h->learning_rate, h->mu, h->weight_decay, gscale, cs);
    else if (z->optimizer == RAFB200_OPT_ADAM)
      rc = rafb200_adam(z->fused_list, step, nullptr, h->learning_rate, h->beta1, h->beta2, h->eps,
                        h->bias_correction, h->weight_decay, h->mode, gscale, cs);
    else
      rc = rafb200_lans(z->fused_list, step, nullptr, h->learning_rate, h->beta1, h->beta2, h->eps,
                        h->bias_correction, h->weight_decay, h->grad_averaging, h->mode, h->normalize_grad,
                        gscale, z->fused_ws, z->fused_ws_bytes, cs);
    if (rc != RAFB200_OK) return rc;
    if (z->fused < 2)
      for (auto& b : z->buckets) {
        rc = symm_allgather(z->p_peers, z->p_mc, z->p_flat, b.dev_ag_segs, b.dev_ag_items, b.n_ag_items, z->n,
                            z->rank, z->comm_blocks, cs);
        if (rc != RAFB200_OK) return rc;
      }
    rc = symm_barrier(z->sig_peers, z->n, z->rank, 1, ++z->epoch[1], z->wait_limit_ns, z->dev_err,
                      z->host_err_dev, cs);
    if (rc != RAFB200_OK) return rc;
    for (auto& b : z->buckets) {
      rc = launch_seg_copy(b.dev_unpack, b.dev_unpack_items, b.n_unpack_items, ps, z->sm_count, cs);
      if (rc != RAFB200_OK) return rc;
    }
    return finish();
  }
  // The communication stream must not run ahead of work already queued on the compute
  // stream that still uses the flat buffers (the previous step's unpack).
  if (!host) RAFB200_CUDA(cudaEventRecord(z->ev_start, cs));
  RAFB200_CUDA(cudaStreamWaitEvent(ms, z->ev_start, 0));
  if (z->symmetric) RAFB200_CUDA(cudaStreamWaitEvent(z->gather_stream, z->ev_start, 0));
  // Software pipeline over buckets; stage s of bucket b is issued in iteration b + s:
  //   0 pack (compute)  1 reduce-scatter (comm)  2 update (compute)  3 all-gather (comm)
  //   4 unpack (compute)
  // so bucket b+1 is on the wire while bucket b is being updated.
  for (int it = 0; it < nb + 2; ++it) {
    if (it < nb) {
      Bucket& b = z->buckets[it];
      int rc = RAFB200_OK;
      if (host) RAFB200_CUDA(cudaStreamWaitEvent(cs, b.h2d_done, 0));
      if (z->stage_mask & 1)
        rc = launch_seg_copy(b.dev_pack, b.dev_pack_items, b.n_pack_items, gs, z->sm_count, cs);
      if (rc != RAFB200_OK) return rc;
      RAFB200_CUDA(cudaEventRecord(b.packed, cs));
      RAFB200_CUDA(cudaStreamWaitEvent(ms, b.packed, 0));
      if ((z->stage_mask & 2) && !z->symmetric)
        rc = rafb200_reduce_scatter(z->comm, b.g_flat, b.g_flat + (size_t)z->rank * b.slot_elems * gs,
                                    b.slot_elems, z->g_dtype, "sum", ms);
      if ((z->stage_mask & 2) && z->symmetric) {
        // every rank has packed this bucket -> sum this rank's slot over all ranks, in place
        rc = symm_barrier(z->sig_peers, z->n, z->rank, 0, ++z->epoch[0], z->wait_limit_ns, z->dev_err,
                          z->host_err_dev, ms);
        if (rc != RAFB200_OK) return rc;
        rc = symm_reduce_scatter(z->g_peers, z->g_mc, z->g_red, b.dev_rs_segs, b.dev_rs_items, b.n_rs_items,
                                 z->g_dtype, z->n, z->comm_blocks, ms);
      }
      if (rc != RAFB200_OK) return rc;
      RAFB200_CUDA(cudaEventRecord(b.rs_done, ms));
    }
    if (it >= 1 && it - 1 < nb) {
      Bucket& b = z->buckets[it - 1];
      RAFB200_CUDA(cudaStreamWaitEvent(cs, b.rs_done, 0));
      int rc = (z->stage_mask & 4) ? run_update(z, b, h, step, gscale, cs) : (int)RAFB200_OK;
      if (rc != RAFB200_OK) return rc;
      RAFB200_CUDA(cudaEventRecord(b.upd_done, cs));
      // In symmetric mode the all-gather has a stream of its own: it loads the links in the
      // direction the reduce-scatter leaves idle, so the two overlap.
      cudaStream_t as = z->symmetric ? z->gather_stream : ms;
      RAFB200_CUDA(cudaStreamWaitEvent(as, b.upd_done, 0));
      if ((z->stage_mask & 8) && !z->symmetric)
        rc = rafb200_allgather(z->comm, b.p_flat + (size_t)z->rank * b.slot_elems * ps, b.p_flat,
                               b.slot_elems, z->param_dtype, ms);
      if ((z->stage_mask & 8) && z->symmetric) {
        rc = symm_allgather(z->p_peers, z->p_mc, z->p_flat, b.dev_ag_segs, b.dev_ag_items, b.n_ag_items, z->n,
                            z->rank, z->comm_blocks, as);
        if (rc != RAFB200_OK) return rc;
        // every rank's slot has landed here before the unpack reads the buffer
        rc = symm_barrier(z->sig_peers, z->n, z->rank, 1, ++z->epoch[1], z->wait_limit_ns, z->dev_err,
                          z->host_err_dev, as);
      }
      if (rc != RAFB200_OK) return rc;
      RAFB200_CUDA(cudaEventRecord(b.ag_done, as));
    }
    if (it >= 2) {
      Bucket& b = z->buckets[it - 2];
      RAFB200_CUDA(cudaStreamWaitEvent(cs, b.ag_done, 0));
      int rc = RAFB200_OK;
      if (z->stage_mask & 16)
        rc = launch_seg_copy(b.dev_unpack, b.dev_unpack_items, b.n_unpack_items, ps, z->sm_count, cs);
      if (rc != RAFB200_OK) return rc;
      if ((rc = copy_out(b)) != RAFB200_OK) return rc;
    }
  }
  return finish();
}

int rafb200_zero_step(rafb200_zero_t z, const rafb200_hyper* h, int step, void* compute_stream,
                      void* comm_stream) {
  return step_impl(z, h, step, compute_stream, comm_stream, nullptr, nullptr);
}

int rafb200_zero_step_host(rafb200_zero_t z, const rafb200_hyper* h, int step,
                           const void* const* grads_host, void* const* params_host,
                           void* compute_stream, void* comm_stream) {
  RAFB200_REQUIRE(z && h && grads_host && params_host, "rafb200_zero_step_host: NULL argument");
  RAFB200_REQUIRE(z->bound, "rafb200_zero_step_host: bind device buffers first");
  return step_impl(z, h, step, compute_stream, comm_stream, grads_host, params_host);
}

}  // extern "C"
