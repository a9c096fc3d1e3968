// Tensor-list objects, error reporting and library identity.
#include <cstdlib>
#include <cstring>

#include "common.h"

namespace rafb200 {

static thread_local char g_last_error[1024] = "";

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

std::vector<Item> build_lans_schedule(const std::vector<int64_t>& numel, int a_elems, bool with_a,
                                      uint32_t park_cap, int64_t lead_elems, int64_t gap_items);
int lans_slots(int g_dtype);
int lans_a_elems(int g_dtype);
uint32_t lans_park_cap(int64_t cells_total);
int lans_grid(int sm_count, int max_blocks);
std::vector<uint32_t> partition_lans_items(const std::vector<Item>& sched, int grid, int slots);
bool pointers_aligned(const void* g, int g_dtype, const void* p, const void* m, const void* v,
                      const void* out, int out_dtype);

static int upload_items(const std::vector<Item>& items, Item** dev, uint32_t* n) {
  if (*dev) {
    cudaFree(*dev);
    *dev = nullptr;
  }
  *n = (uint32_t)items.size();
  if (items.empty()) return RAFB200_OK;
  RAFB200_CUDA(cudaMalloc(reinterpret_cast<void**>(dev), items.size() * sizeof(Item)));
  RAFB200_CUDA(cudaMemcpy(*dev, items.data(), items.size() * sizeof(Item), cudaMemcpyHostToDevice));
  return RAFB200_OK;
}

static int upload_lists(const std::vector<Item>& sched, int grid, int slots, uint32_t** dev) {
  if (*dev) {
    cudaFree(*dev);
    *dev = nullptr;
  }
  const std::vector<uint32_t> table = partition_lans_items(sched, grid, slots);
  RAFB200_CUDA(cudaMalloc(reinterpret_cast<void**>(dev), table.size() * sizeof(uint32_t)));
  RAFB200_CUDA(cudaMemcpy(*dev, table.data(), table.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
  return RAFB200_OK;
}

static int rebuild_lans_schedule(rafb200_tensor_list_s* l) {
  l->lans_grid = lans_grid(l->sm_count, l->max_blocks);
  const int64_t slots_total = (int64_t)l->lans_grid * lans_slots(l->g_dtype);
  const uint32_t cap = lans_park_cap((int64_t)l->lans_grid * kLansCells);
  const int64_t gap = l->gap_items > 0 ? l->gap_items : slots_total;
  const int a_elems = lans_a_elems(l->g_dtype);
  l->custom_items = false;
  int rc = upload_lists(build_lans_schedule(l->numel, a_elems, true, cap, l->lead_elems, gap), l->lans_grid, lans_slots(l->g_dtype),
                        &l->dev_lans_lists);
  if (rc != RAFB200_OK) return rc;
  return upload_lists(build_lans_schedule(l->numel, a_elems, false, cap, l->lead_elems, gap), l->lans_grid, lans_slots(l->g_dtype),
                      &l->dev_lans_lists_nonorm);
}

}  // namespace rafb200

using namespace rafb200;

namespace rafb200 {
int tensor_list_set_fuse(rafb200_tensor_list_s* l, const LansFuse& f, const int64_t* sym_off_bytes) {
  RAFB200_REQUIRE(l && (f.fuse_rs == 0 || sym_off_bytes), "tensor_list_set_fuse: NULL argument");
  RAFB200_REQUIRE(f.world >= 1 && f.world <= kSymmMaxWorld && f.rank >= 0 && f.rank < f.world,
                  "tensor_list_set_fuse: rank %d of %d", f.rank, f.world);
  l->fuse = f;
  if (f.fuse_rs) {
    for (int i = 0; i < l->k; ++i) {
      RAFB200_REQUIRE(sym_off_bytes[i] >= 0 && sym_off_bytes[i] % 16 == 0,
                      "tensor_list_set_fuse: offset of tensor %d is not a multiple of 16 bytes", i);
      l->host_desc[i].first_chunk = (uint32_t)((uint64_t)sym_off_bytes[i] & 0xffffffffu);
      l->host_desc[i].nchunks = (uint32_t)((uint64_t)sym_off_bytes[i] >> 32);
    }
    l->bound = false;  // the rows travel with the next bind
  }
  return RAFB200_OK;
}
}  // namespace rafb200

extern "C" {

const char* rafb200_last_error(void) { return g_last_error; }

int rafb200_version(void) { return 100; }

int rafb200_tensor_list_create(int k, const int64_t* numel, int g_dtype, int out_dtype,
                               rafb200_tensor_list_t* list) {
  RAFB200_REQUIRE(list, "rafb200_tensor_list_create: NULL result pointer");
  *list = nullptr;
  RAFB200_REQUIRE(k >= 0 && (k == 0 || numel), "rafb200_tensor_list_create: bad k / numel");
  RAFB200_REQUIRE((uint32_t)k <= kTensorMask, "rafb200_tensor_list_create: too many tensors");
  RAFB200_REQUIRE(dtype_valid(g_dtype) && dtype_valid(out_dtype),
                  "rafb200_tensor_list_create: bad dtype");
  auto* l = new rafb200_tensor_list_s();
  l->k = k;
  l->g_dtype = g_dtype;
  l->out_dtype = out_dtype;
  l->numel.assign(numel, numel + k);
  l->host_desc.resize(k);
  uint64_t chunks = 0;
  for (int i = 0; i < k; ++i) {
    if (numel[i] < 0 || numel[i] >= (1ll << 31)) {
      delete l;
      return set_error(RAFB200_INVALID_ARGUMENT,
                       "rafb200_tensor_list_create: numel[%d] must be in [0, 2^31)", i);
    }
    TensorDesc& d = l->host_desc[i];
    memset(&d, 0, sizeof(d));
    d.numel = numel[i];
    d.first_chunk = (uint32_t)chunks;
    const uint64_t nc = (uint64_t)((numel[i] + kChunkElems - 1) / kChunkElems);
    d.nchunks = (uint32_t)nc;
    chunks += nc;
    l->total_elems += numel[i];
  }
  if (chunks * 3 >= (1ull << 32)) {
    delete l;
    return set_error(RAFB200_INVALID_ARGUMENT, "rafb200_tensor_list_create: list too large");
  }
  l->total_chunks = (uint32_t)chunks;
  int rc = RAFB200_OK;
  do {
    if (cudaGetDevice(&l->device) != cudaSuccess ||
        cudaDeviceGetAttribute(&l->sm_count, cudaDevAttrMultiProcessorCount, l->device) !=
            cudaSuccess) {
      rc = set_error(RAFB200_CUDA_ERROR, "rafb200_tensor_list_create: no usable CUDA device: %s",
                     cudaGetErrorString(cudaGetLastError()));
      break;
    }
    if (k > 0) {
      cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&l->dev_desc), sizeof(TensorDesc) * k);
      if (e != cudaSuccess) {
        rc = set_error(RAFB200_CUDA_ERROR, "cudaMalloc(descriptor table): %s", cudaGetErrorString(e));
        break;
      }
    }
    std::vector<Item> items;
    items.reserve(chunks);
    for (int i = 0; i < k; ++i)
      for (uint32_t c = 0; c < l->host_desc[i].nchunks; ++c) items.push_back(Item{(uint32_t)i, c});
    rc = upload_items(items, &l->dev_items, &l->n_items);
    if (rc != RAFB200_OK) break;
    // Defaults.  The gradient-norm pass leads by 8 Mi elements: more than any tensor that is
    // kept on chip in full and a few thousand work items of slack, yet little enough
    // (16 MB of 16-bit gradients) that the second read of g comes from L2.  gap_items 0 =
    // one item per slot of the grid between a tensor's last parked item and its streamed
    // update items.
    l->lead_elems = 8ll << 20;
    l->gap_items = 0;
    rc = rebuild_lans_schedule(l);
  } while (false);
  if (rc != RAFB200_OK) {
    rafb200_tensor_list_destroy(l);
    return rc;
  }
  *list = l;
  return RAFB200_OK;
}

int rafb200_tensor_list_bind(rafb200_tensor_list_t l, const void* const* g, float* const* p,
                             float* const* m, float* const* v, void* const* out, void* stream) {
  RAFB200_REQUIRE(l, "rafb200_tensor_list_bind: NULL list");
  RAFB200_REQUIRE(l->k == 0 || (g && p && m), "rafb200_tensor_list_bind: g, p and m are required");
  bool changed = !l->bound;
  for (int i = 0; i < l->k; ++i) {
    TensorDesc d = l->host_desc[i];
    d.g = g[i];
    d.p = p[i];
    d.m = m[i];
    d.v = v ? v[i] : nullptr;
    d.out = out ? out[i] : nullptr;
    if (d.numel > 0) {
      RAFB200_REQUIRE(d.g && d.p && d.m, "rafb200_tensor_list_bind: NULL pointer for tensor %d", i);
      RAFB200_REQUIRE(!v || d.v, "rafb200_tensor_list_bind: NULL v for tensor %d", i);
    }
    d.flags = pointers_aligned(d.g, l->g_dtype, d.p, d.m, d.v, d.out, l->out_dtype) ? 1u : 0u;
    auto a16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if ((d.flags & 1u) && a16(d.g) && a16(d.p) && a16(d.m) && a16(d.v)) d.flags |= 2u;  // kFlagBulk
    if (memcmp(&d, &l->host_desc[i], sizeof(d)) != 0) {
      l->host_desc[i] = d;
      changed = true;
    }
  }
  l->has_v = (v != nullptr);
  l->has_out = (out != nullptr);
  if (changed && l->k > 0) {
    // Pageable source: the runtime stages the table before returning, so
    // host_desc may be modified again right away.
    RAFB200_CUDA(cudaMemcpyAsync(l->dev_desc, l->host_desc.data(), sizeof(TensorDesc) * l->k,
                                 cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  }
  l->bound = true;
  return RAFB200_OK;
}

int rafb200_tensor_list_destroy(rafb200_tensor_list_t l) {
  if (!l) return RAFB200_OK;
  if (l->dev_desc) cudaFree(l->dev_desc);
  if (l->dev_items) cudaFree(l->dev_items);
  if (l->dev_lans_lists) cudaFree(l->dev_lans_lists);
  if (l->dev_lans_lists_nonorm) cudaFree(l->dev_lans_lists_nonorm);
  delete l;
  return RAFB200_OK;
}

int rafb200_tensor_list_set_symmetric(rafb200_tensor_list_t l, int world, int rank, const void* const* g_peer,
                                      const void* g_mc, void* const* p_peer, void* p_mc,
                                      const int64_t* g_offset_bytes, int reduce_scatter, int all_gather) {
  RAFB200_REQUIRE(l, "rafb200_tensor_list_set_symmetric: NULL list");
  RAFB200_REQUIRE(world >= 1 && world <= kSymmMaxWorld && rank >= 0 && rank < world,
                  "rafb200_tensor_list_set_symmetric: rank %d of %d (at most %d ranks)", rank, world, kSymmMaxWorld);
  RAFB200_REQUIRE(!reduce_scatter || (g_peer && g_offset_bytes),
                  "rafb200_tensor_list_set_symmetric: the gradient buffers and offsets are required");
  RAFB200_REQUIRE(!all_gather || p_peer, "rafb200_tensor_list_set_symmetric: the parameter buffers are required");
  LansFuse f;
  f.world = world;
  f.rank = rank;
  f.fuse_rs = reduce_scatter ? 1 : 0;
  f.fuse_ag = all_gather ? 1 : 0;
  f.g_mc = static_cast<const char*>(g_mc);
  f.p_mc = static_cast<char*>(p_mc);
  for (int q = 0; q < world; ++q) {
    if (g_peer) f.g_peer[q] = static_cast<const char*>(g_peer[q]);
    if (p_peer) f.p_peer[q] = static_cast<char*>(p_peer[q]);
    RAFB200_REQUIRE(!reduce_scatter || f.g_peer[q], "rafb200_tensor_list_set_symmetric: NULL gradient buffer of rank %d", q);
    RAFB200_REQUIRE(!all_gather || f.p_peer[q], "rafb200_tensor_list_set_symmetric: NULL parameter buffer of rank %d", q);
  }
  return tensor_list_set_fuse(l, f, g_offset_bytes);
}

int64_t rafb200_tensor_list_total_elems(rafb200_tensor_list_t l) { return l ? l->total_elems : 0; }

int rafb200_tensor_list_tune(rafb200_tensor_list_t l, int64_t lead_elems, int gap_items,
                             int max_blocks) {
  RAFB200_REQUIRE(l, "rafb200_tensor_list_tune: NULL list");
  RAFB200_REQUIRE(lead_elems >= 0 && gap_items >= 0 && max_blocks >= 0,
                  "rafb200_tensor_list_tune: negative argument");
  const bool resched = (lead_elems != l->lead_elems) || (gap_items != l->gap_items) ||
                       (max_blocks != l->max_blocks) || l->custom_items;
  l->lead_elems = lead_elems;
  l->gap_items = gap_items;
  l->max_blocks = max_blocks;
  if (resched) {
    // The old tables may still be read by a kernel in flight.
    RAFB200_CUDA(cudaDeviceSynchronize());
    return rebuild_lans_schedule(l);
  }
  return RAFB200_OK;
}

int rafb200_tensor_list_set_wait_limit(rafb200_tensor_list_t l, int limit_ms) {
  RAFB200_REQUIRE(l && limit_ms > 0, "rafb200_tensor_list_set_wait_limit: bad arguments");
  l->wait_ns = (uint64_t)limit_ms * 1000000ull;
  return RAFB200_OK;
}

int rafb200_tensor_list_set_lans_items(rafb200_tensor_list_t l, const uint32_t* items, size_t count) {
  RAFB200_REQUIRE(l && (count == 0 || items), "rafb200_tensor_list_set_lans_items: bad arguments");
  RAFB200_REQUIRE(count < (1ull << 32), "rafb200_tensor_list_set_lans_items: too many items");
  std::vector<Item> v(count);
  for (size_t i = 0; i < count; ++i) {
    v[i] = Item{items[2 * i], items[2 * i + 1]};
    const uint32_t t = v[i].tensor_phase & kTensorMask, kind = v[i].tensor_phase >> kPhaseShift;
    RAFB200_REQUIRE((int)t < l->k, "rafb200_tensor_list_set_lans_items: item %zu names tensor %u", i, t);
    const int64_t per = kind == kKindA ? lans_a_elems(l->g_dtype) : kLansElems;
    RAFB200_REQUIRE((int64_t)v[i].chunk * per < l->numel[t],
                    "rafb200_tensor_list_set_lans_items: item %zu is past the end of tensor %u", i, t);
  }
  RAFB200_CUDA(cudaDeviceSynchronize());  // the old tables may still be read by a kernel in flight
  int rc = upload_lists(v, l->lans_grid, lans_slots(l->g_dtype), &l->dev_lans_lists);
  if (rc != RAFB200_OK) return rc;
  rc = upload_lists(v, l->lans_grid, lans_slots(l->g_dtype), &l->dev_lans_lists_nonorm);
  l->custom_items = true;
  return rc;
}

}  // extern "C"
