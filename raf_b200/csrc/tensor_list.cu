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

std::vector<Item> build_lans_schedule(const std::vector<uint32_t>& nchunks, bool with_a,
                                      int64_t window_chunks, int slack);
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

static int rebuild_lans_schedule(rafb200_tensor_list_s* l) {
  std::vector<uint32_t> nchunks(l->k);
  for (int i = 0; i < l->k; ++i) nchunks[i] = l->host_desc[i].nchunks;
  int64_t window_chunks = l->window_elems / kChunkElems;
  if (window_chunks < 1) window_chunks = 1;
  int rc = upload_items(build_lans_schedule(nchunks, true, window_chunks, l->slack_items),
                        &l->dev_lans_items, &l->n_lans_items);
  if (rc != RAFB200_OK) return rc;
  return upload_items(build_lans_schedule(nchunks, false, window_chunks, l->slack_items),
                      &l->dev_lans_items_nonorm, &l->n_lans_items_nonorm);
}

}  // namespace rafb200

using namespace rafb200;

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
    if (numel[i] < 0) {
      delete l;
      return set_error(RAFB200_INVALID_ARGUMENT, "rafb200_tensor_list_create: numel[%d] < 0", i);
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
    // Defaults.  A block holds up to three tickets and three blocks run per SM, so about
    // eight items per SM are in flight; that many items are placed between the last item
    // of a phase of a tensor and the first item that depends on it.  With the round-robin
    // order of the three passes the step time is flat in this value (0 to 32 per SM
    // measured within 1 %).  The B pass may lead the C pass by 32 Mi elements at most.
    l->slack_items = 8 * l->sm_count;
    l->window_elems = 32ll << 20;
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
  if (l->dev_lans_items) cudaFree(l->dev_lans_items);
  if (l->dev_lans_items_nonorm) cudaFree(l->dev_lans_items_nonorm);
  delete l;
  return RAFB200_OK;
}

int64_t rafb200_tensor_list_total_elems(rafb200_tensor_list_t l) { return l ? l->total_elems : 0; }

int rafb200_tensor_list_tune(rafb200_tensor_list_t l, int64_t window_elems, int slack_items,
                             int max_blocks) {
  RAFB200_REQUIRE(l, "rafb200_tensor_list_tune: NULL list");
  RAFB200_REQUIRE(window_elems >= 0 && slack_items >= 0 && max_blocks >= 0,
                  "rafb200_tensor_list_tune: negative argument");
  const bool resched = (window_elems != l->window_elems) || (slack_items != l->slack_items);
  l->window_elems = window_elems;
  l->slack_items = slack_items;
  l->max_blocks = max_blocks;
  if (resched) {
    // The old tables may still be read by a kernel in flight.
    RAFB200_CUDA(cudaDeviceSynchronize());
    return rebuild_lans_schedule(l);
  }
  return RAFB200_OK;
}

}  // extern "C"
