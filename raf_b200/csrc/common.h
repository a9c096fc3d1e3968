// Shared host-side declarations of libraf_b200: status handling, the device
// descriptor tables and the tensor-list object.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/raf_b200.h"

namespace rafb200 {

// ---- status ---------------------------------------------------------------
int set_error(int status, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define RAFB200_CUDA(expr)                                                                  \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess)                                                                 \
      return ::rafb200::set_error(RAFB200_CUDA_ERROR, "%s:%d: %s failed: %s", __FILE__,      \
                                  __LINE__, #expr, cudaGetErrorString(e__));                \
  } while (0)

#define RAFB200_REQUIRE(cond, ...)                                                \
  do {                                                                            \
    if (!(cond)) return ::rafb200::set_error(RAFB200_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

inline int dtype_size(int dtype) { return dtype == RAFB200_F32 ? 4 : 2; }
inline bool dtype_valid(int dtype) { return dtype >= RAFB200_F32 && dtype <= RAFB200_BF16; }

// ---- device tables ----------------------------------------------------------
// One row per tensor of a list.  `flags` bit 0: every bound pointer is aligned
// for the vector path (16 bytes for fp32 arrays, 8 bytes for 16-bit arrays).
struct TensorDesc {
  const void* g;
  float* p;
  float* m;
  float* v;
  void* out;
  int64_t numel;
  uint32_t first_chunk;  // index of this tensor's first chunk in the list-wide chunk numbering
  uint32_t nchunks;
  uint32_t flags;
  uint32_t pad_;
};
static_assert(sizeof(TensorDesc) == 64, "TensorDesc is one 64-byte row");

// A work item = one chunk of one tensor in one phase.
// word0: bits 31..30 phase, bits 29..0 tensor index; word1: chunk index inside the tensor.
struct Item {
  uint32_t tensor_phase;
  uint32_t chunk;
};
constexpr uint32_t kPhaseShift = 30;
constexpr uint32_t kTensorMask = (1u << kPhaseShift) - 1u;

constexpr int kChunkElems = 4096;  // elements per work item
constexpr int kBlockThreads = 256;

// Per-tensor control words of the LANS kernel (zeroed at the start of every call).
// A norm word is "final" when its top bit is set: the publisher stores the bits of
// the (non-negative) norm with the sign bit on, in one 4-byte store.  Validity and
// value travel in the same word, so readers need no acquire ordering between a flag
// and the data - a plain load that sees the bit sees the value.
//
// Sums of squares are accumulated per tensor with double-precision atomic adds of
// the per-chunk fp32 partial sums.  A partial has a 24-bit significand and a tensor
// has at most 2^13 chunks here, so as long as the chunk sums of one tensor lie within
// a factor 2^16 of each other every addition is exact and the total does not depend
// on the order in which blocks arrive; outside that range the order can show in the
// 53rd bit, far below the fp32 rounding of the norm.
struct LansCtl {
  unsigned int arrived_a;  // chunks of phase A that have added their partial
  unsigned int arrived_b;
  unsigned int pad_[2];
  unsigned int norm[4];    // ||g||, ||p||, ||update_m||, ||update_g||: bits | 0x80000000 once final
  double sumsq[4];         // running sums of squares of the same four quantities
};
constexpr unsigned int kNormValid = 0x80000000u;
static_assert(sizeof(LansCtl) == 64, "LansCtl is 64 bytes");

struct LansHeader {
  unsigned int ticket;   // next work item to hand out
  unsigned int error;    // 0, or the code of the bounded wait that expired
  unsigned int error_item;
  unsigned int pad_;
  float inv_bc1;         // reciprocal bias corrections when `step` lives on the device
  float inv_bc2;
};

}  // namespace rafb200

// The opaque list object of the C ABI.
struct rafb200_tensor_list_s {
  int k = 0;
  int g_dtype = 0;
  int out_dtype = 0;
  int device = 0;
  int64_t total_elems = 0;
  uint32_t total_chunks = 0;
  std::vector<int64_t> numel;
  std::vector<rafb200::TensorDesc> host_desc;   // last table sent to the device
  rafb200::TensorDesc* dev_desc = nullptr;
  bool bound = false;
  bool has_v = false, has_out = false;
  // single-phase item table (SGD / Adam), tensor-major
  rafb200::Item* dev_items = nullptr;
  uint32_t n_items = 0;
  // LANS schedule (three phases interleaved), rebuilt when tuned
  rafb200::Item* dev_lans_items = nullptr;       // with the gradient-norm phase
  uint32_t n_lans_items = 0;
  rafb200::Item* dev_lans_items_nonorm = nullptr;  // normalize_grad == 0: no phase A
  uint32_t n_lans_items_nonorm = 0;
  int64_t window_elems = 0;
  int slack_items = 0;
  int max_blocks = 0;
  int sm_count = 0;
};
