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

constexpr int kChunkElems = 4096;  // elements per work item of the SGD / Adam kernels
constexpr int kBlockThreads = 256;

// Work items of the LANS kernel.  The two top bits of Item::tensor_phase are the kind:
//   A    sum of squares of a chunk of kLansAElems* gradient elements
//   Bs   stage 1 of a chunk of kLansElems elements, sums only ("streamed")
//   Cs   stage 1 again and stage 2 of the same chunk, stores everything
//   BCp  both on a chunk that stays in shared memory in between ("parked")
constexpr uint32_t kKindA = 0, kKindBs = 1, kKindCs = 2, kKindBCp = 3;
constexpr int kLansVecs = 2;          // 4-element vectors a consumer thread holds per array per item
constexpr int kLansElems = 128 * 4 * kLansVecs;  // elements per Bs / Cs / BCp item = one slot (1024)
constexpr int kLansAElems16 = kLansElems * 7;    // gradient elements per A item (what a slot holds), 16-bit g
constexpr int kLansAElems32 = kLansElems * 4;    // the same for fp32 gradients
// One block per SM.  Its shared memory holds the slots (chunks on their way in: 14 KB each with
// 16-bit gradients, 16 KB with fp32 ones) and eight cells for parked chunks (12 KB each: p,
// update_m, update_g); 21 more cells of 24 columns each live in the SM's tensor memory.
constexpr int kLansSlots16 = 8;
constexpr int kLansSlots32 = 6;
constexpr int kLansTmemCells = 512 / (12 * kLansVecs);  // 21
constexpr int kLansSmemCells = 8;
constexpr int kLansCells = kLansTmemCells + kLansSmemCells;  // parked chunks per block: 29
constexpr int kLansNBits = 13;  // bits of an element count inside an item (<= 7168)
static_assert(kLansVecs == 2, "slot, cell and queue sizes below are for chunks of 1024 elements");
static_assert(kLansAElems16 < (1 << kLansNBits) && kLansAElems32 < (1 << kLansNBits) &&
                  kLansCells <= (1 << (32 - 2 * kLansNBits)),
              "count, bulk count and cell number of an item share one 32-bit word");

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
  // first 64-byte line: read-mostly, polled by the blocks that wait for the tensor
  unsigned int norm[4];    // ||g||, ||p||, ||update_m||, ||update_g||: bits | 0x80000000 once final
  unsigned int pad0_[12];
  // second line: updated with atomics by the blocks that add their parts
  unsigned int arrived_a;  // gradient-norm items that have added their partial
  unsigned int arrived_b;  // stage-1 chunks that have added theirs
  unsigned int pad1_[6];
  double sumsq[4];         // running sums of squares of the same four quantities
};
constexpr unsigned int kNormValid = 0x80000000u;
static_assert(sizeof(LansCtl) == 128, "LansCtl is two 64-byte lines");

struct LansHeader {
  unsigned int ticket;   // next work item to hand out
  unsigned int error;    // 0, or the code of the bounded wait that expired
  unsigned int error_item;
  unsigned int pad1_;
  float inv_bc1;         // reciprocal bias corrections when `step` lives on the device
  float inv_bc2;
};

constexpr int kSymmMaxWorld = 16;   // ranks of one NVLink domain addressed by value

// Collectives inside the LANS kernel (see LansParams in lans.cu): where the symmetric gradient
// and parameter buffers are mapped.  Set on a list by tensor_list_set_fuse, together with each
// tensor's byte offset inside the symmetric gradient buffer, which then takes the place of
// TensorDesc::first_chunk / nchunks (low / high word) - the LANS kernel reads neither.
struct LansFuse {
  int world = 0, rank = 0, fuse_rs = 0, fuse_ag = 0;
  const char* g_mc = nullptr;
  char* p_mc = nullptr;
  const char* g_peer[kSymmMaxWorld] = {};
  char* p_peer[kSymmMaxWorld] = {};
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
  // LANS schedule, rebuilt when tuned: per-block item lists (offsets, then items)
  uint32_t* dev_lans_lists = nullptr;         // with the gradient-norm items
  uint32_t* dev_lans_lists_nonorm = nullptr;  // normalize_grad == 0: no A items
  int64_t lead_elems = 0;   // how far the gradient-norm pass runs ahead
  int gap_items = 0;        // items between a tensor's last parked item and its streamed updates
  int max_blocks = 0;
  int sm_count = 0;
  int lans_grid = 0;        // blocks the LANS schedule was built for
  bool custom_items = false;
  uint64_t wait_ns = 2000000000ull;  // bound of every wait inside the LANS kernel
  rafb200::LansFuse fuse;            // collectives inside the LANS kernel, off by default
};

namespace rafb200 {
int tensor_list_set_fuse(rafb200_tensor_list_s* l, const LansFuse& f, const int64_t* sym_off_bytes);
}
