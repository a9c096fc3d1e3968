// raf.op.lans as ONE persistent kernel that keeps a chunk on chip between its two stages.
//
// The reference runs four norm reductions and two element-wise stages as about
// fifty launches with a global dependency between them
// (src/op/dialect/cuda/kernels/multi_tensor_lans.cu:401-450) and moves about 68 bytes
// per element.  The dependencies are real: stage 1 needs ||g|| of the whole tensor,
// stage 2 needs ||p||, ||update_m|| and ||update_g|| of the whole tensor.  Here one
// block per SM owns shared-memory SLOTS of 1024 elements (g, p, m, v), filled by the TMA
// unit, and CELLS of 1024 elements (p, update_m, update_g) in which a chunk waits while the
// other blocks complete the tensor-wide norms: 21 cells in the SM's tensor memory
// (tcgen05.alloc / st / ld - no MMA is issued, the 256 KB serve as scratchpad) and 8 in
// shared memory.
//   item A    (7168 / 4096 elements of g)  sum of squares of the scaled gradient -> ||g||.
//             Runs a few million elements ahead of the rest, so ||g|| is final
//             when a tensor's other items come up (the re-read of g comes from L2).
//   item BCp  "parked": load g, p, m, v once; when ||g|| is final compute stage 1,
//             store m and v, move p, update_m, update_g into a cell and add the sums of
//             squares to the tensor's accumulators; when the three norms are final,
//             finish stage 2 from the cell and store p and the model-dtype copy.
//             DRAM traffic: every array read once and written once.
//   items Bs + Cs  "streamed", for the part of a tensor that exceeds what the grid may
//             park (five eighths of all cells): Bs computes the sums and stores
//             nothing, Cs loads the chunk again, recomputes stage 1 with the same
//             instructions (same bits) and stores everything.
// The host fixes the order of the items and deals them out to the blocks in turn - inside a
// block to the list of its even or of its odd slots - so every list is run in order.  An
// item only ever waits for items that come earlier in the global order; cells are granted
// by the parked items' running numbers (a later item takes one only while a free cell
// remains for every earlier item without one), and a tensor has fewer parked items in a list
// than the list has cells: the bounded waits below cannot deadlock.
//
// Roles inside a block (640 threads):
//   warps 0-15  four consumer groups of four warps; group q serves the slots s with
//               s % 4 == q.  The warps of a group take turns in the bookkeeping after an
//               operation: free the slot or cell, take the slot's next item from its
//               mailbox and start it (bulk copies + first operation).
//   warps 16,17 prefetchers, one per list: a lane per mailbox resolves the items ahead of
//               their use (item -> descriptor -> the norms its first operation needs are
//               final -> a cell if it parks -> mailbox).
//   warp 18     parker: owns the tensor-memory allocation; lane c polls the norm words of the
//               tensor whose chunk is parked in cell c and queues the chunk's second half;
//               lanes that wait for the same tensor share one load.
//   warp 19     publisher: collects the groups' partial sums, adds them (in double
//               precision) to the tensor's accumulators, counts arrivals; the last
//               arrival takes the square root and publishes the norm together with its
//               "final" bit in one word.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.h"
#include "symm.h"
#include "symm_dev.cuh"
#include "update_core.cuh"

namespace rafb200 {

void bias_corrections(float beta1, float beta2, int step, int bias_correction, float* bc1,
                      float* bc2);

constexpr uint32_t kOpA = 0, kOpB = 1, kOpBP = 2, kOpC = 3, kOpCP = 4, kOpEnd = 7;
constexpr unsigned kErrWaitG = 1, kErrWaitN = 2, kErrRing = 3, kErrData = 4, kErrDone = 5;

struct LansParams {
  const TensorDesc* descs;
  const uint32_t* block_off;  // list h (2b: even slots of block b, 2b + 1: odd) = items[block_off[h] .. block_off[h + 1])
  const Item* items;
  LansHeader* hdr;
  LansCtl* ctl;
  LansStage1 s1;
  float lr;
  const float* step_dev;
  int bias_correction;
  uint64_t wait_ns;  // bound of every wait inside the kernel
  // Collectives inside the kernel (n > 1, symmetric memory; all zero otherwise).
  // fuse_rs: an A item does not read the local gradient but the SUM over ranks of the chunk -
  // through the multicast address (g_mc) or peer by peer (g_peer) - at byte offset
  // TensorDesc::sym_off + chunk start, writes it to the local gradient block (desc.g) for the
  // later stages and squares what it wrote.  fuse_ag: the model-dtype copy (`out`, which then
  // lies in this rank's mapping p_peer[rank] of the symmetric parameter buffer) is stored into
  // every rank's buffer: through p_mc, or to the peers one by one.
  int world, rank, fuse_rs, fuse_ag;
  const char* g_mc;
  char* p_mc;
  const char* g_peer[kSymmMaxWorld];
  char* p_peer[kSymmMaxWorld];
};

// The model-dtype copy of four elements (or one), into every rank's parameter buffer.
template <typename OT>
__device__ __forceinline__ void store_out_everywhere(const LansParams& P, OT* local, const F4& v) {
  store4_everywhere<OT>(P.p_mc, P.p_peer, P.world, P.rank, local, v);
}
template <typename OT>
__device__ __forceinline__ void store_out_everywhere1(const LansParams& P, OT* local, float x) {
  store1_everywhere<OT>(P.p_peer, P.world, P.rank, local, x);
}

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The four norm words of a tensor, read with one relaxed 16-byte load.
__device__ __forceinline__ uint4 ld_norms(const LansCtl* c) {
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(c->norm));
  return r;
}
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ uint2 ld_global_v2(const void* p) {
  uint2 r;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
__device__ __forceinline__ float norm_value(unsigned bits) {
  return __uint_as_float(bits & ~kNormValid);
}

// `step` as a 0-d fp32 device tensor (python/raf/optim/lans.py:239): the bias
// corrections of lans.cc:100-105 (float base, int exponent, evaluated in
// double) are computed by one thread into the workspace header instead of
// copying the step to the host.  Runs after the header was zeroed.
__global__ void lans_bias_kernel(LansHeader* hdr, const float* step_dev, float beta1, float beta2,
                                 int bias_correction) {
  float bc1 = 1.0f, bc2 = 1.0f;
  if (bias_correction == 1) {
    const int step = (int)(*step_dev);
    bc1 = (float)(1.0 - pow((double)beta1, (double)step));
    bc2 = (float)(1.0 - pow((double)beta2, (double)step));
  }
  hdr->inv_bc1 = 1.0f / bc1;
  hdr->inv_bc2 = 1.0f / bc2;
}

// ---- TMA / mbarrier primitives (sm_90+; written for sm_100a) -------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Non-blocking: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Potentially blocking test: the hardware may suspend the thread for a short,
// implementation-defined time while the phase is incomplete.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// One-dimensional bulk copy global -> this CTA's shared memory through the TMA
// unit; completion is signalled on `bar` by byte count.  Both addresses are
// 16-byte aligned and `bytes` is a multiple of 16.
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                            uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later
// accesses of the async proxy (the next bulk copy into the same slot).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tensor memory as a scratchpad ------------------------------------------------------
// 32x32b accesses: the 32 threads of a warp address the 32 lanes of the warp's own quarter
// of tensor memory (lanes 32 * (warp % 4) ...); thread t reads / writes eight consecutive
// 32-bit columns of lane t.  `taddr` = (first lane of the quarter << 16) | first column.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const F4& a, const F4& b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(__float_as_uint(a.x[0])), "r"(__float_as_uint(a.x[1])), "r"(__float_as_uint(a.x[2])),
               "r"(__float_as_uint(a.x[3])), "r"(__float_as_uint(b.x[0])), "r"(__float_as_uint(b.x[1])),
               "r"(__float_as_uint(b.x[2])), "r"(__float_as_uint(b.x[3]))
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, F4& a, F4& b) {
  uint32_t r0, r1, r2, r3, r4, r5, r6, r7;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3), "=r"(r4), "=r"(r5), "=r"(r6), "=r"(r7)
               : "r"(taddr)
               : "memory");
  a.x[0] = __uint_as_float(r0);
  a.x[1] = __uint_as_float(r1);
  a.x[2] = __uint_as_float(r2);
  a.x[3] = __uint_as_float(r3);
  b.x[0] = __uint_as_float(r4);
  b.x[1] = __uint_as_float(r5);
  b.x[2] = __uint_as_float(r6);
  b.x[3] = __uint_as_float(r7);
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// kLansVecs vectors of four values each, to / from 4 * kLansVecs consecutive columns
__device__ __forceinline__ void tmem_st_vecs(uint32_t taddr, const F4 (&a)[kLansVecs]) {
#pragma unroll
  for (int i = 0; i < kLansVecs; i += 2) tmem_st8(taddr + 4 * i, a[i], a[i + 1]);
}
__device__ __forceinline__ void tmem_ld_vecs(uint32_t taddr, F4 (&a)[kLansVecs]) {
#pragma unroll
  for (int i = 0; i < kLansVecs; i += 2) tmem_ld8(taddr + 4 * i, a[i], a[i + 1]);
}
constexpr uint32_t kCellColumns = 12 * kLansVecs;  // p, update_m, update_g of a thread's elements

// A parked chunk waits either in tensor memory (cells 0 .. kLansTmemCells-1; `taddr` = this
// warp's lanes, the cell's columns) or in a shared-memory cell (`scell`, three arrays of
// kLansElems floats; thread t of the group owns the 16 bytes at element q*512 + 4*t).
__device__ __forceinline__ void park_store(bool in_tmem, uint32_t taddr, unsigned char* scell, int gtid,
                                           const F4 (&rp)[kLansVecs], const F4 (&ua)[kLansVecs],
                                           const F4 (&ub)[kLansVecs]) {
  if (in_tmem) {
    tmem_st_vecs(taddr, rp);
    tmem_st_vecs(taddr + 4 * kLansVecs, ua);
    tmem_st_vecs(taddr + 8 * kLansVecs, ub);
  } else {
#pragma unroll
    for (int q = 0; q < kLansVecs; ++q) {
      float4* d = reinterpret_cast<float4*>(scell + (q * 512 + gtid * 4) * 4);
      d[0] = make_float4(rp[q].x[0], rp[q].x[1], rp[q].x[2], rp[q].x[3]);
      d[kLansElems / 4] = make_float4(ua[q].x[0], ua[q].x[1], ua[q].x[2], ua[q].x[3]);
      d[2 * (kLansElems / 4)] = make_float4(ub[q].x[0], ub[q].x[1], ub[q].x[2], ub[q].x[3]);
    }
  }
}
__device__ __forceinline__ void park_load(bool in_tmem, uint32_t taddr, const unsigned char* scell, int gtid,
                                          F4 (&rp)[kLansVecs], F4 (&ua)[kLansVecs], F4 (&ub)[kLansVecs]) {
  if (in_tmem) {
    tmem_ld_vecs(taddr, rp);
    tmem_ld_vecs(taddr + 4 * kLansVecs, ua);
    tmem_ld_vecs(taddr + 8 * kLansVecs, ub);
    tmem_wait_ld();
  } else {
#pragma unroll
    for (int q = 0; q < kLansVecs; ++q) {
      const float4* d = reinterpret_cast<const float4*>(scell + (q * 512 + gtid * 4) * 4);
      const float4 a = d[0], b = d[kLansElems / 4], c = d[2 * (kLansElems / 4)];
      rp[q].x[0] = a.x; rp[q].x[1] = a.y; rp[q].x[2] = a.z; rp[q].x[3] = a.w;
      ua[q].x[0] = b.x; ua[q].x[1] = b.y; ua[q].x[2] = b.z; ua[q].x[3] = b.w;
      ub[q].x[0] = c.x; ub[q].x[1] = c.y; ub[q].x[2] = c.z; ub[q].x[3] = c.w;
    }
  }
}

// Bounded wait on an mbarrier that also gives up as soon as any block has reported an
// error; a timeout reports `code` itself.
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, LansHeader* hdr,
                                          unsigned code, uint32_t where, uint64_t wait_ns) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  unsigned polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 15u) == 0) {
      if (*reinterpret_cast<volatile unsigned*>(&hdr->error) != 0) return false;
      if (global_ns() - t0 > wait_ns) {
        if (atomicCAS(&hdr->error, 0u, code) == 0u) hdr->error_item = where;
        return false;
      }
    }
  }
  return true;
}


// ---- kernel geometry ---------------------------------------------------------------
constexpr int kGroups = 4;                       // consumer groups per block
constexpr int kGroupThreads = 128;               // four warps
constexpr int kConsumerWarps = kGroups * 4;      // 16
constexpr int kPrefWarp = kConsumerWarps;        // 16, 17: resolve the block's items ahead of their use
constexpr int kParkWarp = kConsumerWarps + 2;    // 18: finishes parked chunks
constexpr int kPubWarp = kConsumerWarps + 3;     // 19: adds partial sums to the tensors' accumulators
constexpr int kLansThreads = (kConsumerWarps + 4) * 32;  // 640
constexpr int kQueueDepth = 64;                  // > slots per group + parked cells + end marker
constexpr int kMail = 64;                        // mailboxes of a block: kMailboxes per slot
constexpr uint32_t kMbEmpty = 0, kMbFull = 1, kMbTaking = 2, kMbIdle = 3;
constexpr uint32_t kSeqBits = 11, kSeqMask = (1u << kSeqBits) - 1u;  // see partition_lans_items
constexpr int kBVecs = kLansElems / (kGroupThreads * kVec);  // 2 vectors per thread per chunk
static_assert(kBVecs * kGroupThreads * kVec == kLansElems, "a chunk is whole passes of a group");

// A resolved work item: everything a group needs to run it.  The same 64 bytes serve as
// mailbox entry and as the description of what a slot currently holds.
struct __align__(16) SlotMeta {
  const void* g;  // global addresses of the item's first element (stores, unaligned fallback)
  float* p;
  float* m;
  float* v;
  void* out;
  uint32_t n_nbulk;    // bits 12..0 elements; 25..13 leading elements delivered by bulk copy;
                       // 31..26 tensor-memory cell of a parked item
  uint32_t tensor_op;  // bits 29..0 tensor, bits 31..30 first operation (kOpA, kOpB, kOpBP, kOpC)
  uint32_t nparts;     // arrivals that complete the norm(s) this item adds to
  float cs;            // gradient multiplier  grad_scale / (||g|| + eps)
  float ratio_m;       // -beta1 * lr * ||p|| / ||update_m||   (kOpC)
  float ratio_g;       // -beta3 * lr * ||p|| / ||update_g||
};
static_assert(sizeof(SlotMeta) == 64, "SlotMeta is 64 bytes");

struct __align__(16) RedSlot {
  float val[3][4];  // per warp of the group: sums of squares of this item
  uint32_t tensor;
  uint32_t is_a;    // 1: ||g||^2 ; 0: ||p||^2, ||update_m||^2, ||update_g||^2
  uint32_t nparts;
  uint32_t pad_;
};
static_assert(sizeof(RedSlot) == 64, "RedSlot is 64 bytes");

// Block-wide control words in shared memory.
struct LansCtrl {
  uint32_t done_items;  // items of this block that have finished
  uint32_t mb_state[64]; // mailbox kMailboxes * slot + round % kMailboxes, see kMb*
  uint32_t tail[kGroups];
  uint32_t item_cnt[16], pub_cnt[16], op_cnt[16];  // per slot: parities of its barriers
  uint32_t cell_free;    // cells nobody holds
  uint32_t cell_parked;  // cells whose chunk waits for its tensor's norms
  uint32_t tmem_base;    // address the allocation returned
  uint32_t cellop_cnt[32], cell_grp[32];  // per cell: parity of its barrier, group that parked it
};

// What the second half of a parked item needs: where p and the parameter copy go.
struct __align__(16) CellMeta {
  float* p;
  void* out;
  uint32_t n_nbulk;
  uint32_t tensor;
  uint32_t pad_[2];
};
static_assert(sizeof(CellMeta) == 32, "CellMeta is 32 bytes");

template <typename GT>
struct LansGeo {
  static constexpr int kGBytes = kLansElems * (int)sizeof(GT);
  static constexpr int kFBytes = kLansElems * 4;
  static constexpr int kSlotBytes = kGBytes + 3 * kFBytes;  // 14336 (16-bit g) | 16384 (fp32 g)
  static constexpr int kAElems = sizeof(GT) == 2 ? kLansAElems16 : kLansAElems32;
  static constexpr int kSlots = sizeof(GT) == 2 ? kLansSlots16 : kLansSlots32;
  static_assert(kAElems * (int)sizeof(GT) <= kSlotBytes, "an A item fits a slot");
  // a prefetcher warp gives each slot of its parity 32 / (slots of a parity, rounded up to a
  // power of two) lanes = mailboxes
  static constexpr int kJBits = kSlots <= 8 ? 2 : 3;
  static constexpr uint32_t kMailboxes = 32u >> kJBits;
  static_assert(kSlots <= 16 && kSlots * (int)kMailboxes <= kMail && kLansCells <= 31, "per-slot tables and masks");
  static constexpr int kSmemCellBytes = 3 * kFBytes;  // p, update_m, update_g
  static constexpr int kSmemCellOff = kSlots * kSlotBytes;
  static constexpr int kMetaOff = kSmemCellOff + kLansSmemCells * kSmemCellBytes;
  static constexpr int kMailOff = kMetaOff + kSlots * (int)sizeof(SlotMeta);
  static constexpr int kRedOff = kMailOff + kMail * (int)sizeof(SlotMeta);
  static constexpr int kQueueOff = kRedOff + kSlots * (int)sizeof(RedSlot);
  static constexpr int kCellOff = kQueueOff + kGroups * kQueueDepth * 16;
  static constexpr int kCtrlOff = kCellOff + kLansCells * (int)sizeof(CellMeta);
  static constexpr int kBarOff = (kCtrlOff + (int)sizeof(LansCtrl) + 15) & ~15;
  // barriers: data, done, redfull, redempty per slot; queue entries; end of consumers; per cell
  static constexpr int kNumBars = 4 * kSlots + kGroups * kQueueDepth + 1 + kLansCells;
  static constexpr int kTotal = kBarOff + kNumBars * 8;
  static_assert(kTotal <= 232448, "fits the 227 KB of shared memory a block may use");
};

__device__ __forceinline__ uint32_t ld_shared_volatile(const uint32_t* p) {
  return *reinterpret_cast<const volatile uint32_t*>(p);
}

// FUSED: the instantiation with the collectives inside (LansParams::fuse_rs / fuse_ag); the
// plain one carries none of that code.
template <typename GT, typename OT, bool FUSED>
__global__ void __launch_bounds__(kLansThreads, 1) lans_kernel(const LansParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  using L = LansGeo<GT>;
  constexpr int S = L::kSlots;
  constexpr uint32_t kMailboxes = L::kMailboxes;
  SlotMeta* s_meta = reinterpret_cast<SlotMeta*>(smem + L::kMetaOff);
  SlotMeta* s_mail = reinterpret_cast<SlotMeta*>(smem + L::kMailOff);
  RedSlot* s_red = reinterpret_cast<RedSlot*>(smem + L::kRedOff);
  uint4* s_queue = reinterpret_cast<uint4*>(smem + L::kQueueOff);
  LansCtrl* ctrl = reinterpret_cast<LansCtrl*>(smem + L::kCtrlOff);
  const uint32_t bar_data = smem_u32(smem + L::kBarOff);
  const uint32_t bar_done = bar_data + S * 8;
  const uint32_t bar_redfull = bar_done + S * 8;
  const uint32_t bar_redempty = bar_redfull + S * 8;
  const uint32_t bar_queue = bar_redempty + S * 8;
  const uint32_t bar_end = bar_queue + kGroups * kQueueDepth * 8;
  const uint32_t bar_cell = bar_end + 8;
  const uint32_t data_base = smem_u32(smem);
  CellMeta* s_cell = reinterpret_cast<CellMeta*>(smem + L::kCellOff);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  // two lists per block: the entries of its even slots and of its odd slots
  const uint32_t n_list = P.block_off[2 * blockIdx.x + 2] - P.block_off[2 * blockIdx.x];
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_data + 8 * s, 1);      // whoever starts the item (+ transaction bytes)
      mbar_init(bar_done + 8 * s, 4);      // the four warps of the slot's group
      mbar_init(bar_redfull + 8 * s, 4);
      mbar_init(bar_redempty + 8 * s, 1);  // the publisher
    }
    for (int q = 0; q < kGroups * kQueueDepth; ++q) mbar_init(bar_queue + 8 * q, 1);
    mbar_init(bar_end, kConsumerWarps);
    for (int c = 0; c < kLansCells; ++c) mbar_init(bar_cell + 8 * c, 4);
    memset(ctrl, 0, sizeof(LansCtrl));
    for (int q = 0; q < S; ++q) ctrl->mb_state[kMailboxes * q] = kMbIdle;  // every slot waits for its first item
    ctrl->cell_free = (1u << kLansCells) - 1u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Tensor memory (256 KB per SM, otherwise unused by this kernel) holds the parked chunks.
  // The parker warp allocates all 512 columns and gives them back before it leaves.
  if (warp == kParkWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctrl->tmem_base)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = ctrl->tmem_base;

  LansStage1 s1 = P.s1;
  if (P.step_dev != nullptr) {  // bias corrections were computed on the device, see above
    s1.inv_bc1 = __ldcg(&P.hdr->inv_bc1);
    s1.inv_bc2 = __ldcg(&P.hdr->inv_bc2);
  }
  const uint64_t pol_keep = make_policy_keep(), pol_stream = make_policy_stream();

  // Hands one entry of a group's queue to that group.  Called by a single thread.
  // `slot` is a shared-memory slot, or - for kOpCP - a tensor-memory cell.
  auto push_op = [&](uint32_t slot, uint32_t op, uint32_t dpar, uint32_t rpar, float cs, float rm, float rg) {
    const uint32_t grp = (op == kOpCP) ? ld_shared_volatile(&ctrl->cell_grp[slot]) : (slot & 3u);
    const uint32_t opar = atomicAdd(op == kOpCP ? &ctrl->cellop_cnt[slot] : &ctrl->op_cnt[slot], 1u) & 1u;
    const uint32_t tail = atomicAdd(&ctrl->tail[grp], 1u);
    const uint32_t qi = grp * kQueueDepth + (tail % kQueueDepth);
    s_queue[qi] = make_uint4(op | (slot << 3) | (dpar << 8) | (rpar << 9) | (opar << 10), __float_as_uint(cs),
                             __float_as_uint(rm), __float_as_uint(rg));
    mbar_arrive(bar_queue + 8 * qi);
  };
  // Every slot has two mailboxes for its next items (rounds of the slot alternate between
  // them), filled by the prefetcher.  A mailbox is EMPTY, FULL, being TAKEN, or the slot sits
  // IDLE in front of it: then whoever fills it starts the item himself.
  //
  // Starts the item in mailbox `h` of slot `slot`: copies it into the slot's description,
  // issues the bulk copies and queues the item's first operation.  Called by a single thread.
  auto start_from_mailbox = [&](uint32_t slot, uint32_t h) {
    const uint4* src = reinterpret_cast<const uint4*>(&s_mail[kMailboxes * slot + h]);
    uint4* dst = reinterpret_cast<uint4*>(&s_meta[slot]);
    const uint4 e0 = src[0], e1 = src[1], e2 = src[2], e3 = src[3];
    dst[0] = e0;
    dst[1] = e1;
    dst[2] = e2;
    dst[3] = e3;
    __threadfence_block();
    *reinterpret_cast<volatile uint32_t*>(&ctrl->mb_state[kMailboxes * slot + h]) = kMbEmpty;
    const uint32_t op = e2.w >> 30, nbulk = (e2.z >> kLansNBits) & ((1u << kLansNBits) - 1u);
    const uint32_t dpar = atomicAdd(&ctrl->item_cnt[slot], 1u) & 1u;
    const uint32_t my_data = bar_data + 8 * slot;
    if (nbulk > 0) {
      const char* gsrc = reinterpret_cast<const char*>(((uint64_t)e0.y << 32) | e0.x);
      const char* psrc = reinterpret_cast<const char*>(((uint64_t)e0.w << 32) | e0.z);
      const char* msrc = reinterpret_cast<const char*>(((uint64_t)e1.y << 32) | e1.x);
      const char* vsrc = reinterpret_cast<const char*>(((uint64_t)e1.w << 32) | e1.z);
      const uint32_t gb = nbulk * (uint32_t)sizeof(GT), fb = nbulk * 4u;
      const uint32_t dstaddr = data_base + slot * L::kSlotBytes;
      if (op == kOpA) {
        mbar_arrive_expect_tx(my_data, gb);
        tma_load_1d(dstaddr, gsrc, gb, my_data, pol_keep);  // stage 1 reads it again soon
      } else {
        mbar_arrive_expect_tx(my_data, gb + 3u * fb);
        // a streamed chunk is read once more by its update item soon after: keep it in L2;
        // a parked chunk and the update item's own reads are the last use of the lines
        const uint64_t pol = (op == kOpB) ? pol_keep : pol_stream;
        tma_load_1d(dstaddr, gsrc, gb, my_data, pol);
        tma_load_1d(dstaddr + L::kGBytes, psrc, fb, my_data, pol);
        tma_load_1d(dstaddr + L::kGBytes + L::kFBytes, msrc, fb, my_data, pol);
        tma_load_1d(dstaddr + L::kGBytes + 2 * L::kFBytes, vsrc, fb, my_data, pol);
      }
    } else {
      mbar_arrive(my_data);
    }
    uint32_t rpar = 0;
    if (op != kOpC) rpar = atomicAdd(&ctrl->pub_cnt[slot], 1u) & 1u;
    if (op == kOpBP) rpar |= (atomicAdd(&ctrl->cellop_cnt[e2.z >> (2 * kLansNBits)], 1u) & 1u) << 2;  // lands in bit 11
    push_op(slot, op, dpar, rpar, __uint_as_float(e3.y), __uint_as_float(e3.z), __uint_as_float(e3.w));
  };
  // The slot has run empty: take its next item if the prefetcher has it ready, else leave
  // word that the slot is idle.  Called by a single thread that owns the slot.
  auto take_next = [&](uint32_t slot) {
    const uint32_t h = ld_shared_volatile(&ctrl->item_cnt[slot]) % kMailboxes;
    uint32_t* stp = &ctrl->mb_state[kMailboxes * slot + h];
    uint32_t old = atomicCAS(stp, kMbFull, kMbTaking);
    if (old != kMbFull) {
      old = atomicCAS(stp, kMbEmpty, kMbIdle);
      if (old == kMbFull) old = atomicCAS(stp, kMbFull, kMbTaking);
    }
    if (old == kMbFull) start_from_mailbox(slot, h);
  };

  if (warp == kPrefWarp || warp == kPrefWarp + 1) {
    // =============================== prefetcher ===============================
    // The even slots of a block share one list, the odd slots another; the j-th slot of a
    // parity with S_h slots runs the entries j, j + S_h, j + 2 S_h, ... of its list.  Eight lanes
    // prepare them in turn (round r goes to mailbox r % 8): item -> descriptor of its tensor (kept
    // while the tensor stays the same) -> the norms the item's first operation needs are
    // final -> a tensor-memory cell if the item parks -> the slot's mailbox.
    enum : uint32_t { F_ITEM, F_DESC, F_NORM, F_CELL, F_WRITE, F_DONE };
    // Two warps: warp w serves the slots s with s % 2 == w, kMailboxes lanes per slot,
    // and hands out its own half of the tensor-memory cells.
    const uint32_t pw = (uint32_t)(warp - kPrefWarp);
    constexpr uint32_t kJMask = (1u << L::kJBits) - 1u;
    const uint32_t slot = 2u * ((uint32_t)lane & kJMask) + pw, half = (uint32_t)lane >> L::kJBits;
    const uint32_t my_cells = pw == 0 ? ((1u << ((kLansCells + 1) / 2)) - 1u)
                                      : (((1u << kLansCells) - 1u) & ~((1u << ((kLansCells + 1) / 2)) - 1u));
    const uint32_t list_lo = P.block_off[2 * blockIdx.x + pw];
    const uint32_t my_n = P.block_off[2 * blockIdx.x + pw + 1] - list_lo;
    const uint32_t S_h = ((uint32_t)S + 1u - pw) / 2u;  // slots of my parity
    uint32_t e = ((uint32_t)lane & kJMask) + S_h * half;  // my entry of the list
    uint32_t st = (slot < (uint32_t)S && e < my_n) ? (uint32_t)F_ITEM : (uint32_t)F_DONE;
    uint32_t tp = 0, chunk = 0, seq = 0, my_t = 0xffffffffu, my_cell = 0;
    uint4 d0 = make_uint4(0, 0, 0, 0), d1 = d0, d2 = d0, d3 = d0, nrm = d0;
    bool have_g = false, have_n = false;
    float cs = s1.gscale, rm = 0.f, rg = 0.f;
    uint64_t t_enter = 0;
    const bool normalize = s1.normalize != 0;
    int failed = 0;
    uint32_t g_base = 0, g_mask = 0;
    for (uint32_t iter = 1;; ++iter) {
      const uint32_t st_in = st;
      // ---- global requests of this iteration, all issued before any is used ----
      uint2 it = make_uint2(0, 0);
      if (st_in == F_ITEM) it = ld_global_v2(P.items + list_lo + e);
      if (st_in == F_DESC) {
        const char* src = reinterpret_cast<const char*>(P.descs + my_t);
        d0 = ld_global_v4(src);
        d1 = ld_global_v4(src + 16);
        d2 = ld_global_v4(src + 32);
        d3 = ld_global_v4(src + 48);
      }
      const bool poll = st_in == F_DESC || st_in == F_NORM;
      // lanes that wait for the same tensor share one load of its norm words
      const unsigned same_t = __match_any_sync(0xffffffffu, poll ? my_t : (0x80000000u | (uint32_t)lane));
      const int poll_leader = __ffs(same_t) - 1;
      uint4 nrm_new = make_uint4(0, 0, 0, 0);
      if (poll && poll_leader == lane) nrm_new = ld_norms(P.ctl + my_t);
      // ---- consume ----
      nrm_new.x = __shfl_sync(0xffffffffu, nrm_new.x, poll_leader);
      nrm_new.y = __shfl_sync(0xffffffffu, nrm_new.y, poll_leader);
      nrm_new.z = __shfl_sync(0xffffffffu, nrm_new.z, poll_leader);
      nrm_new.w = __shfl_sync(0xffffffffu, nrm_new.w, poll_leader);
      if (poll) {
        nrm = nrm_new;
        if (!have_g && (nrm.x >> 31)) {
          have_g = true;
          cs = s1.grad_multiplier(norm_value(nrm.x));
        }
        if (!have_n && ((nrm.y & nrm.z & nrm.w) >> 31)) {  // multi_tensor_lans.cu:347-353
          have_n = true;
          const float pn = norm_value(nrm.y), umn = norm_value(nrm.z), ugn = norm_value(nrm.w);
          const float a = (umn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, umn)) : P.lr;
          const float b2 = (ugn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, ugn)) : P.lr;
          rm = -mul(a, s1.beta1);
          rg = -mul(b2, s1.beta3);
        }
      }
      if (st_in == F_ITEM) {
        tp = it.x;
        chunk = it.y & ((1u << (32 - kSeqBits)) - 1u);
        seq = it.y >> (32 - kSeqBits);
        const uint32_t t = tp & kTensorMask;
        if (t != my_t) {
          my_t = t;
          have_g = have_n = false;
          cs = s1.gscale;
          st = F_DESC;
        } else {
          st = F_NORM;
        }
      } else if (st_in == F_DESC) {
        st = F_NORM;
      }
      const uint32_t kind = tp >> kPhaseShift;
      if (st == F_NORM) {
        const bool need_g = normalize && kind != kKindA;
        const bool need_n = kind == kKindCs;
        if ((!need_g || have_g) && (!need_n || have_n)) st = (kind == kKindBCp) ? (uint32_t)F_CELL : (uint32_t)F_WRITE;
      }
      // ---- tensor-memory cells ----
      // `seq` numbers the parked items of this block in list order.  An item may take a cell
      // out of turn as long as a free cell remains for every earlier item that has none yet:
      // then no item ever holds a cell that an earlier one is waiting for.  g_base = lowest
      // number without a cell, bit i of g_mask = number g_base + i has one (warp-uniform).
      {
        const uint32_t off = (seq - g_base) & kSeqMask;
        const bool asks = st == F_CELL && off < 32u;
        uint32_t cand = asks ? (1u << off) : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand |= __shfl_xor_sync(0xffffffffu, cand, o);
        uint32_t free_cells = 0;
        if (lane == 0) free_cells = ld_shared_volatile(&ctrl->cell_free) & my_cells;
        free_cells = __shfl_sync(0xffffffffu, free_cells, 0);
        uint32_t nfree = (uint32_t)__popc(free_cells), newly = 0;
        for (uint32_t c = cand; c != 0 && nfree > 0; c &= c - 1u) {
          const uint32_t o = (uint32_t)__ffs(c) - 1u;
          const uint32_t earlier_without = o - (uint32_t)__popc((g_mask | newly) & ((1u << o) - 1u));
          if (nfree - 1u < earlier_without) break;  // later numbers have at least as many before them
          newly |= 1u << o;
          --nfree;
        }
        if (newly) {
          if (asks && ((newly >> off) & 1u)) {
            my_cell = __fns(free_cells, 0, __popc(newly & ((1u << off) - 1u)) + 1);
            st = F_WRITE;
          }
          uint32_t taken = (st == F_WRITE && asks && ((newly >> off) & 1u)) ? (1u << my_cell) : 0u;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) taken |= __shfl_xor_sync(0xffffffffu, taken, o);
          if (lane == 0) atomicAnd(&ctrl->cell_free, ~taken);
          g_mask |= newly;
          while (g_mask & 1u) {
            g_mask >>= 1;
            ++g_base;
          }
          __syncwarp();
        }
      }
      // ---- hand the item to its slot ----
      if (st == F_WRITE) {
        const uint32_t mb = kMailboxes * slot + half;
        const uint32_t mbs = ld_shared_volatile(&ctrl->mb_state[mb]);
        if (mbs == kMbEmpty || mbs == kMbIdle) {
          const char* dg = reinterpret_cast<const char*>(((uint64_t)d0.y << 32) | d0.x);
          float* dp = reinterpret_cast<float*>(((uint64_t)d0.w << 32) | d0.z);
          float* dm = reinterpret_cast<float*>(((uint64_t)d1.y << 32) | d1.x);
          float* dv = reinterpret_cast<float*>(((uint64_t)d1.w << 32) | d1.z);
          char* dout = reinterpret_cast<char*>(((uint64_t)d2.y << 32) | d2.x);
          const int64_t numel = (int64_t)(((uint64_t)d2.w << 32) | d2.z);
          const uint32_t flags = d3.z;
          const int per = (kind == kKindA) ? L::kAElems : kLansElems;
          const int64_t start = (int64_t)chunk * per;
          const int64_t left = numel - start;
          const int n = left < per ? (int)left : per;
          constexpr int gran = 16 / (int)sizeof(GT);  // elements per 16 bytes of gradient
          const bool through_switch = FUSED && kind == kKindA && P.fuse_rs != 0;
          const int nbulk = ((flags & kFlagBulk) && !through_switch) ? (n / gran) * gran : 0;
          const uint32_t op = kind == kKindA ? kOpA : kind == kKindBs ? kOpB : kind == kKindCs ? kOpC : kOpBP;
          SlotMeta& mt = s_mail[mb];
          mt.g = dg + start * (int64_t)sizeof(GT);
          // an A item that reads through the switch gets the byte offset of its chunk inside the
          // symmetric gradient buffer instead of p, which it does not use
          mt.p = through_switch ? reinterpret_cast<float*>((((uint64_t)d3.y << 32) | d3.x) + (uint64_t)start * sizeof(GT))
                                : dp + start;
          mt.m = dm + start;
          mt.v = dv + start;
          mt.out = dout ? dout + start * (int64_t)sizeof(OT) : nullptr;
          mt.n_nbulk = (uint32_t)n | ((uint32_t)nbulk << kLansNBits) | ((op == kOpBP ? my_cell : 0u) << (2 * kLansNBits));
          mt.tensor_op = my_t | (op << 30);
          mt.nparts = (uint32_t)((numel + per - 1) / per);
          mt.cs = (op == kOpA) ? s1.gscale : cs;
          mt.ratio_m = rm;
          mt.ratio_g = rg;
          if (op == kOpBP) {
            CellMeta& cm = s_cell[my_cell];
            cm.p = dp + start;
            cm.out = mt.out;
            cm.n_nbulk = (uint32_t)n | ((uint32_t)nbulk << kLansNBits);
            cm.tensor = my_t;
          }
          __threadfence_block();
          if (atomicCAS(&ctrl->mb_state[mb], kMbEmpty, kMbFull) == kMbIdle) {
            // the slot has been waiting for this item: start it from here
            *reinterpret_cast<volatile uint32_t*>(&ctrl->mb_state[mb]) = kMbTaking;
            start_from_mailbox(slot, half);
          }
          e += kMailboxes * S_h;
          st = e < my_n ? (uint32_t)F_ITEM : (uint32_t)F_DONE;
        }
      }
      if (st != st_in) t_enter = 0;
      // ---- bounded waits, errors, end ----
      if ((iter & 31u) == 0) {
        const uint64_t now = global_ns();
        if (st == F_NORM || st == F_CELL) {
          if (t_enter == 0) {
            t_enter = now;
          } else if (now - t_enter > P.wait_ns) {
            if (atomicCAS(&P.hdr->error, 0u, (kind == kKindCs || st == F_CELL) ? kErrWaitN : kErrWaitG) == 0u)
              P.hdr->error_item = list_lo + e;
          }
        }
        if (*reinterpret_cast<volatile unsigned*>(&P.hdr->error) != 0) failed = 1;
      }
      if (__all_sync(0xffffffffu, st == F_DONE) || __any_sync(0xffffffffu, failed != 0)) break;
      if (!__any_sync(0xffffffffu, st != st_in)) __nanosleep(100);
    }
    return;
  }

  if (warp == kParkWarp) {
    // ================================= parker =================================
    // Lane c looks after cell c: queues the second half of the chunk parked there when the
    // tensor's norms are final.
    const bool active = lane < S;
    const uint32_t bit = 1u << lane;
    uint64_t t_parked = 0;
    int failed = 0;
    for (uint32_t iter = 1;; ++iter) {
      const uint32_t parked_mask = ld_shared_volatile(&ctrl->cell_parked);
      const bool parked = lane < kLansCells && (parked_mask & bit);
      uint32_t my_t = 0x80000000u | (uint32_t)lane;
      if (parked) my_t = s_cell[lane].tensor;
      const unsigned same_t = __match_any_sync(0xffffffffu, my_t);
      const int leader = __ffs(same_t) - 1;
      uint4 nrm = make_uint4(0, 0, 0, 0);
      if (parked && leader == lane) nrm = ld_norms(P.ctl + my_t);
      nrm.y = __shfl_sync(0xffffffffu, nrm.y, leader);
      nrm.z = __shfl_sync(0xffffffffu, nrm.z, leader);
      nrm.w = __shfl_sync(0xffffffffu, nrm.w, leader);
      if (parked && ((nrm.y & nrm.z & nrm.w) >> 31)) {  // multi_tensor_lans.cu:347-353
        const float pn = norm_value(nrm.y), umn = norm_value(nrm.z), ugn = norm_value(nrm.w);
        const float a = (umn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, umn)) : P.lr;
        const float b2 = (ugn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, ugn)) : P.lr;
        atomicAnd(&ctrl->cell_parked, ~bit);
        push_op((uint32_t)lane, kOpCP, 0, 0, 0.f, -mul(a, s1.beta1), -mul(b2, s1.beta3));
        t_parked = 0;
      }
      __syncwarp();
      const bool all_done = ld_shared_volatile(&ctrl->done_items) >= n_list;
      if ((iter & 31u) == 0) {
        const uint64_t now = global_ns();
        if (parked) {
          if (t_parked == 0) {
            t_parked = now;
          } else if (now - t_parked > P.wait_ns) {
            if (atomicCAS(&P.hdr->error, 0u, kErrWaitN) == 0u) P.hdr->error_item = 0x80000000u | my_t;
          }
        }
        if (*reinterpret_cast<volatile unsigned*>(&P.hdr->error) != 0) failed = 1;
      }
      if (all_done || __any_sync(0xffffffffu, failed != 0)) break;
      if (parked_mask == 0) __nanosleep(200);
    }
    // every group gets its end marker; then nothing of this block may still be in flight
    if (lane < kGroups) {
      const uint32_t tail = atomicAdd(&ctrl->tail[lane], 1u);
      const uint32_t qi = (uint32_t)lane * kQueueDepth + (tail % kQueueDepth);
      s_queue[qi] = make_uint4(kOpEnd, 0, 0, 0);
      mbar_arrive(bar_queue + 8 * qi);
    }
    ring_wait(bar_end, 0, P.hdr, kErrRing, 0x3000u, P.wait_ns);
    if (active) {
      const uint32_t items = ld_shared_volatile(&ctrl->item_cnt[lane]);
      if (items > 0) ring_wait(bar_data + 8 * lane, (items - 1u) & 1u, P.hdr, kErrData, (uint32_t)lane, P.wait_ns);
    }
    // every consumer warp has left (or the bounded wait above gave up): give the tensor
    // memory back
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    return;
  }

  if (warp == kPubWarp) {
    // =============================== publisher ===============================
    const bool active = lane < S;
    uint32_t n_seen = 0;  // publications of this lane's slot read so far
    for (;;) {
      const bool end = mbar_test(bar_end, 0);  // every consumer warp has left (checked first)
      const bool ready = active && mbar_test(bar_redfull + 8 * lane, n_seen & 1u);
      double q0 = 0.0, q1 = 0.0, q2 = 0.0;
      uint32_t key = 0xffffffffu, nparts = 0;
      if (ready) {
        const RedSlot& rs = s_red[lane];
        q0 = (double)rs.val[0][0] + (double)rs.val[0][1] + (double)rs.val[0][2] + (double)rs.val[0][3];
        q1 = (double)rs.val[1][0] + (double)rs.val[1][1] + (double)rs.val[1][2] + (double)rs.val[1][3];
        q2 = (double)rs.val[2][0] + (double)rs.val[2][1] + (double)rs.val[2][2] + (double)rs.val[2][3];
        key = (rs.tensor << 1) | (rs.is_a & 1u);
        nparts = rs.nparts;
        mbar_arrive(bar_redempty + 8 * lane);  // the slot has been read
        ++n_seen;
      }
      unsigned pending = __ballot_sync(0xffffffffu, ready);
      if (pending == 0) {
        if (end) break;
        __nanosleep(64);
        continue;
      }
      // Items of the same tensor and kind that completed since the last look go out as one
      // update of the tensor's accumulators (the lowest of their lanes does it), and all such
      // groups go out at the same time: one pair of round trips to L2 per look, however many
      // tensors the block has chunks of.
      const unsigned same = __match_any_sync(0xffffffffu, ready ? key : (0x80000000u | (uint32_t)lane));
      const bool leads = ready && (__ffs(same) - 1) == lane;
      double a0 = 0.0, a1 = 0.0, a2 = 0.0;
#pragma unroll
      for (int l = 0; l < S; ++l) {
        const double b0 = __shfl_sync(0xffffffffu, q0, l), b1 = __shfl_sync(0xffffffffu, q1, l),
                     b2 = __shfl_sync(0xffffffffu, q2, l);
        const double w = (double)((same >> l) & 1u);  // 1.0 for the lanes of this group, else 0.0
        a0 = fma(b0, w, a0);
        a1 = fma(b1, w, a1);
        a2 = fma(b2, w, a2);
      }
      if (leads) {
        const bool is_a = (key & 1u) != 0;
        LansCtl* ctl = P.ctl + (key >> 1);
        // A -> ||g||^2 ; B -> ||p||^2, ||update_m||^2, ||update_g||^2
        if (is_a) {
          atomicAdd(&ctl->sumsq[0], a0);
        } else {
          atomicAdd(&ctl->sumsq[1], a0);
          atomicAdd(&ctl->sumsq[2], a1);
          atomicAdd(&ctl->sumsq[3], a2);
        }
        __threadfence();
        const unsigned cnt = (unsigned)__popc(same);
        const unsigned old = atomicAdd(is_a ? &ctl->arrived_a : &ctl->arrived_b, cnt);
        if (old + cnt == nparts) {
          // Every part of the tensor has been added: publish the norm(s), value and
          // "final" bit in one word each.
          __threadfence();
          for (int w = is_a ? 0 : 1; w < (is_a ? 1 : 4); ++w) {
            const double total = *reinterpret_cast<volatile double*>(&ctl->sumsq[w]);
            *reinterpret_cast<volatile unsigned*>(&ctl->norm[w]) =
                __float_as_uint(sqrtf((float)total)) | kNormValid;
          }
        }
      }
      __syncwarp();
    }
    return;
  }

  // ================================ consumers ================================
  // Thread `gtid` of a group owns, in every chunk, the vectors of four elements at
  // q*512 + 4*gtid: 16-byte shared-memory accesses without bank conflicts, coalesced
  // 16-byte stores.  Lanes past the end of a ragged chunk hold zeros, which add nothing
  // to any sum.  One warp of the group (they take turns) also turns the slot over when an
  // item's last operation is done: it starts the slot's next item from its mailbox right away.
  const int grp = warp >> 2, wig = warp & 3, gtid = tid & (kGroupThreads - 1);
  Policies pol;
  pol.init();
  // the model-dtype copy: a local store, or - with the all-gather inside the kernel - a store
  // into every rank's parameter buffer
  auto put_out4 = [&](OT* dst, const F4& v) {
    if (FUSED && P.fuse_ag) store_out_everywhere<OT>(P, dst, v);
    else Elem<OT>::template store4<kStream>(dst, v, pol);
  };
  auto put_out1 = [&](OT* dst, float x) {
    if (FUSED && P.fuse_ag) store_out_everywhere1<OT>(P, dst, x);
    else *dst = Elem<OT>::from_f32(x);
  };
  for (uint32_t i = 0;; ++i) {
    const uint32_t qi = (uint32_t)grp * kQueueDepth + (i % kQueueDepth);
    bool ok = ring_wait(bar_queue + 8 * qi, (i / kQueueDepth) & 1u, P.hdr, kErrRing, 0x1000u | (uint32_t)grp,
                        P.wait_ns);
    if (!__all_sync(0xffffffffu, ok)) break;  // every lane of the warp leaves, or none
    const uint4 ent = s_queue[qi];
    const uint32_t op = ent.x & 7u, slot = (ent.x >> 3) & 31u, dpar = (ent.x >> 8) & 1u, rpar = (ent.x >> 9) & 1u,
                   opar = (ent.x >> 10) & 1u, cpar = (ent.x >> 11) & 1u;
    if (op == kOpEnd) break;
    const float cs = __uint_as_float(ent.y), ratio_m = __uint_as_float(ent.z), ratio_g = __uint_as_float(ent.w);
    // kOpCP names a tensor-memory cell, every other operation a shared-memory slot
    SlotMeta mt = s_meta[op == kOpCP ? 0u : slot];
    uint32_t cell = mt.n_nbulk >> (2 * kLansNBits);
    if (op == kOpCP) {
      const CellMeta cm = s_cell[slot];
      mt.p = cm.p;
      mt.out = cm.out;
      mt.n_nbulk = cm.n_nbulk;
      cell = slot;
    }
    const int n = (int)(mt.n_nbulk & ((1u << kLansNBits) - 1u)),
              nbulk = (int)((mt.n_nbulk >> kLansNBits) & ((1u << kLansNBits) - 1u));
    const GT* gg = static_cast<const GT*>(mt.g);
    float* gp = mt.p;
    float* gm = mt.m;
    float* gv = mt.v;
    OT* gout = static_cast<OT*>(mt.out);
    unsigned char* sbase = smem + slot * L::kSlotBytes;
    const uint32_t my_done = (op == kOpCP) ? bar_cell + 8 * slot : bar_done + 8 * slot;
    // this warp's quarter of the cell: lanes 32 * wig ..., columns 24 * cell ...
    const bool in_tmem = cell < (uint32_t)kLansTmemCells;
    const uint32_t taddr = tmem_base + ((uint32_t)(32 * wig) << 16) + kCellColumns * (in_tmem ? cell : 0u);
    unsigned char* scell = smem + L::kSmemCellOff + (in_tmem ? 0 : (int)(cell - kLansTmemCells)) * L::kSmemCellBytes;
    if (op != kOpCP) {  // first use of the slot's data: wait for the copies
      ok = ring_wait(bar_data + 8 * slot, dpar, P.hdr, kErrData, slot, P.wait_ns);
      if (!__all_sync(0xffffffffu, ok)) break;
    }
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
    bool publishes = false;

    // The common case - every element of the item arrived by bulk copy - runs as straight-line
    // code without per-vector tests; ragged or unaligned items take the general code below.
    // Both add an element's square into the same accumulator in the same order.
    const bool whole = nbulk == ((op == kOpA) ? L::kAElems : kLansElems);
    if (FUSED && op == kOpA && P.fuse_rs) {
      // Reduce-scatter inside the kernel: the chunk's sum over ranks, 16 bytes per access, in
      // fp32 with one rounding - written to the local gradient block for the later stages and
      // squared as written.  The symmetric layout pads every row block to 16 bytes with zeros,
      // so the last vector may run past n without harm.
      constexpr int kDT = sizeof(GT) == 4 ? RAFB200_F32 : (std::is_same<GT, __half>::value ? RAFB200_F16 : RAFB200_BF16);
      constexpr int kEV = 16 / (int)sizeof(GT);                 // elements per access
      constexpr int kAcc = L::kAElems / (kGroupThreads * kEV);  // accesses per thread: 7 | 8
      const size_t off = (size_t)reinterpret_cast<uintptr_t>(gp);
      char* dst = const_cast<char*>(reinterpret_cast<const char*>(gg));
      const int nvec = (n + kEV - 1) / kEV;
      if (lane == 0) mbar_arrive(my_done);  // nothing of the slot is used
      uint4 r[kAcc];
      if (P.g_mc) {
#pragma unroll
        for (int u = 0; u < kAcc; ++u) {
          const int i = gtid + u * kGroupThreads;
          r[u] = (i < nvec) ? mc_ld_reduce<kDT>(P.g_mc + off + (size_t)i * 16) : make_uint4(0, 0, 0, 0);
        }
      } else {
        // peer by peer in a fixed order; four accesses in flight per thread
#pragma unroll
        for (int u0 = 0; u0 < kAcc; u0 += 4) {
          float acc[4][8];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
          for (int q = 0; q < P.world; ++q) {
            uint4 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i = gtid + (u0 + u) * kGroupThreads;
              t[u] = (u0 + u < kAcc && i < nvec) ? peer_ld(P.g_peer[q] + off + (size_t)i * 16) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) accumulate<kDT>(acc[u], t[u]);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (u0 + u < kAcc) r[u0 + u] = round_once<kDT>(acc[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kAcc; ++u) {
        const int i = gtid + u * kGroupThreads;
        if (i >= nvec) continue;
        *reinterpret_cast<uint4*>(dst + (size_t)i * 16) = r[u];
        float sq[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        accumulate<kDT>(sq, r[u]);  // the rounded values, as stage 1 will read them
#pragma unroll
        for (int j = 0; j < (kEV < 8 ? kEV : 8); ++j) {
          const float x = sq[j] * s1.gscale;
          acc0 = fmaf(x, x, acc0);
        }
      }
      __threadfence();  // the block of another SM that waits for ||g|| reads these stores next
      publishes = true;
    } else if (__builtin_expect(!whole, 0)) {
      // ragged or unaligned items: kept out of the way of the straight-line code below
      if (op == kOpA) {
        constexpr int kPasses = L::kAElems / (kGroupThreads * kVec);
#pragma unroll 2
        for (int q = 0; q < kPasses; ++q) {
          const int e = q * (kGroupThreads * kVec) + gtid * kVec;
          F4 r;
          if (e < nbulk) {
            r = Elem<GT>::smem4(sbase + e * sizeof(GT));
          } else {
#pragma unroll
            for (int j = 0; j < kVec; ++j) r.x[j] = (e + j < n) ? Elem<GT>::to_f32(gg[e + j]) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            const float x = r.x[j] * s1.gscale;
            acc0 = fmaf(x, x, acc0);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(my_done);
        publishes = true;
      } else if (op == kOpCP) {
        // stage 2 from the parked chunk: p, update_m, update_g are in tensor memory
        F4 rp[kBVecs], um[kBVecs], ug[kBVecs];
        park_load(in_tmem, taddr, scell, gtid, rp, um, ug);
        __syncwarp();
        if (lane == 0) mbar_arrive(my_done);
#pragma unroll
        for (int q = 0; q < kBVecs; ++q) {
          const int e = q * (kGroupThreads * kVec) + gtid * kVec;
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            rp[q].x[j] = fmaf(ratio_g, ug[q].x[j], fmaf(ratio_m, um[q].x[j], rp[q].x[j]));
          if (e < nbulk) {
            Elem<float>::template store4<kStream>(gp + e, rp[q], pol);
            if (gout) put_out4(gout + e, rp[q]);
          } else {
#pragma unroll
            for (int j = 0; j < kVec; ++j)
              if (e + j < n) {
                gp[e + j] = rp[q].x[j];
                if (gout) put_out1(gout + e + j, rp[q].x[j]);
              }
          }
        }
      } else {
        // ---- B (sums only), BP (sums, store m and v, park p / update_m / update_g), C ----
        F4 rg[kBVecs], rp[kBVecs], rm[kBVecs], rv[kBVecs];
#pragma unroll
        for (int q = 0; q < kBVecs; ++q) {
          const int e = q * (kGroupThreads * kVec) + gtid * kVec;
          if (e < nbulk) {
            rg[q] = Elem<GT>::smem4(sbase + e * sizeof(GT));
            rp[q] = Elem<float>::smem4(sbase + L::kGBytes + e * 4);
            rm[q] = Elem<float>::smem4(sbase + L::kGBytes + L::kFBytes + e * 4);
            rv[q] = Elem<float>::smem4(sbase + L::kGBytes + 2 * L::kFBytes + e * 4);
          } else {
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
              const bool in = e + j < n;
              rg[q].x[j] = in ? Elem<GT>::to_f32(gg[e + j]) : 0.f;
              rp[q].x[j] = in ? gp[e + j] : 0.f;
              rm[q].x[j] = in ? gm[e + j] : 0.f;
              rv[q].x[j] = in ? gv[e + j] : 0.f;
            }
          }
        }
        __syncwarp();  // values are in registers: the slot can be refilled
        if (lane == 0) mbar_arrive(my_done);
        // stage 1 of the thread's eight elements, `mode` resolved once
        F4 ua[kBVecs], ub[kBVecs];
        auto stage1 = [&](auto mode_tag) {
          constexpr int kMode = decltype(mode_tag)::value;
#pragma unroll
          for (int q = 0; q < kBVecs; ++q)
#pragma unroll
            for (int j = 0; j < kVec; ++j)
              s1.template apply<kMode>(rg[q].x[j], rp[q].x[j], rm[q].x[j], rv[q].x[j], cs, ua[q].x[j], ub[q].x[j]);
        };
        if (s1.mode == 0) stage1(std::integral_constant<int, 0>{});
        else stage1(std::integral_constant<int, 1>{});
        if (op == kOpC) {
#pragma unroll
          for (int q = 0; q < kBVecs; ++q) {
            const int e = q * (kGroupThreads * kVec) + gtid * kVec;
            // p - ratio_m*update_m - ratio_g*update_g  (:385; the ratios carry the minus sign)
#pragma unroll
            for (int j = 0; j < kVec; ++j)
              rp[q].x[j] = fmaf(ratio_g, ub[q].x[j], fmaf(ratio_m, ua[q].x[j], rp[q].x[j]));
            if (e < nbulk) {  // aligned: 16-byte stores
              Elem<float>::template store4<kStream>(gp + e, rp[q], pol);
              Elem<float>::template store4<kStream>(gm + e, rm[q], pol);
              Elem<float>::template store4<kStream>(gv + e, rv[q], pol);
              if (gout) put_out4(gout + e, rp[q]);
            } else {
#pragma unroll
              for (int j = 0; j < kVec; ++j)
                if (e + j < n) {
                  gp[e + j] = rp[q].x[j];
                  gm[e + j] = rm[q].x[j];
                  gv[e + j] = rv[q].x[j];
                  if (gout) put_out1(gout + e + j, rp[q].x[j]);
                }
            }
          }
        } else {
          publishes = true;
#pragma unroll
          for (int q = 0; q < kBVecs; ++q) {
            const int e = q * (kGroupThreads * kVec) + gtid * kVec;
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
              acc0 = fmaf(rp[q].x[j], rp[q].x[j], acc0);
              acc1 = fmaf(ua[q].x[j], ua[q].x[j], acc1);
              acc2 = fmaf(ub[q].x[j], ub[q].x[j], acc2);
            }
            if (op == kOpBP) {  // m and v are final
              if (e < nbulk) {
                Elem<float>::template store4<kStream>(gm + e, rm[q], pol);
                Elem<float>::template store4<kStream>(gv + e, rv[q], pol);
              } else {
#pragma unroll
                for (int j = 0; j < kVec; ++j)
                  if (e + j < n) {
                    gm[e + j] = rm[q].x[j];
                    gv[e + j] = rv[q].x[j];
                  }
              }
            }
          }
          if (op == kOpBP) {
            // p, update_m and update_g wait in tensor memory for the norms
            park_store(in_tmem, taddr, scell, gtid, rp, ua, ub);
            if (in_tmem) tmem_wait_st();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_cell + 8 * cell);
          }
        }
          }
    } else if (op == kOpA) {
      constexpr int kPasses = L::kAElems / (kGroupThreads * kVec);
      constexpr int kBatch = kPasses % 7 == 0 ? 7 : 8;  // vectors in flight per thread
      static_assert(kPasses % kBatch == 0, "an A item is whole batches of passes");
      for (int q0 = 0; q0 < kPasses; q0 += kBatch) {
        F4 r[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; ++q)
          r[q] = Elem<GT>::smem4(sbase + ((q0 + q) * (kGroupThreads * kVec) + gtid * kVec) * sizeof(GT));
#pragma unroll
        for (int q = 0; q < kBatch; ++q)
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            const float x = r[q].x[j] * s1.gscale;
            acc0 = fmaf(x, x, acc0);
          }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(my_done);
      publishes = true;
    } else if (op == kOpCP) {
      F4 rp[kBVecs], um[kBVecs], ug[kBVecs];
      park_load(in_tmem, taddr, scell, gtid, rp, um, ug);
      __syncwarp();
      if (lane == 0) mbar_arrive(my_done);  // the cell may be given to another chunk
#pragma unroll
      for (int q = 0; q < kBVecs; ++q) {
        const int e = q * (kGroupThreads * kVec) + gtid * kVec;
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          rp[q].x[j] = fmaf(ratio_g, ug[q].x[j], fmaf(ratio_m, um[q].x[j], rp[q].x[j]));
        Elem<float>::template store4<kStream>(gp + e, rp[q], pol);
      }
      if (gout) {
#pragma unroll
        for (int q = 0; q < kBVecs; ++q)
          put_out4(gout + q * (kGroupThreads * kVec) + gtid * kVec, rp[q]);
      }
    } else {
      F4 rg[kBVecs], rp[kBVecs], rm[kBVecs], rv[kBVecs], ua[kBVecs], ub[kBVecs];
#pragma unroll
      for (int q = 0; q < kBVecs; ++q) {
        const int e = q * (kGroupThreads * kVec) + gtid * kVec;
        rg[q] = Elem<GT>::smem4(sbase + e * sizeof(GT));
        rp[q] = Elem<float>::smem4(sbase + L::kGBytes + e * 4);
        rm[q] = Elem<float>::smem4(sbase + L::kGBytes + L::kFBytes + e * 4);
        rv[q] = Elem<float>::smem4(sbase + L::kGBytes + 2 * L::kFBytes + e * 4);
      }
      __syncwarp();  // values are in registers: the slot can be refilled
      if (lane == 0) mbar_arrive(my_done);
      auto stage1 = [&](auto mode_tag) {
        constexpr int kMode = decltype(mode_tag)::value;
#pragma unroll
        for (int q = 0; q < kBVecs; ++q)
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            s1.template apply<kMode>(rg[q].x[j], rp[q].x[j], rm[q].x[j], rv[q].x[j], cs, ua[q].x[j], ub[q].x[j]);
      };
      if (s1.mode == 0) stage1(std::integral_constant<int, 0>{});
      else stage1(std::integral_constant<int, 1>{});
      if (op == kOpC) {
#pragma unroll
        for (int q = 0; q < kBVecs; ++q) {
          const int e = q * (kGroupThreads * kVec) + gtid * kVec;
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            rp[q].x[j] = fmaf(ratio_g, ub[q].x[j], fmaf(ratio_m, ua[q].x[j], rp[q].x[j]));
          Elem<float>::template store4<kStream>(gp + e, rp[q], pol);
          Elem<float>::template store4<kStream>(gm + e, rm[q], pol);
          Elem<float>::template store4<kStream>(gv + e, rv[q], pol);
        }
        if (gout) {
#pragma unroll
          for (int q = 0; q < kBVecs; ++q)
            put_out4(gout + q * (kGroupThreads * kVec) + gtid * kVec, rp[q]);
        }
      } else {
        publishes = true;
#pragma unroll
        for (int q = 0; q < kBVecs; ++q)
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            acc0 = fmaf(rp[q].x[j], rp[q].x[j], acc0);
            acc1 = fmaf(ua[q].x[j], ua[q].x[j], acc1);
            acc2 = fmaf(ub[q].x[j], ub[q].x[j], acc2);
          }
        if (op == kOpBP) {
          // m and v are final; p, update_m and update_g wait in tensor memory for the norms
          park_store(in_tmem, taddr, scell, gtid, rp, ua, ub);
#pragma unroll
          for (int q = 0; q < kBVecs; ++q) {
            const int e = q * (kGroupThreads * kVec) + gtid * kVec;
            Elem<float>::template store4<kStream>(gm + e, rm[q], pol);
            Elem<float>::template store4<kStream>(gv + e, rv[q], pol);
          }
          if (in_tmem) tmem_wait_st();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_cell + 8 * cell);  // this warp's part is parked
        }
      }
    }
    // The bookkeeping after an operation goes to a different warp of the group each time.
    const bool duty = (uint32_t)wig == (i & 3u);
    if (duty) {
      if (lane == 0) {
        ok = ring_wait(my_done, opar, P.hdr, kErrDone, slot, P.wait_ns);
        if (ok && op == kOpCP) {
          // the parked chunk is in registers: its cell is free again, the item is finished
          atomicOr(&ctrl->cell_free, 1u << cell);
          atomicAdd(&ctrl->done_items, 1u);
        } else if (ok) {
          // The other three warps have let go of the slot too: its next item starts in it, or
          // the slot is marked idle and the prefetcher starts the item when it has one.
          if (op != kOpBP) atomicAdd(&ctrl->done_items, 1u);
          take_next(slot);
          if (op == kOpBP) {
            // every warp of the group has parked its part: the parker may queue the second
            // half as soon as the norms are final (which needs this chunk's sums, below)
            ok = ring_wait(bar_cell + 8 * cell, cpar, P.hdr, kErrDone, 0x100u | cell, P.wait_ns);
            if (ok) {
              ctrl->cell_grp[cell] = (uint32_t)grp;
              __threadfence_block();
              atomicOr(&ctrl->cell_parked, 1u << cell);
            }
          }
        }
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
    }
    if (publishes) {
      const float v0 = warp_sum(acc0);
      float v1 = 0.f, v2 = 0.f;
      if (op != kOpA) {
        v1 = warp_sum(acc1);
        v2 = warp_sum(acc2);
      }
      // the publisher has read this slot's previous sums
      if (lane == 0) ok = ring_wait(bar_redempty + 8 * slot, rpar ^ 1u, P.hdr, kErrRing, 0x2000u | slot, P.wait_ns);
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane == 0) {
        RedSlot& rs = s_red[slot];
        rs.val[0][wig] = v0;
        rs.val[1][wig] = v1;
        rs.val[2][wig] = v2;
        if (wig == 0) {
          rs.tensor = mt.tensor_op & kTensorMask;
          rs.is_a = (op == kOpA) ? 1u : 0u;
          rs.nparts = mt.nparts;
        }
        mbar_arrive(bar_redfull + 8 * slot);
      }
    }
  }
  // No more work (or a wait expired): tell the publisher and the parker that this warp has left.
  __syncwarp();
  if (lane == 0) mbar_arrive(bar_end);
}

// One-tensor descriptor, per-block work-item lists and zeroed control words written by the
// device itself: the set-up of the entry point that may not allocate or copy from host
// memory.  Global order: A items, streamed stage-1 items, parked items, streamed updates;
// item i of that order goes to block i % grid.
__global__ void lans_static_init_kernel(unsigned char* ws, size_t ctl_off, size_t desc_off, size_t off_off,
                                        size_t items_off, TensorDesc d, uint32_t n_a, uint32_t n_b,
                                        uint32_t n_park, uint32_t grid, uint32_t slots) {
  const uint32_t n_stream = n_b - n_park;
  const uint32_t total = n_a + n_b + n_stream;
  Item* items = reinterpret_cast<Item*>(ws + items_off);
  uint32_t* off = reinterpret_cast<uint32_t*>(ws + off_off);
  // Same dealing as partition_lans_items, with one tensor and every item in one sequence:
  // block b owns the global positions b, b + grid, ...; its r-th item goes to the list of
  // its even slots when (r % slots) is even, else to the list of its odd slots.
  auto first_of = [&](uint32_t b) {  // entries of blocks 0 .. b-1
    const uint32_t q = total / grid, r = total % grid;
    return b * q + (b < r ? b : r);
  };
  auto in_half = [&](uint32_t r, uint32_t odd) {  // items 0 .. r-1 of a block that go to that list
    const uint32_t full = r / slots, rem = r % slots;
    return odd ? full * (slots / 2) + rem / 2 : full * ((slots + 1) / 2) + (rem + 1) / 2;
  };
  for (uint32_t b = threadIdx.x; b <= grid; b += blockDim.x) {
    off[2 * b] = first_of(b);
    if (b < grid) off[2 * b + 1] = first_of(b) + in_half(first_of(b + 1) - first_of(b), 0);
  }
  for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
    const uint32_t b = i % grid, r = i / grid, odd = (r % slots) & 1u;
    Item it;
    if (i < n_a) it = Item{kKindA << kPhaseShift, i};
    else if (i < n_a + n_stream) it = Item{kKindBs << kPhaseShift, i - n_a};
    else if (i < n_a + n_b) {
      // running number among the parked items of the same list
      const uint32_t lo = n_a + n_stream;
      const uint32_t r_lo = lo > b ? (lo - b + grid - 1) / grid : 0u;
      it = Item{kKindBCp << kPhaseShift, (i - n_a) | (((in_half(r, odd) - in_half(r_lo, odd)) & 2047u) << 21)};
    } else it = Item{kKindCs << kPhaseShift, i - n_a - n_b};
    items[first_of(b) + (odd ? in_half(first_of(b + 1) - first_of(b), 0) : 0u) + in_half(r, odd)] = it;
  }
  uint32_t* head = reinterpret_cast<uint32_t*>(ws);
  for (uint32_t i = threadIdx.x; i < (ctl_off + sizeof(LansCtl)) / 4; i += blockDim.x) head[i] = 0u;
  if (threadIdx.x == 0) *reinterpret_cast<TensorDesc*>(ws + desc_off) = d;
}

// ---- host side -----------------------------------------------------------------

int lans_slots(int g_dtype) { return g_dtype == RAFB200_F32 ? kLansSlots32 : kLansSlots16; }
int lans_a_elems(int g_dtype) { return g_dtype == RAFB200_F32 ? kLansAElems32 : kLansAElems16; }

// How many chunks of one tensor may wait on chip at the same time, for a grid with
// `cells_total` cells (blocks x kLansCells): five eighths.  Every block - the parked items are
// dealt out evenly - then keeps cells for the tensors before and after a large one, whose
// stage 1 overlaps the wait for the large tensor's norms (measured on the BERT-large list:
// 2.20 ms at 5/8, 2.25 ms at 4/5, 2.27 ms at 3/8).
uint32_t lans_park_cap(int64_t cells_total) {
  const int64_t cap = cells_total * 5 / 8;
  return (uint32_t)(cap < 0 ? 0 : cap);
}

// Orders the work items of a list.  Dependencies always point to earlier positions:
//   - the A items of a tensor precede its first Bs / BCp item, and the A pass runs
//     `lead_elems` elements ahead of the rest where the list allows it;
//   - the Bs and BCp items of the tensors come in tensor order, a tensor's Bs items first,
//     then its BCp items (at most `park_cap` of them: the tail of the tensor);
//   - the Cs items of a tensor follow its last BCp item, after `gap_items` further items
//     where other work exists (the norms they wait for are then final when they are drawn),
//     alternating with that other work so that loads and stores stay mixed.
std::vector<Item> build_lans_schedule(const std::vector<int64_t>& numel, int a_elems, bool with_a,
                                      uint32_t park_cap, int64_t lead_elems, int64_t gap_items) {
  const int k = (int)numel.size();
  std::vector<Item> out;
  struct Pending {  // the streamed update items of a tensor, released `gap_items` later
    uint32_t tensor, next, count;
    int64_t release_at;
  };
  std::vector<Pending> pend;
  size_t pend_head = 0;
  int a_t = 0;
  uint32_t a_c = 0;
  int64_t a_done = 0, b_done = 0;
  auto n_a_of = [&](int t) { return (uint32_t)((numel[t] + a_elems - 1) / a_elems); };
  auto n_b_of = [&](int t) { return (uint32_t)((numel[t] + kLansElems - 1) / kLansElems); };
  auto skip_a = [&]() {
    while (a_t < k && n_a_of(a_t) == 0) ++a_t;
  };
  auto emit_a = [&]() {
    out.push_back(Item{(kKindA << kPhaseShift) | (uint32_t)a_t, a_c});
    const int64_t left = numel[a_t] - (int64_t)a_c * a_elems;
    a_done += left < a_elems ? left : a_elems;
    if (++a_c == n_a_of(a_t)) {
      a_c = 0;
      ++a_t;
      skip_a();
    }
  };
  auto emit_pending = [&](bool force) -> bool {
    if (pend_head >= pend.size()) return false;
    Pending& pd = pend[pend_head];
    if (!force && (int64_t)out.size() < pd.release_at) return false;
    out.push_back(Item{(kKindCs << kPhaseShift) | pd.tensor, pd.next});
    if (++pd.next == pd.count) ++pend_head;
    return true;
  };
  if (!with_a) a_t = k;
  skip_a();
  int64_t end_of_t = 0;
  for (int t = 0; t < k; ++t) {
    end_of_t += numel[t];
    const uint32_t nb = n_b_of(t);
    if (nb == 0) continue;
    const uint32_t park = nb < park_cap ? nb : park_cap;
    const uint32_t stream = nb - park;
    for (uint32_t c = 0; c < nb; ++c) {
      // the gradient-norm pass: complete for this tensor, and `lead_elems` ahead
      while (a_t < k && (a_t <= t || a_done < b_done + lead_elems)) emit_a();
      (void)end_of_t;
      emit_pending(false);  // one streamed update item of an earlier tensor, when released
      out.push_back(Item{((c < stream ? kKindBs : kKindBCp) << kPhaseShift) | (uint32_t)t, c});
      const int64_t left = numel[t] - (int64_t)c * kLansElems;
      b_done += left < kLansElems ? left : kLansElems;
    }
    if (stream > 0) pend.push_back(Pending{(uint32_t)t, 0, stream, (int64_t)out.size() + gap_items});
  }
  while (emit_pending(true)) {
  }
  return out;
}

// Deals the items of a schedule out to `grid` blocks, each block keeping the global order.
// Stage-1 items (Bs, BCp) are dealt in turn among themselves, the other items among
// themselves, so that a tensor's parked items spread evenly over the blocks whatever they
// are interleaved with.  Inside a block the r-th item of either sort goes to the list of
// the even slots when (r % slots) is even, else to the list of the odd slots: the two lists
// get work in proportion to their slots, and of any 19 consecutive parked items (the most a
// block gets of one tensor, see lans_park_cap) at most 11 land in either list, which has 14 or
// 15 cells of its own.
// Result: off[0 .. 2 * grid] (list 2b = even slots of block b, 2b + 1 = odd slots),
// followed (8-byte aligned) by the items.
std::vector<uint32_t> partition_lans_items(const std::vector<Item>& sched, int grid, int slots) {
  std::vector<std::vector<Item>> per(2 * (size_t)grid);
  uint64_t rr_b = 0, rr_o = 0;
  for (const Item& it : sched) {
    const uint32_t kind = it.tensor_phase >> kPhaseShift;
    const bool stage1 = kind == kKindBs || kind == kKindBCp;
    const uint64_t r = stage1 ? rr_b++ : rr_o++;
    const uint64_t b = r % (uint64_t)grid, round = r / (uint64_t)grid;
    per[2 * b + ((round % (uint64_t)slots) & 1u)].push_back(it);
  }
  const size_t head = (2 * (size_t)grid + 1 + 1) & ~(size_t)1;  // uint32 words before the items
  std::vector<uint32_t> out(head + 2 * sched.size());
  uint32_t at = 0;
  for (int hb = 0; hb < 2 * grid; ++hb) {
    out[hb] = at;
    // Each list has its own prefetcher warp and its own half of the block's tensor-memory
    // cells.  Its parked items carry their running number among them (modulo 2^11, far more
    // than are ever in flight) in the top bits of the chunk word; chunk indices stay below
    // 2^21.  Cells are handed out by these numbers.
    uint32_t seq = 0;
    for (const Item& it : per[hb]) {
      uint32_t chunk = it.chunk;
      if ((it.tensor_phase >> kPhaseShift) == kKindBCp) chunk |= (seq++ & 2047u) << 21;
      out[head + 2 * (size_t)at] = it.tensor_phase;
      out[head + 2 * (size_t)at + 1] = chunk;
      ++at;
    }
  }
  out[2 * grid] = at;
  return out;
}

size_t lans_ctl_bytes(int k) { return 128 + sizeof(LansCtl) * (size_t)k; }

size_t lans_workspace_bytes(int k) { return (lans_ctl_bytes(k) + 255) & ~(size_t)255; }

// The persistent grid: one block per SM, or fewer when a cap leaves SMs to a concurrent
// collective.  The schedule of a list is built for this number of blocks.
int lans_grid(int sm_count, int max_blocks) {
  int g = sm_count;
  if (max_blocks > 0 && g > max_blocks) g = max_blocks;
  return g < 1 ? 1 : g;
}

template <typename GT, typename OT, bool FUSED>
static int launch_lans_f(int device, int grid, const LansParams& P, cudaStream_t s) {
  static bool configured[64] = {false};
  const int dev = (device >= 0 && device < 64) ? device : 0;
  const int smem = LansGeo<GT>::kTotal;
  if (!configured[dev]) {
    RAFB200_CUDA(cudaFuncSetAttribute(lans_kernel<GT, OT, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  lans_kernel<GT, OT, FUSED><<<(unsigned)grid, kLansThreads, smem, s>>>(P);
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

template <typename GT, typename OT>
static int launch_lans_t(int device, int grid, const LansParams& P, cudaStream_t s) {
  if (P.fuse_rs || P.fuse_ag) return launch_lans_f<GT, OT, true>(device, grid, P, s);
  return launch_lans_f<GT, OT, false>(device, grid, P, s);
}

template <typename GT>
static int launch_lans_g(int device, int grid, int out_dtype, const LansParams& P, cudaStream_t s) {
  switch (out_dtype) {
    case RAFB200_F32: return launch_lans_t<GT, float>(device, grid, P, s);
    case RAFB200_F16: return launch_lans_t<GT, __half>(device, grid, P, s);
    default: return launch_lans_t<GT, __nv_bfloat16>(device, grid, P, s);
  }
}

static int launch_lans(int device, int grid, int g_dtype, int out_dtype, const LansParams& P, cudaStream_t s) {
  switch (g_dtype) {
    case RAFB200_F32: return launch_lans_g<float>(device, grid, out_dtype, P, s);
    case RAFB200_F16: return launch_lans_g<__half>(device, grid, out_dtype, P, s);
    default: return launch_lans_g<__nv_bfloat16>(device, grid, out_dtype, P, s);
  }
}

static void fill_stage1(LansParams* P, int step, float learning_rate, float beta1, float beta2, float eps,
                        int bias_correction, float weight_decay, int grad_averaging, int mode,
                        int normalize_grad, float grad_scale) {
  P->s1.beta1 = beta1;
  P->s1.beta2 = beta2;
  P->s1.beta3 = (grad_averaging == 1) ? 1 - beta1 : 1.0f;  // lans.cc:106-109
  P->s1.one_minus_beta2 = 1 - beta2;
  P->s1.eps = eps;
  float bc1, bc2;
  bias_corrections(beta1, beta2, step, bias_correction, &bc1, &bc2);
  P->s1.inv_bc1 = 1.0f / bc1;
  P->s1.inv_bc2 = 1.0f / bc2;
  P->s1.wd = weight_decay;
  P->s1.gscale = grad_scale;
  P->s1.mode = mode;
  P->s1.normalize = normalize_grad ? 1 : 0;
  P->lr = learning_rate;
  P->bias_correction = bias_correction;
}

}  // namespace rafb200

using namespace rafb200;

// ---- scratch of rafb200_lans_tensor_static --------------------------------------
// Everything rafb200_lans keeps in caller-provided device memory (header, per-tensor
// control words, descriptor row, work-item table) for ONE tensor of at most
// kStaticMaxElems elements, as a statically allocated device array: every GPU that
// loads this library holds these 74 KB until the process exits.
constexpr int64_t kStaticMaxElems = 4ll << 20;  // 4,194,304 elements
constexpr uint32_t kStaticMaxB = (uint32_t)(kStaticMaxElems / kLansElems);
constexpr uint32_t kStaticMaxA = (uint32_t)((kStaticMaxElems + kLansAElems32 - 1) / kLansAElems32);
constexpr size_t kStaticCtlOff = 128, kStaticDescOff = 256, kStaticOffOff = 512, kStaticItemsOff = 2048;
constexpr int kStaticMaxGrid = ((int)((kStaticItemsOff - kStaticOffOff) / 4) - 1) / 2;  // 191 blocks (two lists each)
constexpr size_t kStaticBytes = kStaticItemsOff + (size_t)(kStaticMaxA + 2 * kStaticMaxB) * sizeof(Item);
static __device__ __align__(256) unsigned char g_lans_static_scratch[kStaticBytes];

// Device address of the array above, per device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use: the address has
// to be asked for, once per device, with that device current.
static void* g_lans_static_ptr[64] = {nullptr};
static int g_lans_static_sms[64] = {0};

extern "C" {

size_t rafb200_lans_workspace_bytes(rafb200_tensor_list_t list) {
  if (!list) return 0;
  return lans_workspace_bytes(list->k);
}

int rafb200_lans(rafb200_tensor_list_t list, int step, const float* step_dev, float learning_rate,
                 float beta1, float beta2, float eps, int bias_correction, float weight_decay,
                 int grad_averaging, int mode, int normalize_grad, float grad_scale,
                 void* workspace, size_t workspace_bytes, void* stream) {
  RAFB200_REQUIRE(list, "rafb200_lans: NULL list");
  RAFB200_REQUIRE(list->bound && list->has_v, "rafb200_lans: bind g, p, m and v first");
  RAFB200_REQUIRE(step_dev != nullptr || step >= 1, "rafb200_lans: step counts from 1");
  RAFB200_REQUIRE(mode == 0 || mode == 1, "rafb200_lans: mode must be 0 (L2) or 1 (decoupled)");
  const size_t need = lans_workspace_bytes(list->k);
  RAFB200_REQUIRE(workspace && workspace_bytes >= need,
                  "rafb200_lans: workspace of %zu bytes required, got %zu", need, workspace_bytes);
  RAFB200_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0,
                  "rafb200_lans: workspace must be 16-byte aligned");
  if (list->total_elems == 0) return RAFB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  LansParams P{};
  P.descs = list->dev_desc;
  const LansFuse& fu = list->fuse;
  if (fu.fuse_rs || fu.fuse_ag) {
    RAFB200_REQUIRE(!fu.fuse_rs || normalize_grad,
                    "rafb200_lans: reading the gradients through the switch needs the gradient-norm pass");
    P.world = fu.world;
    P.rank = fu.rank;
    P.fuse_rs = fu.fuse_rs;
    P.fuse_ag = fu.fuse_ag;
    P.g_mc = fu.g_mc;
    P.p_mc = fu.p_mc;
    for (int q = 0; q < kSymmMaxWorld; ++q) {
      P.g_peer[q] = fu.g_peer[q];
      P.p_peer[q] = fu.p_peer[q];
    }
  }
  const uint32_t* table = normalize_grad ? list->dev_lans_lists : list->dev_lans_lists_nonorm;
  const size_t head = (2 * (size_t)list->lans_grid + 1 + 1) & ~(size_t)1;
  P.block_off = table;
  P.items = reinterpret_cast<const Item*>(table + head);
  char* ws = static_cast<char*>(workspace);
  P.hdr = reinterpret_cast<LansHeader*>(ws);
  P.ctl = reinterpret_cast<LansCtl*>(ws + 128);
  fill_stage1(&P, step_dev ? 1 : step, learning_rate, beta1, beta2, eps, bias_correction, weight_decay,
              grad_averaging, mode, normalize_grad, grad_scale);
  P.step_dev = step_dev;
  P.wait_ns = list->wait_ns;

  RAFB200_CUDA(cudaMemsetAsync(workspace, 0, lans_ctl_bytes(list->k), s));
  if (step_dev) {
    lans_bias_kernel<<<1, 1, 0, s>>>(P.hdr, step_dev, beta1, beta2, bias_correction);
    RAFB200_CUDA(cudaGetLastError());
  }
  return launch_lans(list->device, list->lans_grid, list->g_dtype, list->out_dtype, P, s);
}

int rafb200_lans_tensor_static(const void* g, int g_dtype, float* p, float* m, float* v,
                               void* out, int out_dtype, int64_t numel, int step,
                               float learning_rate, float beta1, float beta2, float eps,
                               int bias_correction, float weight_decay, int grad_averaging,
                               int mode, int normalize_grad, float grad_scale, void* stream) {
  RAFB200_REQUIRE(dtype_valid(g_dtype) && dtype_valid(out_dtype),
                  "rafb200_lans_tensor_static: bad dtype");
  RAFB200_REQUIRE(numel >= 0, "rafb200_lans_tensor_static: negative numel");
  RAFB200_REQUIRE(numel <= kStaticMaxElems,
                  "rafb200_lans_tensor_static: %lld elements exceed the static scratch, which is "
                  "sized for at most %lld; use rafb200_lans with a caller-provided workspace",
                  (long long)numel, (long long)kStaticMaxElems);
  RAFB200_REQUIRE(step >= 1, "rafb200_lans_tensor_static: step counts from 1");
  RAFB200_REQUIRE(mode == 0 || mode == 1, "rafb200_lans_tensor_static: mode must be 0 or 1");
  if (numel == 0) return RAFB200_OK;
  RAFB200_REQUIRE(g && p && m && v, "rafb200_lans_tensor_static: g, p, m and v must not be NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  int device = 0;
  RAFB200_CUDA(cudaGetDevice(&device));
  RAFB200_REQUIRE(device >= 0 && device < 64, "rafb200_lans_tensor_static: device %d out of range", device);
  if (g_lans_static_ptr[device] == nullptr) {
    // First call on this device (do it before any stream capture): resolve the symbol.
    void* ptr = nullptr;
    RAFB200_CUDA(cudaGetSymbolAddress(&ptr, g_lans_static_scratch));
    RAFB200_CUDA(cudaDeviceGetAttribute(&g_lans_static_sms[device], cudaDevAttrMultiProcessorCount, device));
    g_lans_static_ptr[device] = ptr;
  }
  unsigned char* ws = static_cast<unsigned char*>(g_lans_static_ptr[device]);

  TensorDesc d{};
  d.g = g;
  d.p = p;
  d.m = m;
  d.v = v;
  d.out = out;
  d.numel = numel;
  d.first_chunk = 0;
  d.nchunks = (uint32_t)((numel + kChunkElems - 1) / kChunkElems);
  auto a16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  const bool vec_ok = a16(p) && a16(m) && a16(v) &&
                      (reinterpret_cast<uintptr_t>(g) % (g_dtype == RAFB200_F32 ? 16 : 8) == 0) &&
                      (!out || reinterpret_cast<uintptr_t>(out) % (out_dtype == RAFB200_F32 ? 16 : 8) == 0);
  d.flags = vec_ok ? kFlagAligned : 0u;
  if (vec_ok && a16(g) && (!out || a16(out))) d.flags |= kFlagBulk;

  int grid = lans_grid(g_lans_static_sms[device], 0);
  if (grid > kStaticMaxGrid) grid = kStaticMaxGrid;
  const int a_elems = lans_a_elems(g_dtype);
  const uint32_t n_a = normalize_grad ? (uint32_t)((numel + a_elems - 1) / a_elems) : 0u;
  const uint32_t n_b = (uint32_t)((numel + kLansElems - 1) / kLansElems);
  const uint32_t cap = lans_park_cap((int64_t)grid * kLansCells);
  const uint32_t n_park = n_b < cap ? n_b : cap;

  LansParams P{};
  P.descs = reinterpret_cast<const TensorDesc*>(ws + kStaticDescOff);
  P.block_off = reinterpret_cast<const uint32_t*>(ws + kStaticOffOff);
  P.items = reinterpret_cast<const Item*>(ws + kStaticItemsOff);
  P.hdr = reinterpret_cast<LansHeader*>(ws);
  P.ctl = reinterpret_cast<LansCtl*>(ws + kStaticCtlOff);
  fill_stage1(&P, step, learning_rate, beta1, beta2, eps, bias_correction, weight_decay, grad_averaging,
              mode, normalize_grad, grad_scale);
  P.step_dev = nullptr;
  P.wait_ns = 2000000000ull;

  // The array keeps whatever the previous call left in it.  A small kernel on the same
  // stream zeroes the ticket counter, the error word, the arrival counters, sums and norm
  // words and writes this call's descriptor and item table; nothing is copied from host
  // memory and nothing is allocated, on the device or on the host.
  lans_static_init_kernel<<<1, 256, 0, s>>>(ws, kStaticCtlOff, kStaticDescOff, kStaticOffOff, kStaticItemsOff, d,
                                            n_a, n_b, n_park, (uint32_t)grid, (uint32_t)lans_slots(g_dtype));
  RAFB200_CUDA(cudaGetLastError());
  return launch_lans(device, grid, g_dtype, out_dtype, P, s);
}

int rafb200_lans_schedule(int k, const int64_t* numel, int g_dtype, int with_norm_phase, int cells_total,
                          int64_t lead_elems, int gap_items, uint32_t* items, size_t capacity,
                          size_t* count) {
  RAFB200_REQUIRE(k >= 0 && (k == 0 || numel) && count && lead_elems >= 0 && gap_items >= 0 &&
                      cells_total >= 1 && dtype_valid(g_dtype),
                  "rafb200_lans_schedule: bad arguments");
  std::vector<int64_t> n(k);
  for (int i = 0; i < k; ++i) {
    RAFB200_REQUIRE(numel[i] >= 0, "rafb200_lans_schedule: numel[%d] < 0", i);
    n[i] = numel[i];
  }
  const std::vector<Item> sched = build_lans_schedule(n, lans_a_elems(g_dtype), with_norm_phase != 0,
                                                      lans_park_cap(cells_total), lead_elems,
                                                      gap_items > 0 ? gap_items : cells_total);
  *count = sched.size();
  if (items) {
    RAFB200_REQUIRE(capacity >= sched.size(), "rafb200_lans_schedule: %zu items, room for %zu", sched.size(),
                    capacity);
    for (size_t i = 0; i < sched.size(); ++i) {
      items[2 * i] = sched[i].tensor_phase;
      items[2 * i + 1] = sched[i].chunk;
    }
  }
  return RAFB200_OK;
}

int rafb200_lans_partition(int k, const int64_t* numel, int g_dtype, int with_norm_phase, int grid,
                           int64_t lead_elems, int gap_items, uint32_t* offsets, uint32_t* items,
                           size_t capacity, size_t* count, int* cells_even, int* cells_odd) {
  RAFB200_REQUIRE(k >= 0 && (k == 0 || numel) && count && grid >= 1 && lead_elems >= 0 && gap_items >= 0 &&
                      dtype_valid(g_dtype),
                  "rafb200_lans_partition: bad arguments");
  std::vector<int64_t> n(k);
  for (int i = 0; i < k; ++i) {
    RAFB200_REQUIRE(numel[i] >= 0, "rafb200_lans_partition: numel[%d] < 0", i);
    n[i] = numel[i];
  }
  const int64_t cells_total = (int64_t)grid * kLansCells;
  const std::vector<Item> sched =
      build_lans_schedule(n, lans_a_elems(g_dtype), with_norm_phase != 0, lans_park_cap(cells_total), lead_elems,
                          gap_items > 0 ? gap_items : (int64_t)grid * lans_slots(g_dtype));
  const std::vector<uint32_t> table = partition_lans_items(sched, grid, lans_slots(g_dtype));
  const size_t head = (2 * (size_t)grid + 1 + 1) & ~(size_t)1;
  *count = sched.size();
  if (cells_even) *cells_even = (kLansCells + 1) / 2;
  if (cells_odd) *cells_odd = kLansCells - (kLansCells + 1) / 2;
  if (offsets)
    for (int h = 0; h <= 2 * grid; ++h) offsets[h] = table[(size_t)h];
  if (items) {
    RAFB200_REQUIRE(capacity >= sched.size(), "rafb200_lans_partition: %zu items, room for %zu", sched.size(), capacity);
    for (size_t i = 0; i < 2 * sched.size(); ++i) items[i] = table[head + i];
  }
  return RAFB200_OK;
}

int rafb200_lans_status(rafb200_tensor_list_t list, const void* workspace, float* norms_host,
                        void* stream) {
  RAFB200_REQUIRE(list && workspace, "rafb200_lans_status: NULL argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RAFB200_CUDA(cudaStreamSynchronize(s));
  std::vector<char> host(lans_ctl_bytes(list->k));
  RAFB200_CUDA(cudaMemcpy(host.data(), workspace, host.size(), cudaMemcpyDeviceToHost));
  const LansHeader* hdr = reinterpret_cast<const LansHeader*>(host.data());
  const LansCtl* ctl = reinterpret_cast<const LansCtl*>(host.data() + 128);
  if (norms_host) {
    for (int t = 0; t < list->k; ++t)
      for (int j = 0; j < 4; ++j) {
        const unsigned bits = ctl[t].norm[j] & ~kNormValid;
        memcpy(&norms_host[4 * t + j], &bits, sizeof(float));
      }
  }
  if (hdr->error != 0)
    return set_error(RAFB200_DEVICE_WAIT_EXPIRED,
                     "rafb200_lans: bounded wait %u expired at work item %u; results are invalid",
                     hdr->error, hdr->error_item);
  return RAFB200_OK;
}

}  // extern "C"
