// raf.op.lans as ONE persistent kernel.
//
// The reference runs four norm reductions and two element-wise stages as about
// fifty launches with a global dependency between them
// (src/op/dialect/cuda/kernels/multi_tensor_lans.cu:401-450).  Here the work of
// a call is a list of items (tensor, chunk, phase):
//   phase A  sum of squares of the (scaled) gradient chunk            -> ||g||
//   phase B  stage 1 on the chunk, results NOT stored: sums of squares of
//            p, update_m, update_g                                     -> norms
//   phase C  stage 1 again (same instructions, same bits), then stage 2 with the
//            trust ratios; writes p, m, v and the model-dtype parameter copy.
// Blocks draw items from a ticket counter in list order.  An item depends only
// on items with smaller tickets (B of a tensor on all its A items, C on all its
// B items), and a ticket is only ever held by a running block, so the bounded
// waits below cannot deadlock whatever the number of resident blocks.  The
// host orders the list so that a tensor's C items follow its B items closely:
// the second read of g, p, m, v then comes out of L2 and HBM traffic approaches
// one read and one write per array.
//
// Norms: every chunk adds its fp32 partial sums to per-tensor double-precision
// accumulators; the block that adds the last chunk of a tensor takes the square
// root and publishes the norm together with its "final" bit in one word.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <type_traits>

#include "common.h"
#include "update_core.cuh"

namespace rafb200 {

void bias_corrections(float beta1, float beta2, int step, int bias_correction, float* bc1,
                      float* bc2);

constexpr int kPhaseA = 0, kPhaseB = 1, kPhaseC = 2;
constexpr unsigned kErrWaitA = 1, kErrWaitB = 2, kErrRing = 3;

struct LansParams {
  const TensorDesc* descs;
  const Item* items;
  uint32_t nitems;
  LansHeader* hdr;
  LansCtl* ctl;
  LansStage1 s1;
  float lr;
  const float* step_dev;
  int bias_correction;
  uint64_t wait_ns;  // bound of every wait inside the kernel
};


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
// B needs ||g|| (word 0), C needs ||p||, ||update_m||, ||update_g|| (words 1-3; they
// are published together with, or after, word 0).
__device__ __forceinline__ bool norms_final(const uint4& n, bool phase_c) {
  return phase_c ? ((n.y & n.z & n.w) >> 31) != 0 : (n.x >> 31) != 0;
}
__device__ __forceinline__ float norm_value(unsigned bits) {
  return __uint_as_float(bits & ~kNormValid);
}

// Bounded wait until the norms a phase needs are final: gives up after `wait_ns`
// nanoseconds (or as soon as another block has reported an error) and returns false.
__device__ __forceinline__ bool wait_norms(const LansCtl* c, bool phase_c, uint4* out,
                                           LansHeader* hdr, unsigned code, uint32_t ticket,
                                           uint64_t wait_ns) {
  uint4 n = ld_norms(c);
  if (!norms_final(n, phase_c)) {
    const uint64_t t0 = global_ns();
    unsigned spins = 0, ns = 32;
    do {
      __nanosleep(ns);
      if (ns < 1024) ns <<= 1;
      if ((++spins & 15u) == 0) {
        if (*reinterpret_cast<volatile unsigned*>(&hdr->error) != 0) return false;
        if (global_ns() - t0 > wait_ns) {
          if (atomicCAS(&hdr->error, 0u, code) == 0u) hdr->error_item = ticket;
          return false;
        }
      }
      n = ld_norms(c);
    } while (!norms_final(n, phase_c));
  }
  *out = n;
  return true;
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
// Same, but the hardware may keep the thread suspended for up to `hint_ns` while the
// phase is incomplete: a waiting warp then leaves the issue slots of its scheduler to
// the warps that have work (here: the producer warp that everybody is waiting for).
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity,
                                                      uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded: try_wait blocks for a short hardware-defined time per call; the loop
// gives up after `wait_ns` nanoseconds and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t wait_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  while (!mbar_try_wait(bar, parity))
    if (global_ns() - t0 > wait_ns) return false;
  return true;
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

// ---- kernel geometry ---------------------------------------------------------------
// A work item is one chunk (kChunkElems elements) of one tensor in one phase.  It is
// streamed as stages: the g, p, m and v slices of kStageElems elements (phases B, C),
// or the whole chunk of g (phase A), copied into shared memory by TMA.  kStages stages
// form a ring per block.  Three kinds of warps share a block:
//   warps 0-7  consumers: wait for a stage, pull their elements into registers, give
//              the slot back, compute, store p/m/v and the parameter copy (phase C) or
//              accumulate sums of squares (A, B).  They never touch a block-wide
//              barrier and never wait on global memory.
//   warp 8     producer (one thread): draws tickets, resolves each item's dependency
//              (bounded wait on the tensor's flag), fills the ring with bulk copies.
//   warp 9     publisher: adds the consumers' per-warp partial sums of an item, writes
//              them to global memory, counts arrivals per tensor and - for the last
//              chunk of a tensor - adds all chunk partials in a fixed order, takes the
//              square root and releases the tensor's flag.
// Three blocks of two stages each are resident per SM (~170 KB of copies in flight per SM,
// 24 consumer warps): measured 1-4 % faster than two blocks of three stages; deeper rings
// did not help and stages of half the size cost 15 %.
#ifndef RAFB200_LANS_STAGE_VECS
#define RAFB200_LANS_STAGE_VECS 2
#endif
constexpr int kStageVecs = RAFB200_LANS_STAGE_VECS;  // 4-element vectors per consumer thread per B/C stage
constexpr int kStageElems = kBlockThreads * 4 * kStageVecs;  // 2048
#ifndef RAFB200_LANS_STAGES
#define RAFB200_LANS_STAGES 2  // ring depth per block
#endif
#ifndef RAFB200_LANS_BLOCKS
#define RAFB200_LANS_BLOCKS 3  // resident blocks per SM the ring and registers are sized for
#endif
constexpr int kStages = RAFB200_LANS_STAGES;
constexpr int kConsumers = kBlockThreads;        // 256
constexpr int kConsumerWarps = kConsumers / 32;  // 8
constexpr int kLansThreads = kConsumers + 64;    // + producer warp + publisher warp
constexpr int kRedSlots = 4;                     // ring of pending reductions
constexpr uint32_t kTicketEnd = 0xffffffffu;
constexpr uint32_t kRedEnd = 3u;
static_assert(kChunkElems % kStageElems == 0, "a chunk is a whole number of stages");
static_assert(kChunkElems % (kConsumers * kVec) == 0, "phase A walks a chunk in whole passes");

struct __align__(16) StageMeta {
  const void* g;  // global addresses of the stage's first element (stores, unaligned fallback)
  float* p;
  float* m;
  float* v;
  void* out;
  uint32_t ticket;      // kTicketEnd: no more work (or a wait expired) - consumers leave
  uint32_t n;           // elements in this stage
  uint32_t nbulk;       // leading elements that were delivered into shared memory
  uint32_t flags;       // bits 0-1 phase, bit 2 first stage of its item, bit 3 last stage
  uint32_t tensor;
  uint32_t part_index;  // slot of the item's partial sums
  uint32_t nchunks;
  uint32_t first_chunk;
  float cs;             // gradient multiplier  grad_scale / (||g|| + eps)
  float ratio_m;        // -beta1 * lr * ||p|| / ||update_m||   (phase C)
  float ratio_g;        // -beta3 * lr * ||p|| / ||update_g||
  uint32_t pad_;
};
static_assert(sizeof(StageMeta) == 96, "StageMeta is 96 bytes");

struct __align__(16) RedSlot {
  float val[3][kConsumerWarps];  // per consumer warp: sums of squares of this item
  uint32_t phase;                // kPhaseA, kPhaseB or kRedEnd (consumers have left)
  uint32_t tensor;
  uint32_t part_index;
  uint32_t nchunks;
  uint32_t first_chunk;
  uint32_t pad_[3];
};
static_assert(sizeof(RedSlot) == 128, "RedSlot is 128 bytes");

// A stage that has been issued but whose norms were not final yet.
struct __align__(16) PendStage {
  uint32_t slot, phase, tensor, ticket;
};

// Metadata of one of the (up to four) tickets a block holds, filled by cp.async.
struct __align__(16) ChainSlot {
  uint32_t ticket;
  uint32_t pad_;
  Item item;
  unsigned int norm[4];
  TensorDesc d;
};
static_assert(sizeof(ChainSlot) == 96, "ChainSlot is 96 bytes");

__device__ __forceinline__ void cp_async8(void* smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async16_ca(void* smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async16_cg(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}

template <typename GT>
struct LansSmem {
  static constexpr int kGBytes = kStageElems * sizeof(GT);
  static constexpr int kFBytes = kStageElems * 4;
  static constexpr int kStageBytes = kGBytes + 3 * kFBytes;
  static_assert(kChunkElems * sizeof(GT) <= kStageBytes, "a phase-A stage holds a chunk of g");
  static constexpr int kMetaOff = kStages * kStageBytes;
  static constexpr int kRedOff = kMetaOff + kStages * (int)sizeof(StageMeta);
  static constexpr int kChainOff = kRedOff + kRedSlots * (int)sizeof(RedSlot);
  static constexpr int kPendOff = kChainOff + 4 * (int)sizeof(ChainSlot);
  static constexpr int kBarOff = kPendOff + kStages * (int)sizeof(PendStage);
  static constexpr int kTotal = kBarOff + (2 * kStages + 2 * kRedSlots) * 8;
};

// Bounded wait on an mbarrier that also gives up as soon as any block has reported an
// error; a timeout reports kErrRing itself.
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, LansHeader* hdr,
                                          uint32_t where, uint64_t wait_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  unsigned polls = 0;
  while (!mbar_try_wait_suspend(bar, parity, 4000u)) {
    if ((++polls & 15u) == 0) {
      if (*reinterpret_cast<volatile unsigned*>(&hdr->error) != 0) return false;
      if (global_ns() - t0 > wait_ns) {
        if (atomicCAS(&hdr->error, 0u, kErrRing) == 0u) hdr->error_item = where;
        return false;
      }
    }
  }
  return true;
}

template <typename GT, typename OT>
__global__ void __launch_bounds__(kLansThreads, RAFB200_LANS_BLOCKS) lans_kernel(const LansParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  using L = LansSmem<GT>;
  StageMeta* s_meta = reinterpret_cast<StageMeta*>(smem + L::kMetaOff);
  RedSlot* s_red = reinterpret_cast<RedSlot*>(smem + L::kRedOff);
  const uint32_t bar_full = smem_u32(smem + L::kBarOff);
  const uint32_t bar_empty = bar_full + kStages * 8;
  const uint32_t red_full = bar_empty + kStages * 8;
  const uint32_t red_empty = red_full + kRedSlots * 8;
  const uint32_t data_base = smem_u32(smem);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 2);                // issue (+ transaction bytes) and resolve
      mbar_init(bar_empty + 8 * s, kConsumerWarps);  // one arrive per consumer warp
    }
    for (int s = 0; s < kRedSlots; ++s) {
      mbar_init(red_full + 8 * s, kConsumerWarps);
      mbar_init(red_empty + 8 * s, 1);               // the publisher
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  LansStage1 s1 = P.s1;
  if (P.step_dev != nullptr) {  // bias corrections were computed on the device, see above
    s1.inv_bc1 = __ldcg(&P.hdr->inv_bc1);
    s1.inv_bc2 = __ldcg(&P.hdr->inv_bc2);
  }

  if (warp == kConsumerWarps) {
    // =============================== producer ===============================
    // Resolving an item is a chain of dependent L2 round trips: ticket -> item ->
    // descriptor and norms.  It is software-pipelined three items deep through shared
    // memory with cp.async, so that no instruction ever waits for a load issued in
    // the same iteration (a register pipeline cannot do that across lanes: the
    // scoreboard tracks registers per warp):
    //   iteration i   draws the ticket of item i+3,
    //                 starts the copy of item i+2's table entry (its ticket was drawn
    //                 in iteration i-1),
    //                 starts the copies of item i+1's descriptor and norm words,
    //                 issues item i, whose metadata landed during iteration i-1.
    // A block thus holds at most four tickets and works them off in order.  Lane 0
    // runs the chain; lanes 0-3 issue the four bulk copies of a stage (g, p, m, v).
    const uint64_t pol_keep = make_policy_keep(), pol_stream = make_policy_stream();
    uint32_t stage_ctr = 0;
    int failed = 0;
    ChainSlot* chain = reinterpret_cast<ChainSlot*>(smem + L::kChainOff);
    auto fetch_item = [&](uint32_t seq) {  // lane 0; the slot's ticket has been stored
      ChainSlot& c = chain[seq & 3u];
      if (c.ticket < P.nitems) cp_async8(&c.item, P.items + c.ticket);
    };
    auto fetch_desc = [&](uint32_t seq) {  // lane 0; the slot's item has landed
      ChainSlot& c = chain[seq & 3u];
      if (c.ticket < P.nitems) {
        const uint32_t t = c.item.tensor_phase & kTensorMask;
        const char* src = reinterpret_cast<const char*>(P.descs + t);
        char* dst = reinterpret_cast<char*>(&c.d);
        cp_async16_ca(dst, src);
        cp_async16_ca(dst + 16, src + 16);
        cp_async16_ca(dst + 32, src + 32);
        cp_async16_ca(dst + 48, src + 48);
        cp_async16_cg(c.norm, P.ctl[t].norm);  // L2 copy: the publisher may just have written it
      }
    };
    if (lane == 0) {  // prologue: items 0, 1, 2
      chain[0].ticket = atomicAdd(&P.hdr->ticket, 1u);
      chain[1].ticket = atomicAdd(&P.hdr->ticket, 1u);
      chain[2].ticket = atomicAdd(&P.hdr->ticket, 1u);
      fetch_item(0);
      fetch_item(1);
      cp_async_wait_all();
      fetch_desc(0);
      cp_async_wait_all();
    }
    __syncwarp();

    // One iteration.  The ticket atomic is issued by lane 1 at the top and its result
    // is only touched (stored to shared memory) at the bottom, after the stages of
    // item `seq` have been issued: nothing waits for its round trip.
    // Issue and resolve are decoupled.  The bulk copies of a stage do not depend on the
    // tensor's norms, only the consumers' arithmetic does, so a stage is ISSUED (first
    // arrival on its full barrier, plus the copies' bytes) as soon as a ring slot is
    // free, and RESOLVED (multiplier and trust ratios written into its metadata, second
    // arrival) once the norms it needs are final.  A stage whose norms were already
    // final when the item's metadata was fetched is resolved on the spot; the others
    // queue up - at most kStages of them - and the producer only blocks on a norm when
    // it has no free slot left to fill.  While it waits, data keeps streaming in.
    PendStage* pend = reinterpret_cast<PendStage*>(smem + L::kPendOff);
    uint32_t pend_head = 0, pend_count = 0;
    // last norms seen final, per (tensor, phase C?) - lane 0 only
    uint32_t known_t = kTicketEnd;
    uint4 known_nrm = make_uint4(0, 0, 0, 0);

    auto ratios = [&](uint32_t phase, const uint4& nrm, float* cs, float* rm, float* rg) {
      *cs = s1.gscale;
      *rm = 0.f;
      *rg = 0.f;
      if (phase != kPhaseA) *cs = s1.grad_multiplier(norm_value(nrm.x));
      if (phase == kPhaseC) {  // multi_tensor_lans.cu:347-353
        const float pn = norm_value(nrm.y), umn = norm_value(nrm.z), ugn = norm_value(nrm.w);
        float a = (umn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, umn)) : P.lr;
        float b2 = (ugn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, ugn)) : P.lr;
        *rm = -mul(a, s1.beta1);
        *rg = -mul(b2, s1.beta3);
      }
    };
    auto needs_norms = [&](uint32_t phase) {
      return (phase == kPhaseB && s1.normalize) || phase == kPhaseC;
    };
    // lane 0: second arrival of stage `slot` with the final multipliers
    auto resolve_stage = [&](uint32_t slot, uint32_t phase, const uint4& nrm) {
      float cs, rm, rg;
      ratios(phase, nrm, &cs, &rm, &rg);
      StageMeta& mt = s_meta[slot];
      mt.cs = cs;
      mt.ratio_m = rm;
      mt.ratio_g = rg;
      mbar_arrive(bar_full + 8 * slot);
    };
    // lane 0: resolve the oldest pending stage, waiting (bounded) for its norms if need be,
    // then every following pending stage that the same norms settle.
    auto resolve_oldest = [&]() -> int {
      int bad = 0;
      bool waited = false;
      while (pend_count > 0) {
        const PendStage ps = pend[pend_head];
        const bool phase_c = ps.phase == kPhaseC;
        const bool settled = !needs_norms(ps.phase) ||
                             (known_t == ps.tensor && norms_final(known_nrm, phase_c));
        if (!settled) {
          if (waited) break;  // one blocking wait per call; the rest stays queued
          uint4 nrm;
          if (!wait_norms(P.ctl + ps.tensor, phase_c, &nrm, P.hdr, phase_c ? kErrWaitB : kErrWaitA,
                          ps.ticket, P.wait_ns)) {
            bad = 1;
            break;
          }
          known_t = ps.tensor;
          known_nrm = nrm;
          waited = true;
        }
        resolve_stage(ps.slot, ps.phase, known_nrm);
        pend_head = (pend_head + 1) % kStages;
        --pend_count;
      }
      return bad;
    };

    auto iteration = [&](uint32_t seq) -> bool {
      uint32_t drawn = 0;
      if (lane == 1) drawn = atomicAdd(&P.hdr->ticket, 1u);  // item seq + 3
      {
      if (lane == 0) {
        cp_async_wait_all();  // copies of the previous iteration
        fetch_item(seq + 2);  // its ticket was stored at the bottom of the previous iteration
        fetch_desc(seq + 1);
      }
      __syncwarp();
        }
      auto finish = [&]() {
        if (lane == 1) chain[(seq + 3u) & 3u].ticket = drawn;
        __syncwarp();
      };
      const ChainSlot& c = chain[seq & 3u];
      const uint32_t ticket = c.ticket;
      if (ticket >= P.nitems) {
        finish();
        return false;
      }
      const uint32_t tp = c.item.tensor_phase, chunk = c.item.chunk;
      const TensorDesc d = c.d;
      const uint4 nrm0 = *reinterpret_cast<const uint4*>(c.norm);  // as of one iteration ago
      const uint32_t t = tp & kTensorMask;
      const uint32_t phase = tp >> kPhaseShift;
      const bool want = needs_norms(phase);
      const bool have = !want || norms_final(nrm0, phase == kPhaseC);
      if (lane == 0 && want && have) {
        known_t = t;
        known_nrm = nrm0;
      }

      const int64_t start = (int64_t)chunk * kChunkElems;
      const int64_t left = d.numel - start;
      const int len = left < kChunkElems ? (int)left : kChunkElems;
      const bool bulk_ok = (d.flags & kFlagBulk) != 0;
      const uint64_t pol = (phase == kPhaseC) ? pol_stream : pol_keep;
      const int stage_cap = (phase == kPhaseA) ? kChunkElems : kStageElems;
      const int gran = 16 / (int)sizeof(GT);  // elements per 16 bytes of gradient
      // lane q (0..3) copies array q of every stage: g, p, m, v
      const char* my_src = lane == 0   ? static_cast<const char*>(d.g)
                           : lane == 1 ? reinterpret_cast<const char*>(d.p)
                           : lane == 2 ? reinterpret_cast<const char*>(d.m)
                                       : reinterpret_cast<const char*>(d.v);
      const uint32_t my_esize = lane == 0 ? (uint32_t)sizeof(GT) : 4u;
      const uint32_t my_dst_off = lane == 0 ? 0u : (uint32_t)(L::kGBytes + (lane - 1) * L::kFBytes);
      const bool my_copy = lane < (phase == kPhaseA ? 1 : 4);
      for (int off = 0; off < len; off += stage_cap) {
        const uint32_t slot = stage_ctr % kStages;
        const uint32_t use = stage_ctr / kStages;
        // A free slot: take it.  None free: settle pending stages first (their consumers
        // are what frees slots), and only with nothing pending wait for the consumers.
        if (lane == 0) {
          const uint32_t eb = bar_empty + 8 * slot, par = (use & 1u) ^ 1u;
          while (!failed && !mbar_try_wait(eb, par)) {
            if (pend_count > 0) {
              failed = resolve_oldest();
            } else {
              failed = ring_wait(eb, par, P.hdr, ticket, P.wait_ns) ? 0 : 1;
              break;
            }
          }
        }
        failed = __shfl_sync(0xffffffffu, failed, 0);
        if (failed) {
          finish();
          return false;
        }
        const int n = (len - off) < stage_cap ? (len - off) : stage_cap;
        const int nbulk = bulk_ok ? (n / gran) * gran : 0;
        const uint32_t full = bar_full + 8 * slot;
        {
        if (lane == 0) {
          StageMeta& mt = s_meta[slot];
          const int64_t e = start + off;
          mt.g = static_cast<const char*>(d.g) + e * (int64_t)sizeof(GT);
          mt.p = d.p + e;
          mt.m = d.m + e;
          mt.v = d.v + e;
          mt.out = d.out ? static_cast<char*>(d.out) + e * (int64_t)sizeof(OT) : nullptr;
          mt.ticket = ticket;
          mt.n = (uint32_t)n;
          mt.nbulk = (uint32_t)nbulk;
          mt.flags = phase | (off == 0 ? 4u : 0u) | (off + stage_cap >= len ? 8u : 0u);
          mt.tensor = t;
          mt.part_index = d.first_chunk + chunk;
          mt.nchunks = d.nchunks;
          mt.first_chunk = d.first_chunk;
          if (nbulk > 0) {
            const uint32_t gb = (uint32_t)nbulk * (uint32_t)sizeof(GT), fb = (uint32_t)nbulk * 4u;
            mbar_arrive_expect_tx(full, phase == kPhaseA ? gb : gb + 3u * fb);  // arrival 1 of 2
          } else {
            mbar_arrive(full);
          }
          // arrival 2 of 2: now if the norms are known, later otherwise
          const bool settled = !want || (known_t == t && norms_final(known_nrm, phase == kPhaseC));
          if (settled && pend_count == 0) {
            resolve_stage(slot, phase, known_nrm);
          } else {
            PendStage& ps = pend[(pend_head + pend_count) % kStages];
            ps.slot = slot;
            ps.phase = phase;
            ps.tensor = t;
            ps.ticket = ticket;
            ++pend_count;
          }
        }
        __syncwarp();
        }
        {
          if (my_copy && nbulk > 0)
            tma_load_1d(data_base + slot * L::kStageBytes + my_dst_off,
                        my_src + (start + off) * (int64_t)my_esize, (uint32_t)nbulk * my_esize, full,
                        pol);
          __syncwarp();
        }
        ++stage_ctr;
      }
      finish();
      return true;
    };
    for (uint32_t seq = 0; iteration(seq); ++seq) {
    }
    // settle what is still pending (each wait is bounded)
    if (lane == 0) {
      while (!failed && pend_count > 0) failed = resolve_oldest();
    }
    failed = __shfl_sync(0xffffffffu, failed, 0);
    if (lane == 0) cp_async_wait_all();  // nothing of this thread may still be in flight
    // Terminator.  Every stage published before it is consumed (its copies have
    // landed) before the consumers see it, so nothing is in flight when they leave.
    if (lane == 0) {
      const uint32_t slot = stage_ctr % kStages;
      if (ring_wait(bar_empty + 8 * slot, ((stage_ctr / kStages) & 1u) ^ 1u, P.hdr, kTicketEnd,
                    P.wait_ns)) {
        s_meta[slot].ticket = kTicketEnd;
        mbar_arrive(bar_full + 8 * slot);
        mbar_arrive(bar_full + 8 * slot);
      }
    }
    return;
  }

  if (warp == kConsumerWarps + 1) {
    // =============================== publisher ===============================
    for (uint32_t r = 0;; ++r) {
      const uint32_t buf = r % kRedSlots, use = r / kRedSlots;
      if (!ring_wait(red_full + 8 * buf, use & 1u, P.hdr, r, P.wait_ns)) return;
      const RedSlot& rs = s_red[buf];
      const uint32_t phase = rs.phase;
      if (phase == kRedEnd) return;
      const uint32_t t = rs.tensor, nchunks = rs.nchunks;
      const int nq = (phase == kPhaseA) ? 1 : 3;
      float sum = 0.f;
      if (lane < nq) {
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) sum += rs.val[lane][w];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(red_empty + 8 * buf);  // the slot has been read
      // lane q owns quantity q: A -> ||g||^2 ; B -> ||p||^2, ||update_m||^2, ||update_g||^2
      LansCtl* ctl = P.ctl + t;
      const int word = (phase == kPhaseA) ? 0 : 1 + lane;
      if (lane < nq) {
        atomicAdd(&ctl->sumsq[word], (double)sum);
        __threadfence();
      }
      __syncwarp();
      unsigned is_last = 0;
      if (lane == 0) {
        const unsigned old = atomicAdd(phase == kPhaseA ? &ctl->arrived_a : &ctl->arrived_b, 1u);
        is_last = (old + 1u == nchunks);
      }
      is_last = __shfl_sync(0xffffffffu, is_last, 0);
      if (is_last && lane < nq) {
        // Every chunk of the tensor has been added: publish the norm, value and
        // "final" bit in one word.
        __threadfence();
        const double total = *reinterpret_cast<volatile double*>(&ctl->sumsq[word]);
        *reinterpret_cast<volatile unsigned*>(&ctl->norm[word]) =
            __float_as_uint(sqrtf((float)total)) | kNormValid;
      }
    }
  }

  // ================================ consumers ================================
  // Thread `tid` owns, in every stage, the vectors of four elements at q*1024 + 4*tid:
  // 16-byte shared-memory reads without bank conflicts, coalesced 16-byte stores.
  // Lanes past the end of a ragged stage hold zeros, which add nothing to any sum.
  Policies pol;
  pol.init();
  float acc[3] = {0.f, 0.f, 0.f};
  uint32_t red_ctr = 0;
  // Hands this warp's sums of the finished item (or the end marker) to the publisher.
  auto hand_over = [&](uint32_t phase, uint32_t tensor, uint32_t part_index, uint32_t nchunks,
                       uint32_t first_chunk) {
    float v0 = 0.f, v1 = 0.f, v2 = 0.f;
    if (phase != kRedEnd) v0 = warp_sum(acc[0]);
    if (phase == kPhaseB) {
      v1 = warp_sum(acc[1]);
      v2 = warp_sum(acc[2]);
    }
    if (lane == 0) {
      const uint32_t buf = red_ctr % kRedSlots, use = red_ctr / kRedSlots;
      ring_wait(red_empty + 8 * buf, (use & 1u) ^ 1u, P.hdr, red_ctr, P.wait_ns);
      RedSlot& rs = s_red[buf];
      rs.val[0][warp] = v0;
      rs.val[1][warp] = v1;
      rs.val[2][warp] = v2;
      if (warp == 0) {
        rs.phase = phase;
        rs.tensor = tensor;
        rs.part_index = part_index;
        rs.nchunks = nchunks;
        rs.first_chunk = first_chunk;
      }
      mbar_arrive(red_full + 8 * buf);
    }
    ++red_ctr;
  };

  for (uint32_t stage_ctr = 0;; ++stage_ctr) {
    const uint32_t slot = stage_ctr % kStages;
    {
    if (!ring_wait(bar_full + 8 * slot, (stage_ctr / kStages) & 1u, P.hdr, stage_ctr, P.wait_ns))
      break;
        }
    const StageMeta& mt = s_meta[slot];
    if (mt.ticket == kTicketEnd) break;
    const uint32_t phase = mt.flags & 3u;
    const bool first = (mt.flags & 4u) != 0, last = (mt.flags & 8u) != 0;
    const int n = (int)mt.n, nbulk = (int)mt.nbulk;
    const GT* gg = static_cast<const GT*>(mt.g);
    const uint32_t tensor = mt.tensor, part_index = mt.part_index, nchunks = mt.nchunks,
                   first_chunk = mt.first_chunk;
    const unsigned char* sbase = smem + slot * L::kStageBytes;
    if (first) acc[0] = acc[1] = acc[2] = 0.f;

    if (phase == kPhaseA) {
      // The whole chunk of g sits in the stage: four vectors per thread.
      constexpr int kPasses = kChunkElems / (kConsumers * kVec);
      F4 rg[kPasses];
#pragma unroll
      for (int q = 0; q < kPasses; ++q) {
        const int e = q * (kConsumers * kVec) + tid * kVec;
        if (e < nbulk) {
          rg[q] = Elem<GT>::smem4(sbase + e * sizeof(GT));
        } else {
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            rg[q].x[j] = (e + j < n) ? Elem<GT>::to_f32(gg[e + j]) : 0.f;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * slot);  // values are in registers
#pragma unroll
      for (int q = 0; q < kPasses; ++q)
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float x = rg[q].x[j] * s1.gscale;
          acc[0] = fmaf(x, x, acc[0]);
        }
      if (last) hand_over(kPhaseA, tensor, part_index, nchunks, first_chunk);
      continue;
    }

    // ---- phases B and C: g, p, m, v of kStageElems elements ----
    float* gp = mt.p;
    float* gm = mt.m;
    float* gv = mt.v;
    OT* gout = static_cast<OT*>(mt.out);
    const float cs = mt.cs, ratio_m = mt.ratio_m, ratio_g = mt.ratio_g;
    const bool whole = nbulk == kStageElems;  // the common case: nothing ragged or unaligned
    F4 rg[kStageVecs], rp[kStageVecs], rm[kStageVecs], rv[kStageVecs];
    int cnt[kStageVecs];
#pragma unroll
    for (int q = 0; q < kStageVecs; ++q) {
      const int e = q * (kConsumers * kVec) + tid * kVec;
      if (whole || e < nbulk) {
        cnt[q] = kVec;
        rg[q] = Elem<GT>::smem4(sbase + e * sizeof(GT));
        rp[q] = Elem<float>::smem4(sbase + L::kGBytes + e * 4);
        rm[q] = Elem<float>::smem4(sbase + L::kGBytes + L::kFBytes + e * 4);
        rv[q] = Elem<float>::smem4(sbase + L::kGBytes + 2 * L::kFBytes + e * 4);
      } else {
        cnt[q] = e < n ? ((n - e) < kVec ? (n - e) : kVec) : 0;
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const bool ok = j < cnt[q];
          rg[q].x[j] = ok ? Elem<GT>::to_f32(gg[e + j]) : 0.f;
          rp[q].x[j] = ok ? gp[e + j] : 0.f;
          rm[q].x[j] = ok ? gm[e + j] : 0.f;
          rv[q].x[j] = ok ? gv[e + j] : 0.f;
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * slot);  // values are in registers

    if (phase == kPhaseB) {
#pragma unroll
      for (int q = 0; q < kStageVecs; ++q)
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          float um, ug, mm = rm[q].x[j], vv = rv[q].x[j];
          const float pp = rp[q].x[j];
          s1(rg[q].x[j], pp, mm, vv, cs, um, ug);
          acc[0] = fmaf(pp, pp, acc[0]);
          acc[1] = fmaf(um, um, acc[1]);
          acc[2] = fmaf(ug, ug, acc[2]);
        }
      if (last) hand_over(kPhaseB, tensor, part_index, nchunks, first_chunk);
    } else {  // phase C
#pragma unroll
      for (int q = 0; q < kStageVecs; ++q) {
        const int e = q * (kConsumers * kVec) + tid * kVec;
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          float um, ug;
          s1(rg[q].x[j], rp[q].x[j], rm[q].x[j], rv[q].x[j], cs, um, ug);
          // p - ratio_m*update_m - ratio_g*update_g  (:385; the ratios carry the minus sign)
          rp[q].x[j] = fmaf(ratio_g, ug, fmaf(ratio_m, um, rp[q].x[j]));
        }
        if (whole || e < nbulk) {  // aligned: 16-byte stores
          Elem<float>::template store4<kStream>(gp + e, rp[q], pol);
          Elem<float>::template store4<kStream>(gm + e, rm[q], pol);
          Elem<float>::template store4<kStream>(gv + e, rv[q], pol);
          if (gout) Elem<OT>::template store4<kStream>(gout + e, rp[q], pol);
        } else {
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            if (j < cnt[q]) {
              gp[e + j] = rp[q].x[j];
              gm[e + j] = rm[q].x[j];
              gv[e + j] = rv[q].x[j];
              if (gout) gout[e + j] = Elem<OT>::from_f32(rp[q].x[j]);
            }
        }
      }
    }
  }
  // No more stages (or a wait expired): release the publisher.
  hand_over(kRedEnd, 0, 0, 0, 0);
}

// ---- host side -----------------------------------------------------------------

// Orders the (tensor, chunk, phase) items of a list.  Dependencies always point
// to earlier positions.  Priority C > B > A keeps a tensor's update pass right
// behind its norm pass; `slack` items are placed between the last item of a
// phase and the first dependent item where other work is available, so that
// the dependent block rarely has to wait; `window` bounds how many chunks the
// B cursor may lead the C cursor (and A lead B) when there is a choice.
std::vector<Item> build_lans_schedule(const std::vector<uint32_t>& nchunks, bool with_a,
                                      int64_t window_chunks, int slack) {
  const int k = (int)nchunks.size();
  std::vector<Item> out;
  uint64_t total = 0;
  for (uint32_t n : nchunks) total += n;
  out.reserve(total * (with_a ? 3 : 2));
  struct Cursor {
    int t = 0;
    uint32_t c = 0;
    uint64_t emitted = 0;
  } A, B, Cc;
  auto skip_empty = [&](Cursor& cur) {
    while (cur.t < k && nchunks[cur.t] == 0) cur.t++;
  };
  skip_empty(A);
  skip_empty(B);
  skip_empty(Cc);
  std::vector<int64_t> done_a(k, -1), done_b(k, -1);
  auto emit = [&](Cursor& cur, int phase, std::vector<int64_t>* done) {
    const uint32_t chunk = cur.c;
    out.push_back(Item{((uint32_t)phase << kPhaseShift) | (uint32_t)cur.t, chunk});
    cur.emitted++;
    if (++cur.c == nchunks[cur.t]) {
      if (done) (*done)[cur.t] = (int64_t)out.size();
      cur.c = 0;
      cur.t++;
      skip_empty(cur);
    }
  };
  if (!with_a) A.t = k;
  // Round-robin: in every round each phase that may run emits one item.  The three passes
  // then advance at the same rate, reads and writes reach DRAM in a steady 2:1 mix, and a
  // block that holds an item whose norm is not final yet is one of few, not one of all:
  // measured 2.21 ms against 2.45 ms for "phase C first, in bursts" on the 335 M-element list.
  // Phase C trails phase B by the largest tensor seen so far, so on lists with tensors
  // beyond a few MB its reads come from DRAM, not from L2; schedules that kept it closer
  // (bursts, 2:1 to 8:1 catch-up) re-read less but stalled more and measured slower, and
  // visiting the tensors smallest first cut the DRAM reads by 12 % but left the huge ones
  // as an unoverlapped tail (2.33 ms); huge tensors first, the rest smallest first, with
  // phase C catching up to one tensor behind cut the reads by 7 % and took 2.39 ms (2.42 ms
  // with the tiny tensors left mixed among the medium ones).  Fewer
  // DRAM bytes did not buy time in any of them: what limits the kernel once phase C runs
  // close behind phase B is the wait for the norms, not bandwidth.
  while (Cc.t < k) {
    bool progressed = false;
    {
      const int64_t n = (int64_t)out.size();
      const bool c_ready = Cc.t < k && B.t > Cc.t;
      if (c_ready && (Cc.c > 0 || n - done_b[Cc.t] >= slack)) {
        emit(Cc, kPhaseC, nullptr);
        progressed = true;
      }
    }
    {
      const int64_t n = (int64_t)out.size();
      const bool b_ready = B.t < k && (!with_a || A.t > B.t);
      if (b_ready && (B.c > 0 || !with_a || n - done_a[B.t] >= slack) &&
          (int64_t)(B.emitted - Cc.emitted) < window_chunks) {
        emit(B, kPhaseB, &done_b);
        progressed = true;
      }
    }
    if (with_a && A.t < k && (int64_t)(A.emitted - B.emitted) < window_chunks + 2048) {
      emit(A, kPhaseA, &done_a);
      progressed = true;
    }
    if (!progressed) {  // slack or window not met anywhere: advance what the dependencies allow
      const bool b_ready = B.t < k && (!with_a || A.t > B.t);
      if (with_a && A.t < k) emit(A, kPhaseA, &done_a);
      else if (b_ready) emit(B, kPhaseB, &done_b);
      else emit(Cc, kPhaseC, nullptr);
    }
  }
  return out;
}

size_t lans_ctl_bytes(int k) { return 64 + sizeof(LansCtl) * (size_t)k; }

size_t lans_workspace_bytes(int k, uint32_t total_chunks) {
  (void)total_chunks;  // partial sums are accumulated per tensor, not stored per chunk
  return (lans_ctl_bytes(k) + 255) & ~(size_t)255;
}

template <typename GT, typename OT>
static int launch_lans_t(const rafb200_tensor_list_s* l, const LansParams& P, cudaStream_t s) {
  static int occ[64] = {0};
  const int dev = (l->device >= 0 && l->device < 64) ? l->device : 0;
  const int smem = LansSmem<GT>::kTotal;
  if (occ[dev] == 0) {
    RAFB200_CUDA(cudaFuncSetAttribute(lans_kernel<GT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, lans_kernel<GT, OT>, kLansThreads, smem) !=
            cudaSuccess || n <= 0)
      n = 1;
    occ[dev] = n;
  }
  // Persistent grid: every SM holds `occ` blocks; a cap leaves SMs to a concurrent collective.
  int64_t grid = (int64_t)l->sm_count * occ[dev];
  if (l->max_blocks > 0 && grid > l->max_blocks) grid = l->max_blocks;
  if (grid > (int64_t)P.nitems) grid = P.nitems;
  if (grid < 1) grid = 1;
  lans_kernel<GT, OT><<<(unsigned)grid, kLansThreads, smem, s>>>(P);
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

template <typename GT>
static int launch_lans_g(const rafb200_tensor_list_s* l, const LansParams& P, cudaStream_t s) {
  switch (l->out_dtype) {
    case RAFB200_F32: return launch_lans_t<GT, float>(l, P, s);
    case RAFB200_F16: return launch_lans_t<GT, __half>(l, P, s);
    default: return launch_lans_t<GT, __nv_bfloat16>(l, P, s);
  }
}

}  // namespace rafb200

using namespace rafb200;

// ---- scratch of rafb200_lans_tensor_static --------------------------------------
// Everything rafb200_lans keeps in caller-provided device memory (header, per-tensor
// control words, descriptor row, work-item table) for ONE tensor of at most
// kStaticMaxElems elements, as a statically allocated device array: every GPU that
// loads this library holds these 25 KB until the process exits.
constexpr int64_t kStaticMaxElems = 4ll << 20;                          // 4,194,304 elements
constexpr uint32_t kStaticMaxChunks = (uint32_t)(kStaticMaxElems / kChunkElems);  // 1024
constexpr size_t kStaticCtlOff = 64, kStaticDescOff = 256, kStaticItemsOff = 512;
constexpr size_t kStaticBytes = kStaticItemsOff + 3 * (size_t)kStaticMaxChunks * sizeof(Item);
static __device__ __align__(256) unsigned char g_lans_static_scratch[kStaticBytes];

// Device address of the array above, per device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use: the address has
// to be asked for, once per device, with that device current.
static void* g_lans_static_ptr[64] = {nullptr};

extern "C" {

size_t rafb200_lans_workspace_bytes(rafb200_tensor_list_t list) {
  if (!list) return 0;
  return lans_workspace_bytes(list->k, list->total_chunks);
}

int rafb200_lans(rafb200_tensor_list_t list, int step, const float* step_dev, float learning_rate,
                 float beta1, float beta2, float eps, int bias_correction, float weight_decay,
                 int grad_averaging, int mode, int normalize_grad, float grad_scale,
                 void* workspace, size_t workspace_bytes, void* stream) {
  RAFB200_REQUIRE(list, "rafb200_lans: NULL list");
  RAFB200_REQUIRE(list->bound && list->has_v, "rafb200_lans: bind g, p, m and v first");
  RAFB200_REQUIRE(step_dev != nullptr || step >= 1, "rafb200_lans: step counts from 1");
  RAFB200_REQUIRE(mode == 0 || mode == 1, "rafb200_lans: mode must be 0 (L2) or 1 (decoupled)");
  const size_t need = lans_workspace_bytes(list->k, list->total_chunks);
  RAFB200_REQUIRE(workspace && workspace_bytes >= need,
                  "rafb200_lans: workspace of %zu bytes required, got %zu", need, workspace_bytes);
  RAFB200_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0,
                  "rafb200_lans: workspace must be 16-byte aligned");
  if (list->total_chunks == 0) return RAFB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  LansParams P;
  P.descs = list->dev_desc;
  if (normalize_grad) {
    P.items = list->dev_lans_items;
    P.nitems = list->n_lans_items;
  } else {
    P.items = list->dev_lans_items_nonorm;
    P.nitems = list->n_lans_items_nonorm;
  }
  char* ws = static_cast<char*>(workspace);
  P.hdr = reinterpret_cast<LansHeader*>(ws);
  P.ctl = reinterpret_cast<LansCtl*>(ws + 64);
  P.s1.beta1 = beta1;
  P.s1.beta2 = beta2;
  P.s1.beta3 = (grad_averaging == 1) ? 1 - beta1 : 1.0f;  // lans.cc:106-109
  P.s1.one_minus_beta2 = 1 - beta2;
  P.s1.eps = eps;
  float bc1, bc2;
  bias_corrections(beta1, beta2, step_dev ? 1 : step, bias_correction, &bc1, &bc2);
  P.s1.inv_bc1 = 1.0f / bc1;
  P.s1.inv_bc2 = 1.0f / bc2;
  P.s1.wd = weight_decay;
  P.s1.gscale = grad_scale;
  P.s1.mode = mode;
  P.s1.normalize = normalize_grad ? 1 : 0;
  P.lr = learning_rate;
  P.step_dev = step_dev;
  P.bias_correction = bias_correction;
  P.wait_ns = 2000000000ull;  // two seconds: far beyond any legitimate wait

  RAFB200_CUDA(cudaMemsetAsync(workspace, 0, lans_ctl_bytes(list->k), s));
  if (step_dev) {
    lans_bias_kernel<<<1, 1, 0, s>>>(P.hdr, step_dev, beta1, beta2, bias_correction);
    RAFB200_CUDA(cudaGetLastError());
  }
  switch (list->g_dtype) {
    case RAFB200_F32: return launch_lans_g<float>(list, P, s);
    case RAFB200_F16: return launch_lans_g<__half>(list, P, s);
    default: return launch_lans_g<__nv_bfloat16>(list, P, s);
  }
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
    g_lans_static_ptr[device] = ptr;
  }
  char* ws = static_cast<char*>(g_lans_static_ptr[device]);

  // One-tensor list on the host stack: nothing here touches a device allocator.
  rafb200_tensor_list_s one;
  one.k = 1;
  one.g_dtype = g_dtype;
  one.out_dtype = out_dtype;
  one.device = device;
  RAFB200_CUDA(cudaDeviceGetAttribute(&one.sm_count, cudaDevAttrMultiProcessorCount, device));
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
  if (vec_ok && a16(g)) d.flags |= kFlagBulk;
  const std::vector<Item> items =
      build_lans_schedule(std::vector<uint32_t>{d.nchunks}, normalize_grad != 0,
                          (int64_t)kStaticMaxChunks, 0);

  LansParams P;
  P.descs = reinterpret_cast<const TensorDesc*>(ws + kStaticDescOff);
  P.items = reinterpret_cast<const Item*>(ws + kStaticItemsOff);
  P.nitems = (uint32_t)items.size();
  P.hdr = reinterpret_cast<LansHeader*>(ws);
  P.ctl = reinterpret_cast<LansCtl*>(ws + kStaticCtlOff);
  P.s1.beta1 = beta1;
  P.s1.beta2 = beta2;
  P.s1.beta3 = (grad_averaging == 1) ? 1 - beta1 : 1.0f;
  P.s1.one_minus_beta2 = 1 - beta2;
  P.s1.eps = eps;
  float bc1, bc2;
  bias_corrections(beta1, beta2, step, bias_correction, &bc1, &bc2);
  P.s1.inv_bc1 = 1.0f / bc1;
  P.s1.inv_bc2 = 1.0f / bc2;
  P.s1.wd = weight_decay;
  P.s1.gscale = grad_scale;
  P.s1.mode = mode;
  P.s1.normalize = normalize_grad ? 1 : 0;
  P.lr = learning_rate;
  P.step_dev = nullptr;
  P.bias_correction = bias_correction;
  P.wait_ns = 2000000000ull;

  // The array keeps whatever the previous call left in it: ticket counter, error word,
  // arrival counters, sums and norm words must start at zero; descriptor and item table
  // are rewritten.  (Pageable sources: the runtime stages them before returning.)
  RAFB200_CUDA(cudaMemsetAsync(ws, 0, kStaticCtlOff + sizeof(LansCtl), s));
  RAFB200_CUDA(cudaMemcpyAsync(ws + kStaticDescOff, &d, sizeof(d), cudaMemcpyHostToDevice, s));
  RAFB200_CUDA(cudaMemcpyAsync(ws + kStaticItemsOff, items.data(), items.size() * sizeof(Item),
                               cudaMemcpyHostToDevice, s));
  switch (g_dtype) {
    case RAFB200_F32: return launch_lans_g<float>(&one, P, s);
    case RAFB200_F16: return launch_lans_g<__half>(&one, P, s);
    default: return launch_lans_g<__nv_bfloat16>(&one, P, s);
  }
}

int rafb200_lans_schedule(int k, const int64_t* numel, int with_norm_phase, int64_t window_elems,
                          int slack_items, uint32_t* items, size_t capacity, size_t* count) {
  RAFB200_REQUIRE(k >= 0 && (k == 0 || numel) && count && window_elems >= 0 && slack_items >= 0,
                  "rafb200_lans_schedule: bad arguments");
  std::vector<uint32_t> nchunks(k);
  for (int i = 0; i < k; ++i) {
    RAFB200_REQUIRE(numel[i] >= 0, "rafb200_lans_schedule: numel[%d] < 0", i);
    nchunks[i] = (uint32_t)((numel[i] + kChunkElems - 1) / kChunkElems);
  }
  int64_t window_chunks = window_elems / kChunkElems;
  if (window_chunks < 1) window_chunks = 1;
  const std::vector<Item> sched = build_lans_schedule(nchunks, with_norm_phase != 0, window_chunks, slack_items);
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

int rafb200_lans_status(rafb200_tensor_list_t list, const void* workspace, float* norms_host,
                        void* stream) {
  RAFB200_REQUIRE(list && workspace, "rafb200_lans_status: NULL argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RAFB200_CUDA(cudaStreamSynchronize(s));
  std::vector<char> host(lans_ctl_bytes(list->k));
  RAFB200_CUDA(cudaMemcpy(host.data(), workspace, host.size(), cudaMemcpyDeviceToHost));
  const LansHeader* hdr = reinterpret_cast<const LansHeader*>(host.data());
  const LansCtl* ctl = reinterpret_cast<const LansCtl*>(host.data() + 64);
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
