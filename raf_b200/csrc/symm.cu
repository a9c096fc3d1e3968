// Collectives of the ZeRO step over symmetric memory: every rank's bucket buffer is mapped
// into every process (peer pointers) and, where the NVSwitch offers it, bound to one
// multicast address.  Reduce-scatter is then a `multimem.ld_reduce` of this rank's slot
// (the switch fetches the slot from every GPU and returns the sum, accumulated in fp32),
// all-gather a `multimem.st` of this rank's slot (the switch stores it into every GPU).
// Per direction a rank moves (n-1)/n of a bucket for the pair instead of twice that with a
// ring, and the two run in opposite directions, so they overlap.  Without a multicast
// address the same kernels read / write the peers one by one.
//
// No kernel here waits on another kernel of the same GPU.  The only cross-GPU wait is the
// flag barrier below; it is bounded by a clock and reports expiry instead of hanging.
#include "symm.h"

#include "symm_dev.cuh"
#include "vec_io.cuh"

namespace rafb200 {

__device__ __forceinline__ uint64_t symm_now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- flag barrier across GPUs ----------------------------------------------------
// Rank r stores `epoch` into word [lane][r] of every rank's signal pad, then waits until
// every word [lane][q] of its own pad has reached `epoch`.  Epochs only grow, so a peer
// that is already one barrier ahead does no harm.  Work issued before the barrier in
// stream order is complete, hence published by the release stores; work issued after it
// starts only when every peer has arrived.
__global__ void xbarrier_kernel(SymmPeers sig, int world, int rank, int lane, uint32_t epoch,
                                uint64_t timeout_ns, unsigned int* err, unsigned int* host_err) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  uint32_t* remote = static_cast<uint32_t*>(sig.ptr[t]) + lane * kSymmMaxWorld + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const uint32_t* mine = static_cast<const uint32_t*>(sig.ptr[rank]) + lane * kSymmMaxWorld + t;
  const uint64_t t0 = symm_now_ns();
  // After a first expiry the step is lost anyway: later barriers do not wait again.
  if (*reinterpret_cast<volatile unsigned int*>(err) != 0) return;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) break;
    if (symm_now_ns() - t0 > timeout_ns) {  // a peer never arrived: report, do not hang
      const unsigned code = 0x100u | (unsigned)(lane << 4) | (unsigned)t;
      if (atomicCAS(err, 0u, code) == 0u && host_err != nullptr) {
        *reinterpret_cast<volatile unsigned int*>(host_err) = code;  // the host reads it without a sync
        __threadfence_system();
      }
      break;
    }
    __nanosleep(200);
  }
}

constexpr int kSymmThreads = 256;
constexpr int kSymmUnroll = 8;  // 16-byte accesses in flight per thread
static_assert(kSymmThreads * kSymmUnroll * 16 == kSymmChunkBytes, "one work item = one pass of a block");

// A work item = one 32 KB chunk of one segment; a segment = this rank's row block of one
// tensor, `off` bytes into the (symmetric) buffer, a multiple of 16 bytes long.
// Reduce-scatter: out[dst_off..] = sum over ranks of buffer[off..].
template <int DT, bool MC>
__global__ void __launch_bounds__(kSymmThreads)
    symm_reduce_scatter_kernel(SymmPeers peers, const char* mc, char* local, const SymmSeg* __restrict__ segs,
                               const Item* __restrict__ items, uint32_t nitems, int world) {
  for (uint32_t it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item item = items[it];
    const SymmSeg sg = segs[item.tensor_phase];
    const size_t base = sg.off + (size_t)item.chunk * kSymmChunkBytes;
    const size_t dst = sg.dst_off + (size_t)item.chunk * kSymmChunkBytes;
    int64_t left = sg.bytes - (int64_t)item.chunk * kSymmChunkBytes;
    const int nvec = (int)((left > kSymmChunkBytes ? kSymmChunkBytes : left) >> 4);
    uint4 out[kSymmUnroll];
#pragma unroll
    for (int u = 0; u < kSymmUnroll; ++u) {
      const int i = threadIdx.x + u * kSymmThreads;
      if (i >= nvec) continue;
      if (MC) {
        out[u] = mc_ld_reduce<DT>(mc + base + (size_t)i * 16);
      } else {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int q = 0; q < world; ++q)  // fixed order: the same bits on every run
          accumulate<DT>(acc, peer_ld(static_cast<const char*>(peers.ptr[q]) + base + (size_t)i * 16));
        out[u] = round_once<DT>(acc);
      }
    }
#pragma unroll
    for (int u = 0; u < kSymmUnroll; ++u) {
      const int i = threadIdx.x + u * kSymmThreads;
      if (i < nvec) *reinterpret_cast<uint4*>(local + dst + (size_t)i * 16) = out[u];
    }
  }
}

// All-gather: buffer[off..] on every rank = local[off..].
template <bool MC>
__global__ void __launch_bounds__(kSymmThreads)
    symm_allgather_kernel(SymmPeers peers, char* mc, const char* local, const SymmSeg* __restrict__ segs,
                          const Item* __restrict__ items, uint32_t nitems, int world, int rank) {
  for (uint32_t it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item item = items[it];
    const SymmSeg sg = segs[item.tensor_phase];
    const size_t base = sg.off + (size_t)item.chunk * kSymmChunkBytes;
    int64_t left = sg.bytes - (int64_t)item.chunk * kSymmChunkBytes;
    const int nvec = (int)((left > kSymmChunkBytes ? kSymmChunkBytes : left) >> 4);
    uint4 v[kSymmUnroll];
#pragma unroll
    for (int u = 0; u < kSymmUnroll; ++u) {
      const int i = threadIdx.x + u * kSymmThreads;
      if (i < nvec) v[u] = *reinterpret_cast<const uint4*>(local + base + (size_t)i * 16);
    }
#pragma unroll
    for (int u = 0; u < kSymmUnroll; ++u) {
      const int i = threadIdx.x + u * kSymmThreads;
      if (i >= nvec) continue;
      if (MC) {
        mc_st(mc + base + (size_t)i * 16, v[u]);
      } else {
        for (int q = 0; q < world; ++q)
          if (q != rank) *reinterpret_cast<uint4*>(static_cast<char*>(peers.ptr[q]) + base + (size_t)i * 16) = v[u];
      }
    }
  }
}

static unsigned symm_grid(uint32_t nitems, int blocks) {
  int64_t g = nitems < (uint32_t)blocks ? nitems : blocks;
  return (unsigned)(g < 1 ? 1 : g);
}

int symm_barrier(const SymmPeers& sig, int world, int rank, int lane, uint32_t epoch, uint64_t limit_ns,
                 unsigned int* err, unsigned int* host_err, cudaStream_t s) {
  xbarrier_kernel<<<1, 32, 0, s>>>(sig, world, rank, lane, epoch, limit_ns, err, host_err);
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

template <int DT>
static int launch_rs(const SymmPeers& peers, const void* mc, void* local, const SymmSeg* segs, const Item* items,
                     uint32_t nitems, int world, int blocks, cudaStream_t s) {
  const unsigned g = symm_grid(nitems, blocks);
  if (mc)
    symm_reduce_scatter_kernel<DT, true><<<g, kSymmThreads, 0, s>>>(peers, static_cast<const char*>(mc),
                                                                    static_cast<char*>(local), segs, items, nitems, world);
  else
    symm_reduce_scatter_kernel<DT, false><<<g, kSymmThreads, 0, s>>>(peers, nullptr, static_cast<char*>(local),
                                                                     segs, items, nitems, world);
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

int symm_reduce_scatter(const SymmPeers& peers, const void* mc, void* local, const SymmSeg* segs,
                        const Item* items, uint32_t nitems, int dtype, int world, int blocks, cudaStream_t s) {
  if (nitems == 0) return RAFB200_OK;
  switch (dtype) {
    case RAFB200_F32: return launch_rs<RAFB200_F32>(peers, mc, local, segs, items, nitems, world, blocks, s);
    case RAFB200_F16: return launch_rs<RAFB200_F16>(peers, mc, local, segs, items, nitems, world, blocks, s);
    default: return launch_rs<RAFB200_BF16>(peers, mc, local, segs, items, nitems, world, blocks, s);
  }
}

int symm_allgather(const SymmPeers& peers, void* mc, const void* local, const SymmSeg* segs, const Item* items,
                   uint32_t nitems, int world, int rank, int blocks, cudaStream_t s) {
  if (nitems == 0) return RAFB200_OK;
  const unsigned g = symm_grid(nitems, blocks);
  if (mc)
    symm_allgather_kernel<true><<<g, kSymmThreads, 0, s>>>(peers, static_cast<char*>(mc),
                                                          static_cast<const char*>(local), segs, items, nitems, world, rank);
  else
    symm_allgather_kernel<false><<<g, kSymmThreads, 0, s>>>(peers, nullptr, static_cast<const char*>(local), segs,
                                                           items, nitems, world, rank);
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

}  // namespace rafb200
