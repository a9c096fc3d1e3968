// Collectives over symmetric (peer-mapped, optionally multicast-bound) memory; see symm.cu.
#pragma once
#include "common.h"

namespace rafb200 {

constexpr int kSymmLanes = 4;       // independent barrier sequences per signal pad
constexpr size_t kSymmSignalBytes = kSymmLanes * kSymmMaxWorld * sizeof(uint32_t);

// The same buffer as seen on every rank, mapped into this process; entry `rank` is local.
struct SymmPeers {
  void* ptr[kSymmMaxWorld];
};

// Cross-GPU flag barrier on `lane` (epochs grow by one per call, in the same order on every rank).
// A wait that exceeds `limit_ns` records (lane, late rank) in *err and, when host_err is not
// NULL, in that word of host-mapped memory as well; later barriers then pass without waiting.
int symm_barrier(const SymmPeers& sig, int world, int rank, int lane, uint32_t epoch, uint64_t limit_ns,
                 unsigned int* err, unsigned int* host_err, cudaStream_t s);
constexpr int kSymmChunkBytes = 32768;  // bytes per work item of the collective kernels

// This rank's row block of one tensor inside the symmetric buffer.
struct SymmSeg {
  size_t off;      // byte offset from the start of the symmetric buffer, a multiple of 16
  size_t dst_off;  // reduce-scatter only: byte offset of the result in the local output buffer
  int64_t bytes;   // a multiple of 16
};

// out[seg.dst_off ..] = sum over ranks of buffer[seg.off ..] for every segment; `out` is a plain
// local buffer, so the callers' data in the symmetric buffer stays as it was; mc = multicast
// address or NULL.
// `items` lists (segment, 32 KB chunk) pairs; segs and items are device arrays.
int symm_reduce_scatter(const SymmPeers& peers, const void* mc, void* out, const SymmSeg* segs,
                        const Item* items, uint32_t nitems, int dtype, int world, int blocks, cudaStream_t s);
// buffer[seg] on every rank = local[seg] for every segment.
int symm_allgather(const SymmPeers& peers, void* mc, const void* local, const SymmSeg* segs, const Item* items,
                   uint32_t nitems, int world, int rank, int blocks, cudaStream_t s);

}  // namespace rafb200
