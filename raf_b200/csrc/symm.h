// Collectives over symmetric (peer-mapped, optionally multicast-bound) memory; see symm.cu.
#pragma once
#include "common.h"

namespace rafb200 {

constexpr int kSymmMaxWorld = 16;   // ranks of one NVLink domain addressed by value
constexpr int kSymmLanes = 4;       // independent barrier sequences per signal pad
constexpr size_t kSymmSignalBytes = kSymmLanes * kSymmMaxWorld * sizeof(uint32_t);

// The same buffer as seen on every rank, mapped into this process; entry `rank` is local.
struct SymmPeers {
  void* ptr[kSymmMaxWorld];
};

// Cross-GPU flag barrier on `lane` (epochs grow by one per call, in the same order on every rank).
int symm_barrier(const SymmPeers& sig, int world, int rank, int lane, uint32_t epoch,
                 unsigned int* err, cudaStream_t s);
// dst[0..bytes) = sum over ranks of (buffer + off)[0..bytes); mc = multicast address or NULL.
int symm_reduce_scatter(const SymmPeers& peers, const void* mc, size_t off, void* dst, int64_t bytes,
                        int dtype, int world, int blocks, cudaStream_t s);
// (buffer + off)[0..bytes) on every rank = src[0..bytes).
int symm_allgather(const SymmPeers& peers, void* mc, size_t off, const void* src, int64_t bytes, int world,
                   int rank, int blocks, cudaStream_t s);

}  // namespace rafb200
