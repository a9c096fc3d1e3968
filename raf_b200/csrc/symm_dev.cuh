// Device-side access to symmetric memory: multimem loads / stores through the NVSwitch
// multicast address and plain loads from a peer's mapping, 16 bytes per call, plus the
// fp32 accumulation and single rounding the reductions share.  Used by the collective
// kernels (symm.cu) and by the LANS kernel when it reads its gradients through the switch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "vec_io.cuh"

namespace rafb200 {

template <int DT>
__device__ __forceinline__ uint4 mc_ld_reduce(const void* mc) {
  uint4 r;
  if (DT == RAFB200_F16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  } else if (DT == RAFB200_BF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  }
  return r;
}

__device__ __forceinline__ void mc_st(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint4 peer_ld(const void* p) {
  uint4 r;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}

template <int DT>
__device__ __forceinline__ void accumulate(float (&acc)[8], uint4 v) {
  if (DT == RAFB200_F32) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f;
      if (DT == RAFB200_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
}

template <int DT>
__device__ __forceinline__ uint4 round_once(const float (&acc)[8]) {
  uint4 r;
  if (DT == RAFB200_F32) {
    r.x = __float_as_uint(acc[0]);
    r.y = __float_as_uint(acc[1]);
    r.z = __float_as_uint(acc[2]);
    r.w = __float_as_uint(acc[3]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (DT == RAFB200_F16) {
        __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    r = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return r;
}


// Four elements of the gradient dtype, summed over the ranks: 16 bytes (fp32) or 8 bytes
// (16-bit types) per access, through the multicast address or peer by peer in a fixed order,
// fp32 accumulation and one rounding either way.  -> the rounded sum as floats, and its bits.
template <int DT>
__device__ __forceinline__ void reduced4(const char* mc, const char* const* peer, int world, size_t off,
                                         float (&x)[4], uint32_t (&bits)[4]) {
  if (DT == RAFB200_F32) {
    uint4 r;
    if (mc) {
      r = mc_ld_reduce<DT>(mc + off);
    } else {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = 0; q < world; ++q) accumulate<DT>(acc, peer_ld(peer[q] + off));
      r = round_once<DT>(acc);
    }
    bits[0] = r.x; bits[1] = r.y; bits[2] = r.z; bits[3] = r.w;
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = __uint_as_float(bits[j]);
  } else {
    uint2 r;
    if (mc) {
      if (DT == RAFB200_F16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.f16x2 {%0,%1}, [%2];"
                     : "=r"(r.x), "=r"(r.y) : "l"(mc + off) : "memory");
      else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.bf16x2 {%0,%1}, [%2];"
                     : "=r"(r.x), "=r"(r.y) : "l"(mc + off) : "memory");
    } else {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = 0; q < world; ++q) {
        uint2 t;
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(t.x), "=r"(t.y) : "l"(peer[q] + off) : "memory");
        accumulate<DT>(acc, make_uint4(t.x, t.y, 0u, 0u));
      }
      const uint4 w = round_once<DT>(acc);
      r = make_uint2(w.x, w.y);
    }
    bits[0] = r.x; bits[1] = r.y; bits[2] = 0; bits[3] = 0;
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    accumulate<DT>(f, make_uint4(r.x, r.y, 0u, 0u));
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = f[j];
  }
}

// 8 bytes through the multicast address (four 16-bit elements)
__device__ __forceinline__ void mc_st8(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}


// Four elements of the model-dtype copy into every rank's parameter buffer: `local` lies in
// this rank's mapping p_peer[rank]; one multimem.st through p_mc, or one store per rank.
template <typename OT>
__device__ __forceinline__ void store4_everywhere(char* p_mc, char* const* p_peer, int world, int rank, OT* local,
                                                  const F4& v) {
  uint32_t w[4];
  if (sizeof(OT) == 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = __float_as_uint(v.x[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const OT lo = Elem<OT>::from_f32(v.x[2 * j]), hi = Elem<OT>::from_f32(v.x[2 * j + 1]);
      w[j] = (uint32_t)(*reinterpret_cast<const unsigned short*>(&lo)) |
             ((uint32_t)(*reinterpret_cast<const unsigned short*>(&hi)) << 16);
    }
  }
  const size_t delta = (size_t)(reinterpret_cast<char*>(local) - p_peer[rank]);
  if (p_mc) {
    if (sizeof(OT) == 4) mc_st(p_mc + delta, make_uint4(w[0], w[1], w[2], w[3]));
    else mc_st8(p_mc + delta, make_uint2(w[0], w[1]));
  } else {
    for (int q = 0; q < world; ++q) {
      char* dst = p_peer[q] + delta;
      if (sizeof(OT) == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
      else *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    }
  }
}
template <typename OT>
__device__ __forceinline__ void store1_everywhere(char* const* p_peer, int world, int rank, OT* local, float x) {
  const size_t delta = (size_t)(reinterpret_cast<char*>(local) - p_peer[rank]);
  const OT val = Elem<OT>::from_f32(x);
  for (int q = 0; q < world; ++q) *reinterpret_cast<OT*>(p_peer[q] + delta) = val;
}

}  // namespace rafb200
