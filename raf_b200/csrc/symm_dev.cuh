// Device-side access to symmetric memory: multimem loads / stores through the NVSwitch
// multicast address and plain loads from a peer's mapping, 16 bytes per call, plus the
// fp32 accumulation and single rounding the reductions share.  Used by the collective
// kernels (symm.cu) and by the LANS kernel when it reads its gradients through the switch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"

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


// 8 bytes through the multicast address (four 16-bit elements)
__device__ __forceinline__ void mc_st8(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}

}  // namespace rafb200
