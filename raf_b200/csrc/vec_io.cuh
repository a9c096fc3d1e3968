// Device helpers: 4-element vector loads/stores for fp32 / fp16 / bf16 arrays
// with optional L2 eviction hints, exact (unfused) fp32 arithmetic wrappers,
// and deterministic block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rafb200 {

// L2 eviction hint attached to a load or store.
//   kStream : touched once, make it the first candidate for eviction
//   kKeep   : will be read again soon by another block, keep it resident
//   kDefault: no hint
enum CacheHint { kDefault = 0, kStream = 1, kKeep = 2 };

__device__ __forceinline__ uint64_t make_policy_stream() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t make_policy_keep() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

struct Policies {
  uint64_t stream;
  uint64_t keep;
  __device__ __forceinline__ void init() {
    stream = make_policy_stream();
    keep = make_policy_keep();
  }
  template <int H>
  __device__ __forceinline__ uint64_t get() const {
    return H == kKeep ? keep : stream;
  }
};

// ---- raw 16-byte / 8-byte accesses ---------------------------------------
template <int H>
__device__ __forceinline__ uint4 ld16(const void* p, const Policies& pol) {
  uint4 r;
  if (H == kDefault) {
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
  } else {
    asm volatile("ld.global.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p), "l"(pol.get<H>()));
  }
  return r;
}
template <int H>
__device__ __forceinline__ uint2 ld8(const void* p, const Policies& pol) {
  uint2 r;
  if (H == kDefault) {
    asm volatile("ld.global.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  } else {
    asm volatile("ld.global.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;"
                 : "=r"(r.x), "=r"(r.y)
                 : "l"(p), "l"(pol.get<H>()));
  }
  return r;
}
template <int H>
__device__ __forceinline__ void st16(void* p, uint4 v, const Policies& pol) {
  if (H == kDefault) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
  } else {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol.get<H>())
                 : "memory");
  }
}
template <int H>
__device__ __forceinline__ void st8(void* p, uint2 v, const Policies& pol) {
  if (H == kDefault) {
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
  } else {
    asm volatile("st.global.L2::cache_hint.v2.u32 [%0], {%1,%2}, %3;" ::"l"(p), "r"(v.x),
                 "r"(v.y), "l"(pol.get<H>())
                 : "memory");
  }
}

// ---- typed 4-element groups --------------------------------------------
struct F4 {
  float x[4];
};
__device__ __forceinline__ F4 f4_zero() {
  F4 o;
  o.x[0] = o.x[1] = o.x[2] = o.x[3] = 0.f;
  return o;
}

template <typename T>
struct Elem;  // scalar conversion + raw vector width

template <>
struct Elem<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
  // four elements from (16-byte aligned) shared memory
  static __device__ __forceinline__ F4 smem4(const void* p) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    F4 o;
    o.x[0] = q.x;
    o.x[1] = q.y;
    o.x[2] = q.z;
    o.x[3] = q.w;
    return o;
  }
  template <int H>
  static __device__ __forceinline__ F4 load4(const float* p, const Policies& pol) {
    uint4 r = ld16<H>(p, pol);
    F4 o;
    o.x[0] = __uint_as_float(r.x);
    o.x[1] = __uint_as_float(r.y);
    o.x[2] = __uint_as_float(r.z);
    o.x[3] = __uint_as_float(r.w);
    return o;
  }
  template <int H>
  static __device__ __forceinline__ void store4(float* p, const F4& v, const Policies& pol) {
    uint4 r;
    r.x = __float_as_uint(v.x[0]);
    r.y = __float_as_uint(v.x[1]);
    r.z = __float_as_uint(v.x[2]);
    r.w = __float_as_uint(v.x[3]);
    st16<H>(p, r, pol);
  }
};

template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ F4 smem4(const void* p) {  // 8-byte aligned shared memory
    uint2 r = *reinterpret_cast<const uint2*>(p);
    float2 fa = __half22float2(*reinterpret_cast<__half2*>(&r.x));
    float2 fb = __half22float2(*reinterpret_cast<__half2*>(&r.y));
    F4 o;
    o.x[0] = fa.x;
    o.x[1] = fa.y;
    o.x[2] = fb.x;
    o.x[3] = fb.y;
    return o;
  }
  template <int H>
  static __device__ __forceinline__ F4 load4(const __half* p, const Policies& pol) {
    uint2 r = ld8<H>(p, pol);
    __half2 a = *reinterpret_cast<__half2*>(&r.x);
    __half2 b = *reinterpret_cast<__half2*>(&r.y);
    float2 fa = __half22float2(a), fb = __half22float2(b);
    F4 o;
    o.x[0] = fa.x;
    o.x[1] = fa.y;
    o.x[2] = fb.x;
    o.x[3] = fb.y;
    return o;
  }
  template <int H>
  static __device__ __forceinline__ void store4(__half* p, const F4& v, const Policies& pol) {
    __half2 a = __floats2half2_rn(v.x[0], v.x[1]);
    __half2 b = __floats2half2_rn(v.x[2], v.x[3]);
    uint2 r;
    r.x = *reinterpret_cast<unsigned*>(&a);
    r.y = *reinterpret_cast<unsigned*>(&b);
    st8<H>(p, r, pol);
  }
};

template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) {
    return __float2bfloat16_rn(v);
  }
  static __device__ __forceinline__ F4 smem4(const void* p) {  // 8-byte aligned shared memory
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    F4 o;
    o.x[0] = __uint_as_float(r.x << 16);
    o.x[1] = __uint_as_float(r.x & 0xffff0000u);
    o.x[2] = __uint_as_float(r.y << 16);
    o.x[3] = __uint_as_float(r.y & 0xffff0000u);
    return o;
  }
  template <int H>
  static __device__ __forceinline__ F4 load4(const __nv_bfloat16* p, const Policies& pol) {
    uint2 r = ld8<H>(p, pol);
    F4 o;  // bf16 -> fp32 is a 16-bit shift
    o.x[0] = __uint_as_float(r.x << 16);
    o.x[1] = __uint_as_float(r.x & 0xffff0000u);
    o.x[2] = __uint_as_float(r.y << 16);
    o.x[3] = __uint_as_float(r.y & 0xffff0000u);
    return o;
  }
  template <int H>
  static __device__ __forceinline__ void store4(__nv_bfloat16* p, const F4& v,
                                                const Policies& pol) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x[0], v.x[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v.x[2], v.x[3]);
    uint2 r;
    r.x = *reinterpret_cast<unsigned*>(&a);
    r.y = *reinterpret_cast<unsigned*>(&b);
    st8<H>(p, r, pol);
  }
};

// ---- exact fp32 arithmetic (never contracted into fused multiply-add) -----
__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float fsqrt(float a) { return __fsqrt_rn(a); }

// ---- block reductions (fixed order: xor-shuffle tree, then warps 0..W-1) ---
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sums N values per thread over the block; result valid in every thread.
// `smem` needs N * (blockDim.x/32) floats.  Contains two __syncthreads().
template <int N>
__device__ __forceinline__ void block_sum(float (&v)[N], float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = warp_sum(v[i]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) smem[i * nwarp + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float s = 0.f;
    for (int w = 0; w < nwarp; ++w) s += smem[i * nwarp + w];
    v[i] = s;
  }
  __syncthreads();
}

// ---- flags ---------------------------------------------------------------
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

}  // namespace rafb200
