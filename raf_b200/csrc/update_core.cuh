// Chunk-level building blocks shared by the SGD / Adam kernels and the LANS
// persistent kernel: a block of kBlockThreads threads walks one chunk
// (<= kChunkElems elements of one tensor) with 16-byte accesses, two vector
// passes in flight per thread, and falls back to scalar accesses for unaligned
// tensors and ragged tails.
#pragma once
#include "common.h"
#include "vec_io.cuh"

namespace rafb200 {

constexpr int kVec = 4;                              // elements per thread per pass
constexpr int kPassElems = kBlockThreads * kVec;     // 1024
constexpr int kUnroll = 2;                           // passes in flight
constexpr uint32_t kFlagAligned = 1u;  // vector accesses allowed (16 B fp32, 8 B 16-bit arrays)
constexpr uint32_t kFlagBulk = 2u;     // every array is 16-byte aligned: TMA bulk copies allowed

// ---- per-element arithmetic -------------------------------------------------
// All three follow the reference expression by expression; see the C ABI
// header for the citations.  Every operation is a separately rounded fp32 op.

struct SgdOp {
  float lr, mu, wd, gscale;
  // v1 = mu*v0 + dx ; x1 = x0 - lr*v1      (python/raf/_tvm_op/sgd.py:21-29)
  __device__ __forceinline__ void operator()(float g, float& p, float& m, float& /*v*/) const {
    if (gscale != 1.0f) g = mul(g, gscale);
    if (wd != 0.0f) g = add(g, mul(wd, p));
    float v1 = add(mul(mu, m), g);
    p = sub(p, mul(lr, v1));
    m = v1;
  }
};

struct AdamOp {
  float lr, beta1, beta2, beta3, one_minus_beta2, eps, bc1, bc2, wd, gscale;
  int mode;
  __device__ __forceinline__ void operator()(float g, float& p, float& m, float& v) const {
    if (gscale != 1.0f) g = mul(g, gscale);
    if (mode == 0) g = add(g, mul(wd, p));
    m = add(mul(m, beta1), mul(beta3, g));
    v = add(mul(v, beta2), mul(mul(one_minus_beta2, g), g));
    float denom = add(fsqrt(fdiv(v, bc2)), eps);
    float update = fdiv(fdiv(m, bc1), denom);
    if (mode != 0) update = add(update, mul(wd, p));
    p = sub(p, mul(lr, update));
  }
};

// LANS stage 1 (src/op/dialect/cuda/kernels/multi_tensor_lans.cu:281-306).
// The reference divides five times and takes one square root per element; at
// 28 bytes per element that is more arithmetic than a B200 SM can issue in the
// time HBM delivers the data (two passes need it).  The divisions by values
// that are constant per call or per tensor (bias corrections, ||g||+eps) become
// multiplications by reciprocals computed once, the two divisions by the
// denominator share one reciprocal, and sqrt / reciprocal use the 1-ulp hardware
// approximations (flush-to-zero forms: the square root's argument only matters
// when it is far above the denormal range, and the reciprocal's is >= eps).
// Each substitution moves a result by at most about one unit
// in the last place (1.2e-7 relative); the tests bound the total against the
// exact restatement at 2e-6 for m and v and far less for p.
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float sqrt_approx(float x) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct LansStage1 {
  float beta1, beta2, beta3, one_minus_beta2, eps, inv_bc1, inv_bc2, wd, gscale;
  int mode, normalize;
  // Multiplier that turns a raw gradient element into the scaled gradient:
  // grad_scale / (||g|| + eps) when gradients are normalised and ||g|| != 0.
  __device__ __forceinline__ float grad_multiplier(float gnorm) const {
    if (normalize && gnorm != 0.0f) return gscale * fdiv(1.0f, add(gnorm, eps));
    return gscale;
  }
  // in: g (raw), p, m, v, cs = grad_multiplier   out: m, v updated; um, ug.
  // MODE is the `mode` argument (0 = L2, 1 = decoupled weight decay) as a compile-time
  // constant: with the choice made once per chunk, the arithmetic of the elements a thread
  // holds is one straight line of code that the compiler can interleave.
  template <int MODE>
  __device__ __forceinline__ void apply(float g, float p, float& m, float& v, float cs, float& um,
                                        float& ug) const {
    float sg = g * cs;
    if (MODE == 0) {
      sg = fmaf(wd, p, sg);
      m = fmaf(beta3, sg, m * beta1);
      v = fmaf(one_minus_beta2 * sg, sg, v * beta2);
      const float r = rcp_approx(sqrt_approx(v * inv_bc2) + eps);
      um = (m * inv_bc1) * r;
      ug = sg * r;
    } else {
      m = fmaf(beta3, sg, m * beta1);
      v = fmaf(one_minus_beta2 * sg, sg, v * beta2);
      const float r = rcp_approx(sqrt_approx(v * inv_bc2) + eps);
      const float sp = wd * p;
      um = fmaf(m * inv_bc1, r, sp);
      ug = fmaf(sg, r, sp);
    }
  }
};

// ---- chunk walkers ------------------------------------------------------------
struct ChunkView {
  const void* g;
  float* p;
  float* m;
  float* v;
  void* out;
  int len;       // elements in this chunk
  bool aligned;  // vector path allowed
};

__device__ __forceinline__ ChunkView chunk_view(const TensorDesc& d, uint32_t chunk, int g_size,
                                                int out_size) {
  ChunkView c;
  const int64_t start = (int64_t)chunk * kChunkElems;
  const int64_t left = d.numel - start;
  c.len = left < kChunkElems ? (int)left : kChunkElems;
  c.g = static_cast<const char*>(d.g) + start * g_size;
  c.p = d.p + start;
  c.m = d.m + start;
  c.v = d.v ? d.v + start : nullptr;
  c.out = d.out ? static_cast<char*>(d.out) + start * out_size : nullptr;
  c.aligned = (d.flags & kFlagAligned) != 0;
  return c;
}

// Read-modify-write of p, m (and v when NSTATE == 2) over one chunk.
template <int NSTATE, typename GT, typename OT, typename Op>
__device__ __forceinline__ void update_chunk(const ChunkView& c, const Op& op,
                                             const Policies& pol) {
  const GT* g = static_cast<const GT*>(c.g);
  OT* out = static_cast<OT*>(c.out);
  const int tid = threadIdx.x;
  int done = 0;
  if (c.aligned) {
    const int len4 = c.len & ~(kVec - 1);
    for (int base = 0; base < len4; base += kUnroll * kPassElems) {
      F4 rg[kUnroll], rp[kUnroll], rm[kUnroll], rv[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int e = base + u * kPassElems + tid * kVec;
        if (e < len4) {
          rg[u] = Elem<GT>::template load4<kStream>(g + e, pol);
          rp[u] = Elem<float>::template load4<kStream>(c.p + e, pol);
          rm[u] = Elem<float>::template load4<kStream>(c.m + e, pol);
          if (NSTATE == 2) rv[u] = Elem<float>::template load4<kStream>(c.v + e, pol);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int e = base + u * kPassElems + tid * kVec;
        if (e < len4) {
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            float vv = NSTATE == 2 ? rv[u].x[j] : 0.f;
            op(rg[u].x[j], rp[u].x[j], rm[u].x[j], vv);
            if (NSTATE == 2) rv[u].x[j] = vv;
          }
          Elem<float>::template store4<kDefault>(c.p + e, rp[u], pol);
          Elem<float>::template store4<kDefault>(c.m + e, rm[u], pol);
          if (NSTATE == 2) Elem<float>::template store4<kDefault>(c.v + e, rv[u], pol);
          if (out) Elem<OT>::template store4<kDefault>(out + e, rp[u], pol);
        }
      }
    }
    done = len4;
  }
  for (int e = done + tid; e < c.len; e += kBlockThreads) {
    float gg = Elem<GT>::to_f32(g[e]);
    float pp = c.p[e], mm = c.m[e], vv = NSTATE == 2 ? c.v[e] : 0.f;
    op(gg, pp, mm, vv);
    c.p[e] = pp;
    c.m[e] = mm;
    if (NSTATE == 2) c.v[e] = vv;
    if (out) out[e] = Elem<OT>::from_f32(pp);
  }
}

}  // namespace rafb200
