/*
 * CPU oracle for the ZeRO optimizer step of awslabs/raf.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is a plain-C restatement of the
 * arithmetic the reference performs on this path and exists only so that the
 * CUDA kernels of this repository can be checked against it and so that a
 * CPU baseline can be timed beside them.  Nothing that ships (the raf_b200
 * package, its shared library) links, imports or calls it.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the awslabs/raf tree).  Floating point is evaluated exactly as written:
 * compile with -ffp-contract=off so that no multiply-add is fused unless the
 * source asks for it with fmaf().
 *
 * Pinning status
 *   sgd          pinned: formula of tests/python/op/tvm/test_tvm_loss.py:158-175
 *                and torch.optim.SGD as used by tests/python/optim/test_sgd.py:99.
 *   lans, norms  pinned on a GPU against the reference's own
 *                multi_tensor_lans_cuda<float> compiled unchanged (oracle/_ref),
 *                and on CPU against fixtures that kernel produced
 *                (tests/golden/lans_ref_*.npz).
 *   collectives  pinned: exact values of
 *                tests/python/distributed/test_collective_communication.py.
 *   adam         PARITY UNPINNED - the reference has no Adam operator; the
 *                semantics are defined by this repository and only
 *                cross-checked against torch.optim.AdamW.
 *   bf16, SGD weight decay, fused grad unscale: unpinned extensions (the
 *                reference has none of them on this path).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* dtype codes shared with the C-ABI of the product library */
enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_BF16 = 2 };

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the thread count of every later call (a launcher may have exported
 * OMP_NUM_THREADS=1 before this library was loaded); returns the count in use. */
ORACLE_API int oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* 16-bit float conversions.  raf.op.cast lowers to topi.cast               */
/* (python/raf/_tvm_op/transform.py:444-450, declared at                    */
/* src/op/declare/transform.cc:868-913): IEEE round-to-nearest-even.        */
/* ------------------------------------------------------------------------ */
static inline float bits_to_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

ORACLE_API float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_f32(sign);
    /* subnormal: value = man * 2^-24 */
    float v = (float)man * 5.9604644775390625e-08f;
    return sign ? -v : v;
  }
  if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
  return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

ORACLE_API uint16_t oracle_f32_to_f16(float f) {
  uint32_t x = f32_to_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0u));
  }
  if (ax >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (ax < 0x38800000u) { /* below the smallest normal half: subnormal result */
    if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to zero (ties-to-even) */
    uint32_t e = ax >> 23;                          /* biased fp32 exponent, 102..112 */
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;      /* 24-bit significand */
    uint32_t shift = 126u - e;                      /* 14..24 */
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1u);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
  }
  uint32_t e = (ax >> 23) - 112u;
  uint32_t m = ax & 0x7fffffu;
  uint32_t q = (e << 10) | (m >> 13);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++; /* carry may roll into exponent: correct */
  return (uint16_t)(sign | q);
}

ORACLE_API float oracle_bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

ORACLE_API uint16_t oracle_f32_to_bf16(float f) {
  uint32_t x = f32_to_bits(f);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u); /* quiet nan */
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7fffu + lsb;
  return (uint16_t)(x >> 16);
}

static inline float load_as_f32(const void* p, int dtype, int64_t i) {
  switch (dtype) {
    case ORACLE_F16: return oracle_f16_to_f32(((const uint16_t*)p)[i]);
    case ORACLE_BF16: return oracle_bf16_to_f32(((const uint16_t*)p)[i]);
    default: return ((const float*)p)[i];
  }
}

static inline void store_from_f32(void* p, int dtype, int64_t i, float v) {
  switch (dtype) {
    case ORACLE_F16: ((uint16_t*)p)[i] = oracle_f32_to_f16(v); break;
    case ORACLE_BF16: ((uint16_t*)p)[i] = oracle_f32_to_bf16(v); break;
    default: ((float*)p)[i] = v; break;
  }
}

/* raf.op.cast / raf.op.group_cast element loop (src/op/dialect/tvm/transform.cc:620-673). */
ORACLE_API void oracle_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) store_from_f32(dst, dst_dtype, i, load_as_f32(src, src_dtype, i));
}

/* ------------------------------------------------------------------------ */
/* raf.op.sgd                                                                */
/*   python/raf/_tvm_op/sgd.py:13-33 :  v1 = mu*v0 + dx ;  x1 = x0 - lr*v1    */
/*   (lr and mu are constants of x0's dtype).  The traced chain of           */
/*   python/raf/optim/sgd.py:198-201 computes the same two statements with   */
/*   multiply/add/subtract ops.  Updated in place here (the reference        */
/*   returns new tensors that the caller writes back, sgd.py:56-58).         */
/* Extensions without a reference counterpart (both default to "off"):       */
/*   grad_scale multiplies the gradient first (loss-scale / 1/n),            */
/*   weight_decay adds wd*x0 to it (torch.optim.SGD convention),             */
/*   out/out_dtype receives cast(x1) (the cast before _allgather,            */
/*   python/raf/optim/sgd.py:203-204).                                       */
/* ------------------------------------------------------------------------ */
ORACLE_API void oracle_sgd(float* x, const void* dx, int dx_dtype, float* v, int64_t n, float lr,
                           float mu, float weight_decay, float grad_scale, void* out,
                           int out_dtype) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float g = load_as_f32(dx, dx_dtype, i);
    if (grad_scale != 1.0f) g = g * grad_scale;
    if (weight_decay != 0.0f) g = g + weight_decay * x[i];
    float v1 = mu * v[i] + g;
    float x1 = x[i] - lr * v1;
    v[i] = v1;
    x[i] = x1;
    if (out) store_from_f32(out, out_dtype, i, x1);
  }
}

/* ------------------------------------------------------------------------ */
/* Per-tensor L2 norm, restating the reduction ORDER of the reference kernel */
/*   src/op/dialect/cuda/kernels/multi_tensor_lans.cu:95-167 (L2NormFunctor) */
/*   :42-87 (reduce_block_into_lanes), :169-185 (cleanup),                   */
/*   launch geometry :14-15 (512 threads, ILP 4), lans.cc:22 (chunk 65536).  */
/* One chunk = one thread block of 512 threads with 4 accumulators each.     */
/*   aligned path  (n%4==0, pointer 16-byte aligned): thread t, lane ii      */
/*        accumulates elements 4*(t+512*r)+ii, r = 0,1,...                   */
/*   generic path: thread t, lane ii accumulates r*2048 + t + 512*ii.        */
/* then per thread val = ((l0+l1)+l2)+l3, a shared-memory tree 512->64, a    */
/* final x[t]+x[t+32] and five shuffle-down steps.  `fused` selects          */
/* fmaf(x,x,acc) for the accumulation (what nvcc emits by default for        */
/* `vals[ii] += next*next`) instead of a separately rounded product.         */
/* ------------------------------------------------------------------------ */
#define REF_BLOCK 512
#define REF_ILP 4
#define REF_CHUNK 65536

static float ref_block_tree(float* x /* REF_BLOCK values, clobbered */) {
  for (int i = REF_BLOCK >> 1; i >= 64; i >>= 1)
    for (int t = 0; t < i; ++t) x[t] = x[t] + x[t + i];
  float w[32];
  for (int t = 0; t < 32; ++t) w[t] = x[t] + x[t + 32];
  for (int i = 16; i >= 1; i >>= 1)
    for (int t = 0; t < i; ++t) w[t] = w[t] + w[t + i]; /* lane 0 only ever reads in-range lanes */
  return w[0];
}

static float ref_chunk_sumsq(const void* base, int dtype, int64_t start, int64_t n_left,
                             int aligned, float scale, int fused) {
  float lanes[REF_BLOCK * REF_ILP];
  memset(lanes, 0, sizeof(lanes));
  int64_t len = n_left < REF_CHUNK ? n_left : REF_CHUNK;
  const int64_t row = REF_BLOCK * REF_ILP;
  for (int64_t r0 = 0; r0 < len; r0 += row) {
    int64_t lim = len - r0 < row ? len - r0 : row;
    for (int64_t j = 0; j < lim; ++j) {
      float xv = load_as_f32(base, dtype, start + r0 + j);
      if (scale != 1.0f) xv = xv * scale;
      /* j = position inside this row of 2048 consecutive elements */
      int lane = aligned ? (int)j /* 4*t+ii */ : (int)((j % REF_BLOCK) * REF_ILP + j / REF_BLOCK);
      lanes[lane] = fused ? fmaf(xv, xv, lanes[lane]) : lanes[lane] + xv * xv;
    }
  }
  float vals[REF_BLOCK];
  for (int t = 0; t < REF_BLOCK; ++t) {
    float v = 0.f;
    for (int ii = 0; ii < REF_ILP; ++ii) v += lanes[t * REF_ILP + ii];
    vals[t] = v;
  }
  return ref_block_tree(vals);
}

/* sum of squares of one tensor in the reference order; returns sqrt() like cleanup(). */
ORACLE_API float oracle_l2norm_ref_order(const void* x, int dtype, int64_t n, float scale,
                                         int max_chunks_per_tensor, int fused) {
  int64_t nchunks = (n + REF_CHUNK - 1) / REF_CHUNK;
  if (max_chunks_per_tensor < nchunks) max_chunks_per_tensor = (int)nchunks;
  if (max_chunks_per_tensor < 1) max_chunks_per_tensor = 1;
  float* partial = (float*)calloc((size_t)max_chunks_per_tensor, sizeof(float));
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t c = 0; c < nchunks; ++c) {
    int64_t start = c * REF_CHUNK;
    int64_t left = n - start;
    /* multi_tensor_lans.cu:125: n % ILP == 0 && chunk_size % ILP == 0 && is_aligned(x).
     * The kernel only ever sees fp32 tensors whose base comes from a device
     * allocator (256-byte aligned), so every chunk start is 16-byte aligned and
     * the choice of path depends on the remaining length alone. */
    int aligned = (left % REF_ILP == 0);
    partial[c] = ref_chunk_sumsq(x, dtype, start, left, aligned, scale, fused);
  }
  /* cleanup(): thread t sums partial[t], partial[t+512], ... then the same tree */
  float vals[REF_BLOCK];
  for (int t = 0; t < REF_BLOCK; ++t) {
    float v = 0.f;
    for (int i = t; i < max_chunks_per_tensor; i += REF_BLOCK) v += partial[i];
    vals[t] = v;
  }
  free(partial);
  return sqrtf(ref_block_tree(vals));
}

/* Same quantity accumulated in double: the "exact" value both the reference
 * order and this repository's kernel order are compared with. */
ORACLE_API double oracle_l2norm_f64(const void* x, int dtype, int64_t n, float scale) {
  double acc = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : acc)
  for (int64_t i = 0; i < n; ++i) {
    float xv = load_as_f32(x, dtype, i);
    if (scale != 1.0f) xv = xv * scale;
    acc += (double)xv * (double)xv;
  }
  return sqrt(acc);
}

/* ------------------------------------------------------------------------ */
/* raf.op.lans                                                               */
/*   host side   src/op/dialect/cuda/lans.cc:92-131                          */
/*       step = (int)step_tensor; bias corrections 1 - pow(beta, step)       */
/*       (float base, int exponent -> evaluated in double, :103-104) when    */
/*       bias_correction == 1 else 1; beta3 = 1-beta1 when grad_averaging.   */
/*   sequence    multi_tensor_lans.cu:401-450                                */
/*       ||g||, ||p|| -> stage 1 -> ||update_m||, ||update_g|| -> stage 2    */
/*   stage 1     multi_tensor_lans.cu:207-322                                */
/*   stage 2     multi_tensor_lans.cu:326-399                                */
/* One tensor per call (the op treats every tensor of tensor_list            */
/* independently, with non-overlapping scratch).  `g` may be 16-bit: the     */
/* reference casts gradients to fp32 first (python/raf/optim/lans.py:261-265)*/
/* which is what load_as_f32 does.  grad_scale (no reference counterpart)    */
/* multiplies the gradient before anything else.                             */
/* norm_mode: 0 reference reduction order, separately rounded squares        */
/*            1 reference reduction order, fused multiply-add accumulation   */
/*            2 double accumulation                                          */
/* norms_out[4] (optional) receives ||g||, ||p||, ||update_m||, ||update_g||.*/
/* In place on p, m, v.  g is left untouched (the reference overwrites it    */
/* with update_m, which nobody reads afterwards).  out receives cast(p).     */
/* ------------------------------------------------------------------------ */
static float norm_of(const void* x, int dtype, int64_t n, float scale, int max_chunks,
                     int norm_mode) {
  if (norm_mode == 2) return (float)oracle_l2norm_f64(x, dtype, n, scale);
  return oracle_l2norm_ref_order(x, dtype, n, scale, max_chunks, norm_mode == 1);
}

ORACLE_API void oracle_lans_bias_corrections(float beta1, float beta2, int step,
                                             int bias_correction, float* bc1, float* bc2) {
  *bc1 = 1.0f;
  *bc2 = 1.0f;
  if (bias_correction == 1) { /* lans.cc:102-105 */
    *bc1 = (float)(1 - pow((double)beta1, (double)step));
    *bc2 = (float)(1 - pow((double)beta2, (double)step));
  }
}

ORACLE_API void oracle_lans_tensor(const void* g, int g_dtype, float* p, float* m, float* v,
                                   int64_t n, int step, float lr, float beta1, float beta2,
                                   float eps, int bias_correction, float weight_decay,
                                   int grad_averaging, int mode, int normalize_grad,
                                   float grad_scale, int max_chunks_per_tensor, int norm_mode,
                                   void* out, int out_dtype, float* norms_out) {
  float bc1, bc2;
  oracle_lans_bias_corrections(beta1, beta2, step, bias_correction, &bc1, &bc2);
  float beta3 = 1.0f;
  if (grad_averaging == 1) beta3 = 1 - beta1; /* lans.cc:106-109 */

  float grad_norm = norm_of(g, g_dtype, n, grad_scale, max_chunks_per_tensor, norm_mode);
  float param_norm = norm_of(p, ORACLE_F32, n, 1.0f, max_chunks_per_tensor, norm_mode);

  float* um = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
  float* ug = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
  const float decay = weight_decay;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) { /* multi_tensor_lans.cu:281-306 */
    float r_g = load_as_f32(g, g_dtype, i);
    if (grad_scale != 1.0f) r_g = r_g * grad_scale;
    float r_p = (decay == 0) ? 0.0f : p[i]; /* :263-268 */
    float r_m = m[i];
    float r_v = v[i];
    float scaled_grad = r_g;
    if (normalize_grad && grad_norm != 0.0f) scaled_grad /= (grad_norm + eps);
    float upd_m, upd_g;
    if (mode == 0) {
      scaled_grad = scaled_grad + decay * r_p;
      r_m = r_m * beta1 + beta3 * scaled_grad;
      r_v = r_v * beta2 + (1 - beta2) * scaled_grad * scaled_grad;
      float next_m_unbiased = r_m / bc1;
      float next_v_unbiased = r_v / bc2;
      float denom = sqrtf(next_v_unbiased) + eps;
      upd_m = next_m_unbiased / denom;
      upd_g = scaled_grad / denom;
    } else {
      r_m = r_m * beta1 + beta3 * scaled_grad;
      r_v = r_v * beta2 + (1 - beta2) * scaled_grad * scaled_grad;
      float next_m_unbiased = r_m / bc1;
      float next_v_unbiased = r_v / bc2;
      float denom = sqrtf(next_v_unbiased) + eps;
      float scaled_p = decay * r_p;
      upd_m = (next_m_unbiased / denom) + scaled_p;
      upd_g = (scaled_grad / denom) + scaled_p;
    }
    um[i] = upd_m;
    ug[i] = upd_g;
    m[i] = r_m;
    v[i] = r_v;
  }
  float update_m_norm = norm_of(um, ORACLE_F32, n, 1.0f, max_chunks_per_tensor, norm_mode);
  float update_g_norm = norm_of(ug, ORACLE_F32, n, 1.0f, max_chunks_per_tensor, norm_mode);

  /* multi_tensor_lans.cu:350-353 */
  float ratio_m = (update_m_norm != 0.0f && param_norm != 0.0f) ? lr * (param_norm / update_m_norm)
                                                                : lr;
  float ratio_g = (update_g_norm != 0.0f && param_norm != 0.0f) ? lr * (param_norm / update_g_norm)
                                                                : lr;
  ratio_m *= beta1;
  ratio_g *= beta3;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) { /* :385 */
    float r_p = p[i] - (ratio_m * um[i]) - (ratio_g * ug[i]);
    p[i] = r_p;
    if (out) store_from_f32(out, out_dtype, i, r_p);
  }
  free(um);
  free(ug);
  if (norms_out) {
    norms_out[0] = grad_norm;
    norms_out[1] = param_norm;
    norms_out[2] = update_m_norm;
    norms_out[3] = update_g_norm;
  }
}

/* The whole raf.op.lans call: tensor_list = [g..., p..., m..., v...]
 * (python/raf/optim/lans.py:267).  max_chunks_per_tensor is the maximum over
 * the list as lans.cc:68-73 computes it (it changes the stride of the
 * cleanup sum, not its value, but is restated for fidelity). */
ORACLE_API void oracle_lans(int k, const void* const* g, int g_dtype, float* const* p,
                            float* const* m, float* const* v, const int64_t* numel, int step,
                            float lr, float beta1, float beta2, float eps, int bias_correction,
                            float weight_decay, int grad_averaging, int mode, int normalize_grad,
                            float grad_scale, int norm_mode, void* const* out, int out_dtype,
                            float* norms_out /* 4*k or NULL */) {
  int max_chunks = 1;
  for (int t = 0; t < k; ++t) {
    int c = (int)((numel[t] + REF_CHUNK - 1) / REF_CHUNK);
    if (c > max_chunks) max_chunks = c;
  }
  for (int t = 0; t < k; ++t) {
    oracle_lans_tensor(g[t], g_dtype, p[t], m[t], v[t], numel[t], step, lr, beta1, beta2, eps,
                       bias_correction, weight_decay, grad_averaging, mode, normalize_grad,
                       grad_scale, max_chunks, norm_mode, out ? out[t] : NULL, out_dtype,
                       norms_out ? norms_out + 4 * t : NULL);
  }
}

/* ------------------------------------------------------------------------ */
/* Adam.  PARITY UNPINNED: awslabs/raf has no Adam operator.  Defined here   */
/* as LANS stage 1 without gradient normalisation and without trust ratios   */
/* (same moment, bias-correction and denominator expressions as              */
/* multi_tensor_lans.cu:281-306):                                            */
/*   mode 1 (decoupled): m=b1*m+(1-b1)*g; v=b2*v+(1-b2)*g*g;                  */
/*          p = p - lr*((m/bc1)/(sqrt(v/bc2)+eps) + wd*p)                    */
/*   mode 0 (L2):        g = g + wd*p first, no decoupled term.              */
/* ------------------------------------------------------------------------ */
ORACLE_API void oracle_adam(const void* g, int g_dtype, float* p, float* m, float* v, int64_t n,
                            int step, float lr, float beta1, float beta2, float eps,
                            int bias_correction, float weight_decay, int mode, float grad_scale,
                            void* out, int out_dtype) {
  float bc1, bc2;
  oracle_lans_bias_corrections(beta1, beta2, step, bias_correction, &bc1, &bc2);
  const float beta3 = 1 - beta1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float r_g = load_as_f32(g, g_dtype, i);
    if (grad_scale != 1.0f) r_g = r_g * grad_scale;
    float r_p = p[i];
    float r_m = m[i];
    float r_v = v[i];
    if (mode == 0) r_g = r_g + weight_decay * r_p;
    r_m = r_m * beta1 + beta3 * r_g;
    r_v = r_v * beta2 + (1 - beta2) * r_g * r_g;
    float next_m_unbiased = r_m / bc1;
    float next_v_unbiased = r_v / bc2;
    float denom = sqrtf(next_v_unbiased) + eps;
    float update = next_m_unbiased / denom;
    if (mode != 0) update = update + weight_decay * r_p;
    r_p = r_p - lr * update;
    p[i] = r_p;
    m[i] = r_m;
    v[i] = r_v;
    if (out) store_from_f32(out, out_dtype, i, r_p);
  }
}

/* ------------------------------------------------------------------------ */
/* Shard geometry and bucketing (integer work, must match exactly).          */
/* ------------------------------------------------------------------------ */

/* Rows of dim 0 each rank owns: python/raf/optim/utils.py:46-47 (ceil) and
 * src/pass/partition_gradient.cc:191-197 (d0/n + 1 when d0 % n != 0). */
ORACLE_API int64_t oracle_shard_rows(int64_t d0, int n_part) {
  if (d0 % n_part == 0) return d0 / n_part;
  return d0 / n_part + 1;
}

/* Bucket assignment by element count.
 * rule 0: src/pass/partition_gradient.cc:269-300 - a gradient joins the open
 *         bucket when curr + size < bucket_size, else the open bucket is
 *         issued and the gradient opens a new one; the last gradient always
 *         joins and flushes (:282-288).
 * rule 1: src/pass/group_allgather.cc:110-145 - same comparison, but the
 *         trailing bucket is simply flushed at the end (a lone trailing
 *         tensor is kept, unlike the reference's `size() > 1` quirk at :149).
 * sizes are UNPADDED element counts.  Writes bucket_of[i]; returns #buckets. */
ORACLE_API int oracle_plan_buckets(const int64_t* sizes, int k, int64_t bucket_size, int rule,
                                   int* bucket_of) {
  int b = 0;
  int64_t curr = 0;
  int open = 0; /* tensors in the open bucket */
  for (int i = 0; i < k; ++i) {
    if (rule == 0 && i == k - 1) { /* last_all_reduce_: join, then flush */
      bucket_of[i] = b;
      open++;
      break;
    }
    if (curr + sizes[i] < bucket_size) {
      bucket_of[i] = b;
      curr += sizes[i];
      open++;
    } else {
      if (open > 0) b++; /* issue the open bucket (the reference would issue an empty group) */
      bucket_of[i] = b;
      curr = sizes[i];
      open = 1;
    }
  }
  return k > 0 ? b + 1 : 0;
}
