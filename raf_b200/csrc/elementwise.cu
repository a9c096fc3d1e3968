// SGD-momentum and Adam update kernels (single pass, HBM-bound: every byte is
// touched once), raf.op.cast / group_cast and fuse_tensor / defuse_tensor.
#include <cmath>
#include <type_traits>

#include "common.h"
#include "symm_dev.cuh"
#include "update_core.cuh"

namespace rafb200 {

// ---- update kernels -----------------------------------------------------------
// Work items are handed out statically: block b takes items b, b+grid, ...
template <int NSTATE, typename GT, typename OT, typename Op>
__global__ void __launch_bounds__(kBlockThreads)
    update_list_kernel(const TensorDesc* __restrict__ descs, const Item* __restrict__ items,
                       uint32_t nitems, Op op) {
  Policies pol;
  pol.init();
  for (uint32_t it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item item = items[it];
    const TensorDesc d = descs[item.tensor_phase & kTensorMask];
    ChunkView c = chunk_view(d, item.chunk, sizeof(GT), sizeof(OT));
    update_chunk<NSTATE, GT, OT>(c, op, pol);
  }
}

// The same update with the collectives inside (n > 1, symmetric memory; no counterpart in the
// reference): the gradient is the sum over ranks of the chunk, read through the multicast
// address or peer by peer at TensorDesc's symmetric offset (kept in first_chunk / nchunks) and
// also written to the rank's local gradient block; the model-dtype copy goes into every rank's
// parameter buffer.  The symmetric layout is 16-byte aligned and zero-padded per row block.
// passes in flight per thread (four were measured slower: 128 registers, half the resident blocks)
constexpr int kFusedUnroll = 2;
template <int NSTATE, typename GT, typename OT, typename Op>
__global__ void __launch_bounds__(kBlockThreads)
    update_list_fused_kernel(const TensorDesc* __restrict__ descs, const Item* __restrict__ items,
                             uint32_t nitems, Op op, LansFuse fu) {
  constexpr int kDT = sizeof(GT) == 4 ? RAFB200_F32 : (std::is_same<GT, __half>::value ? RAFB200_F16 : RAFB200_BF16);
  Policies pol;
  pol.init();
  const int tid = threadIdx.x;
  for (uint32_t it = blockIdx.x; it < nitems; it += gridDim.x) {
    const Item item = items[it];
    const TensorDesc d = descs[item.tensor_phase & kTensorMask];
    const ChunkView c = chunk_view(d, item.chunk, sizeof(GT), sizeof(OT));
    const size_t sym = ((((size_t)d.nchunks) << 32) | d.first_chunk) + (size_t)item.chunk * kChunkElems * sizeof(GT);
    GT* gred = const_cast<GT*>(static_cast<const GT*>(c.g));
    OT* out = static_cast<OT*>(c.out);
    const int len4 = c.len & ~(kVec - 1);
    for (int base = 0; base < len4; base += kFusedUnroll * kPassElems) {
      F4 rg[kFusedUnroll], rp[kFusedUnroll], rm[kFusedUnroll], rv[kFusedUnroll];
      uint32_t bits[kFusedUnroll][4];
#pragma unroll
      for (int u = 0; u < kFusedUnroll; ++u) {
        const int e = base + u * kPassElems + tid * kVec;
        if (sizeof(GT) == 2) {
          // 16-bit gradients: a pair of lanes shares one 16-byte access (eight elements); the even
          // lane makes it - the row block's zero padding covers a missing partner - and hands the
          // upper half over.  Every lane of the warp takes part in the exchange.
          uint4 raw = make_uint4(0, 0, 0, 0);
          if ((tid & 1) == 0 && e < len4) {
            const size_t off = sym + (size_t)e * sizeof(GT);
            if (fu.g_mc) {
              raw = mc_ld_reduce<kDT>(fu.g_mc + off);
            } else {
              float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
              for (int q = 0; q < fu.world; ++q) accumulate<kDT>(acc, peer_ld(fu.g_peer[q] + off));
              raw = round_once<kDT>(acc);
            }
          }
          const uint32_t hi0 = __shfl_sync(0xffffffffu, raw.z, (tid & 31) & ~1);
          const uint32_t hi1 = __shfl_sync(0xffffffffu, raw.w, (tid & 31) & ~1);
          bits[u][0] = (tid & 1) ? hi0 : raw.x;
          bits[u][1] = (tid & 1) ? hi1 : raw.y;
          bits[u][2] = bits[u][3] = 0;
          float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          accumulate<kDT>(f, make_uint4(bits[u][0], bits[u][1], 0u, 0u));
#pragma unroll
          for (int j = 0; j < 4; ++j) rg[u].x[j] = f[j];
        }
        if (e < len4) {
          if (sizeof(GT) == 4)
            reduced4<kDT>(fu.g_mc, fu.g_peer, fu.world, sym + (size_t)e * sizeof(GT), rg[u].x, bits[u]);
          rp[u] = Elem<float>::template load4<kStream>(c.p + e, pol);
          rm[u] = Elem<float>::template load4<kStream>(c.m + e, pol);
          if (NSTATE == 2) rv[u] = Elem<float>::template load4<kStream>(c.v + e, pol);
        }
      }
#pragma unroll
      for (int u = 0; u < kFusedUnroll; ++u) {
        const int e = base + u * kPassElems + tid * kVec;
        if (e < len4) {
          if (sizeof(GT) == 4) *reinterpret_cast<uint4*>(gred + e) = make_uint4(bits[u][0], bits[u][1], bits[u][2], bits[u][3]);
          else *reinterpret_cast<uint2*>(gred + e) = make_uint2(bits[u][0], bits[u][1]);
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            float vv = NSTATE == 2 ? rv[u].x[j] : 0.f;
            op(rg[u].x[j], rp[u].x[j], rm[u].x[j], vv);
            if (NSTATE == 2) rv[u].x[j] = vv;
          }
          Elem<float>::template store4<kDefault>(c.p + e, rp[u], pol);
          Elem<float>::template store4<kDefault>(c.m + e, rm[u], pol);
          if (NSTATE == 2) Elem<float>::template store4<kDefault>(c.v + e, rv[u], pol);
          if (out) {
            if (fu.fuse_ag) store4_everywhere<OT>(fu.p_mc, fu.p_peer, fu.world, fu.rank, out + e, rp[u]);
            else Elem<OT>::template store4<kDefault>(out + e, rp[u], pol);
          }
        }
      }
    }
    // the last one to three elements of a tensor: element by element, peer by peer
    for (int e = len4 + tid; e < c.len; e += kBlockThreads) {
      float acc = 0.f;
      for (int q = 0; q < fu.world; ++q)
        acc += Elem<GT>::to_f32(*reinterpret_cast<const volatile GT*>(fu.g_peer[q] + sym + (size_t)e * sizeof(GT)));
      const GT rounded = Elem<GT>::from_f32(acc);
      gred[e] = rounded;
      float gg = Elem<GT>::to_f32(rounded);
      float pp = c.p[e], mm = c.m[e], vv = NSTATE == 2 ? c.v[e] : 0.f;
      op(gg, pp, mm, vv);
      c.p[e] = pp;
      c.m[e] = mm;
      if (NSTATE == 2) c.v[e] = vv;
      if (out) {
        if (fu.fuse_ag) store1_everywhere<OT>(fu.p_peer, fu.world, fu.rank, out + e, pp);
        else out[e] = Elem<OT>::from_f32(pp);
      }
    }
  }
}

// One tensor described by value: chunk i is work item i.
template <int NSTATE, typename GT, typename OT, typename Op>
__global__ void __launch_bounds__(kBlockThreads)
    update_flat_kernel(TensorDesc d, Op op) {
  Policies pol;
  pol.init();
  for (uint32_t ch = blockIdx.x; ch < d.nchunks; ch += gridDim.x) {
    ChunkView c = chunk_view(d, ch, sizeof(GT), sizeof(OT));
    update_chunk<NSTATE, GT, OT>(c, op, pol);
  }
}

static int grid_for(uint32_t nitems, int device) {
  static int sm_count[64] = {0};
  if (device < 0 || device >= 64) device = 0;
  if (sm_count[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = 148;
    sm_count[device] = n;
  }
  // 8 resident blocks of 256 threads per SM; a multiple of the SM count.
  uint32_t cap = (uint32_t)sm_count[device] * 8u;
  return (int)(nitems < cap ? (nitems ? nitems : 1) : cap);
}

template <int NSTATE, typename Op, typename GT>
static int launch_list_out(const rafb200_tensor_list_s* l, const Op& op, cudaStream_t s) {
  const int grid = grid_for(l->n_items, l->device);
  if (l->fuse.fuse_rs) {
    switch (l->out_dtype) {
      case RAFB200_F32:
        update_list_fused_kernel<NSTATE, GT, float><<<grid, kBlockThreads, 0, s>>>(l->dev_desc, l->dev_items, l->n_items, op, l->fuse);
        break;
      case RAFB200_F16:
        update_list_fused_kernel<NSTATE, GT, __half><<<grid, kBlockThreads, 0, s>>>(l->dev_desc, l->dev_items, l->n_items, op, l->fuse);
        break;
      default:
        update_list_fused_kernel<NSTATE, GT, __nv_bfloat16><<<grid, kBlockThreads, 0, s>>>(l->dev_desc, l->dev_items, l->n_items, op, l->fuse);
        break;
    }
    RAFB200_CUDA(cudaGetLastError());
    return RAFB200_OK;
  }
  switch (l->out_dtype) {
    case RAFB200_F32:
      update_list_kernel<NSTATE, GT, float><<<grid, kBlockThreads, 0, s>>>(l->dev_desc, l->dev_items, l->n_items, op);
      break;
    case RAFB200_F16:
      update_list_kernel<NSTATE, GT, __half><<<grid, kBlockThreads, 0, s>>>(l->dev_desc, l->dev_items, l->n_items, op);
      break;
    default:
      update_list_kernel<NSTATE, GT, __nv_bfloat16><<<grid, kBlockThreads, 0, s>>>(l->dev_desc, l->dev_items, l->n_items, op);
      break;
  }
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

template <int NSTATE, typename Op>
static int launch_list(const rafb200_tensor_list_s* l, const Op& op, cudaStream_t s) {
  if (l->n_items == 0) return RAFB200_OK;
  switch (l->g_dtype) {
    case RAFB200_F32: return launch_list_out<NSTATE, Op, float>(l, op, s);
    case RAFB200_F16: return launch_list_out<NSTATE, Op, __half>(l, op, s);
    default: return launch_list_out<NSTATE, Op, __nv_bfloat16>(l, op, s);
  }
}

template <typename GT>
static int launch_flat_sgd_out(const TensorDesc& d, int out_dtype, const SgdOp& op, int device,
                               cudaStream_t s) {
  const int grid = grid_for(d.nchunks, device);
  switch (out_dtype) {
    case RAFB200_F32: update_flat_kernel<1, GT, float><<<grid, kBlockThreads, 0, s>>>(d, op); break;
    case RAFB200_F16: update_flat_kernel<1, GT, __half><<<grid, kBlockThreads, 0, s>>>(d, op); break;
    default: update_flat_kernel<1, GT, __nv_bfloat16><<<grid, kBlockThreads, 0, s>>>(d, op); break;
  }
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

bool pointers_aligned(const void* g, int g_dtype, const void* p, const void* m, const void* v,
                      const void* out, int out_dtype) {
  auto ok = [](const void* ptr, int bytes) { return (reinterpret_cast<uintptr_t>(ptr) % bytes) == 0; };
  bool a = ok(g, g_dtype == RAFB200_F32 ? 16 : 8) && ok(p, 16) && ok(m, 16);
  if (v) a = a && ok(v, 16);
  if (out) a = a && ok(out, out_dtype == RAFB200_F32 ? 16 : 8);
  return a;
}

// Bias corrections exactly as the reference's host code computes them
// (src/op/dialect/cuda/lans.cc:100-105: float base, int exponent -> double pow).
void bias_corrections(float beta1, float beta2, int step, int bias_correction, float* bc1,
                      float* bc2) {
  *bc1 = 1.0f;
  *bc2 = 1.0f;
  if (bias_correction == 1) {
    *bc1 = static_cast<float>(1 - std::pow(static_cast<double>(beta1), static_cast<double>(step)));
    *bc2 = static_cast<float>(1 - std::pow(static_cast<double>(beta2), static_cast<double>(step)));
  }
}

// ---- cast ----------------------------------------------------------------------
template <typename ST, typename DT>
__global__ void __launch_bounds__(kBlockThreads)
    cast_kernel(const ST* __restrict__ src, DT* __restrict__ dst, int64_t n, bool aligned) {
  Policies pol;
  pol.init();
  const int64_t n4 = aligned ? (n & ~(int64_t)3) : 0;
  for (int64_t e = ((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) * 4; e < n4;
       e += (int64_t)gridDim.x * kBlockThreads * 4) {
    F4 v = Elem<ST>::template load4<kStream>(src + e, pol);
    Elem<DT>::template store4<kDefault>(dst + e, v, pol);
  }
  for (int64_t e = n4 + (int64_t)blockIdx.x * kBlockThreads + threadIdx.x; e < n;
       e += (int64_t)gridDim.x * kBlockThreads)
    dst[e] = Elem<DT>::from_f32(Elem<ST>::to_f32(src[e]));
}

template <typename ST>
static int launch_cast_dst(const void* src, void* dst, int dst_dtype, int64_t n, bool aligned,
                           int grid, cudaStream_t s) {
  switch (dst_dtype) {
    case RAFB200_F32:
      cast_kernel<ST, float><<<grid, kBlockThreads, 0, s>>>((const ST*)src, (float*)dst, n, aligned);
      break;
    case RAFB200_F16:
      cast_kernel<ST, __half><<<grid, kBlockThreads, 0, s>>>((const ST*)src, (__half*)dst, n, aligned);
      break;
    default:
      cast_kernel<ST, __nv_bfloat16><<<grid, kBlockThreads, 0, s>>>((const ST*)src, (__nv_bfloat16*)dst, n, aligned);
      break;
  }
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

static int cast_impl(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n,
                     cudaStream_t s) {
  if (n == 0) return RAFB200_OK;
  int device = 0;
  cudaGetDevice(&device);
  auto ok = [](const void* ptr, int dt) {
    return (reinterpret_cast<uintptr_t>(ptr) % (dt == RAFB200_F32 ? 16 : 8)) == 0;
  };
  const bool aligned = ok(src, src_dtype) && ok(dst, dst_dtype);
  const int64_t per_block = (int64_t)kBlockThreads * 4;
  const int64_t blocks = (n + per_block - 1) / per_block;
  const int grid = grid_for((uint32_t)(blocks > (1 << 30) ? (1 << 30) : blocks), device);
  switch (src_dtype) {
    case RAFB200_F32: return launch_cast_dst<float>(src, dst, dst_dtype, n, aligned, grid, s);
    case RAFB200_F16: return launch_cast_dst<__half>(src, dst, dst_dtype, n, aligned, grid, s);
    default: return launch_cast_dst<__nv_bfloat16>(src, dst, dst_dtype, n, aligned, grid, s);
  }
}

// ---- batched byte movers (group_cast, fuse_tensor, defuse_tensor) -----------
constexpr int kBatch = 96;  // tensors per launch: 96 * 24 B of pointers/sizes fit the 4 KB parameter space
struct CopyBatch {
  const void* src[kBatch];
  void* dst[kBatch];
  int64_t numel[kBatch];
};

template <typename ST, typename DT>
__global__ void __launch_bounds__(kBlockThreads) group_cast_kernel(CopyBatch b) {
  const int t = blockIdx.y;
  const ST* src = static_cast<const ST*>(b.src[t]);
  DT* dst = static_cast<DT*>(b.dst[t]);
  const int64_t n = b.numel[t];
  const bool aligned = (reinterpret_cast<uintptr_t>(src) % (sizeof(ST) * 4) == 0) &&
                       (reinterpret_cast<uintptr_t>(dst) % (sizeof(DT) * 4) == 0);
  Policies pol;
  pol.init();
  const int64_t n4 = aligned ? (n & ~(int64_t)3) : 0;
  for (int64_t e = ((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) * 4; e < n4;
       e += (int64_t)gridDim.x * kBlockThreads * 4) {
    F4 v = Elem<ST>::template load4<kStream>(src + e, pol);
    Elem<DT>::template store4<kDefault>(dst + e, v, pol);
  }
  for (int64_t e = n4 + (int64_t)blockIdx.x * kBlockThreads + threadIdx.x; e < n;
       e += (int64_t)gridDim.x * kBlockThreads)
    dst[e] = Elem<DT>::from_f32(Elem<ST>::to_f32(src[e]));
}

// Plain byte copy of each (src, dst, nbytes) triple; 16-byte accesses when both ends allow.
__global__ void __launch_bounds__(kBlockThreads) group_copy_kernel(CopyBatch b) {
  const int t = blockIdx.y;
  const char* src = static_cast<const char*>(b.src[t]);
  char* dst = static_cast<char*>(b.dst[t]);
  const int64_t n = b.numel[t];  // bytes
  const bool aligned = (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(dst) % 16 == 0);
  Policies pol;
  pol.init();
  const int64_t n16 = aligned ? (n & ~(int64_t)15) : 0;
  for (int64_t e = ((int64_t)blockIdx.x * kBlockThreads + threadIdx.x) * 16; e < n16;
       e += (int64_t)gridDim.x * kBlockThreads * 16)
    st16<kDefault>(dst + e, ld16<kStream>(src + e, pol), pol);
  for (int64_t e = n16 + (int64_t)blockIdx.x * kBlockThreads + threadIdx.x; e < n;
       e += (int64_t)gridDim.x * kBlockThreads)
    dst[e] = src[e];
}

template <typename Launch>
static int for_each_batch(int k, const void* const* src, void* const* dst, const int64_t* numel,
                          int64_t scale, int work_per_thread, Launch launch) {
  for (int t0 = 0; t0 < k; t0 += kBatch) {
    CopyBatch b;
    const int nb = (k - t0 < kBatch) ? k - t0 : kBatch;
    int64_t maxn = 0;
    for (int i = 0; i < nb; ++i) {
      b.src[i] = src[t0 + i];
      b.dst[i] = dst[t0 + i];
      b.numel[i] = numel[t0 + i] * scale;
      if (b.numel[i] > maxn) maxn = b.numel[i];
    }
    if (maxn == 0) continue;
    const int64_t per_block = (int64_t)kBlockThreads * work_per_thread;
    int64_t gx = (maxn + per_block - 1) / per_block;
    if (gx > 148 * 4) gx = 148 * 4;
    int rc = launch(b, dim3((unsigned)gx, (unsigned)nb));
    if (rc != RAFB200_OK) return rc;
  }
  return RAFB200_OK;
}

template <typename ST>
static int group_cast_dst(const CopyBatch& b, dim3 grid, int dst_dtype, cudaStream_t s) {
  switch (dst_dtype) {
    case RAFB200_F32: group_cast_kernel<ST, float><<<grid, kBlockThreads, 0, s>>>(b); break;
    case RAFB200_F16: group_cast_kernel<ST, __half><<<grid, kBlockThreads, 0, s>>>(b); break;
    default: group_cast_kernel<ST, __nv_bfloat16><<<grid, kBlockThreads, 0, s>>>(b); break;
  }
  RAFB200_CUDA(cudaGetLastError());
  return RAFB200_OK;
}

}  // namespace rafb200

using namespace rafb200;

extern "C" {

int rafb200_sgd(float* x, const void* dx, int dx_dtype, float* v, int64_t numel,
                float learning_rate, float mu, float weight_decay, float grad_scale, void* out,
                int out_dtype, void* stream) {
  RAFB200_REQUIRE(numel >= 0, "rafb200_sgd: negative numel");
  RAFB200_REQUIRE(dtype_valid(dx_dtype) && dtype_valid(out_dtype), "rafb200_sgd: bad dtype");
  if (numel == 0) return RAFB200_OK;
  RAFB200_REQUIRE(x && dx && v, "rafb200_sgd: x, dx and v must not be NULL");
  RAFB200_REQUIRE((numel + kChunkElems - 1) / kChunkElems < (int64_t)1 << 31,
                  "rafb200_sgd: tensor too large");
  TensorDesc d{};
  d.g = dx;
  d.p = x;
  d.m = v;
  d.v = nullptr;
  d.out = out;
  d.numel = numel;
  d.first_chunk = 0;
  d.nchunks = (uint32_t)((numel + kChunkElems - 1) / kChunkElems);
  d.flags = pointers_aligned(dx, dx_dtype, x, v, nullptr, out, out_dtype) ? kFlagAligned : 0;
  SgdOp op{learning_rate, mu, weight_decay, grad_scale};
  int device = 0;
  cudaGetDevice(&device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dx_dtype) {
    case RAFB200_F32: return launch_flat_sgd_out<float>(d, out_dtype, op, device, s);
    case RAFB200_F16: return launch_flat_sgd_out<__half>(d, out_dtype, op, device, s);
    default: return launch_flat_sgd_out<__nv_bfloat16>(d, out_dtype, op, device, s);
  }
}

int rafb200_sgd_list(rafb200_tensor_list_t list, float learning_rate, float mu,
                     float weight_decay, float grad_scale, void* stream) {
  RAFB200_REQUIRE(list, "rafb200_sgd_list: NULL list");
  RAFB200_REQUIRE(list->bound, "rafb200_sgd_list: bind the tensor list first");
  SgdOp op{learning_rate, mu, weight_decay, grad_scale};
  return launch_list<1>(list, op, static_cast<cudaStream_t>(stream));
}

int rafb200_adam(rafb200_tensor_list_t list, int step, const float* step_dev,
                 float learning_rate, float beta1, float beta2, float eps, int bias_correction,
                 float weight_decay, int mode, float grad_scale, void* stream) {
  RAFB200_REQUIRE(list, "rafb200_adam: NULL list");
  RAFB200_REQUIRE(list->bound && list->has_v, "rafb200_adam: bind g, p, m and v first");
  RAFB200_REQUIRE(step_dev == nullptr,
                  "rafb200_adam: a device-resident step is only supported by rafb200_lans");
  RAFB200_REQUIRE(step >= 1, "rafb200_adam: step counts from 1");
  AdamOp op;
  op.lr = learning_rate;
  op.beta1 = beta1;
  op.beta2 = beta2;
  op.beta3 = 1 - beta1;
  op.one_minus_beta2 = 1 - beta2;
  op.eps = eps;
  bias_corrections(beta1, beta2, step, bias_correction, &op.bc1, &op.bc2);
  op.wd = weight_decay;
  op.gscale = grad_scale;
  op.mode = mode;
  return launch_list<2>(list, op, static_cast<cudaStream_t>(stream));
}

int rafb200_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t numel,
                 void* stream) {
  RAFB200_REQUIRE(dtype_valid(src_dtype) && dtype_valid(dst_dtype), "rafb200_cast: bad dtype");
  RAFB200_REQUIRE(numel >= 0 && (numel == 0 || (src && dst)), "rafb200_cast: bad arguments");
  return cast_impl(src, src_dtype, dst, dst_dtype, numel, static_cast<cudaStream_t>(stream));
}

int rafb200_group_cast(int k, const void* const* src, int src_dtype, void* const* dst,
                       int dst_dtype, const int64_t* numel, void* stream) {
  RAFB200_REQUIRE(k >= 0 && (k == 0 || (src && dst && numel)), "rafb200_group_cast: bad arguments");
  RAFB200_REQUIRE(dtype_valid(src_dtype) && dtype_valid(dst_dtype), "rafb200_group_cast: bad dtype");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return for_each_batch(k, src, dst, numel, 1, 4, [&](const CopyBatch& b, dim3 grid) {
    switch (src_dtype) {
      case RAFB200_F32: return group_cast_dst<float>(b, grid, dst_dtype, s);
      case RAFB200_F16: return group_cast_dst<__half>(b, grid, dst_dtype, s);
      default: return group_cast_dst<__nv_bfloat16>(b, grid, dst_dtype, s);
    }
  });
}

static int group_copy(int k, const void* const* src, void* const* dst, const int64_t* numel,
                      int elem_size, cudaStream_t s) {
  return for_each_batch(k, src, dst, numel, elem_size, 16, [&](const CopyBatch& b, dim3 grid) {
    group_copy_kernel<<<grid, kBlockThreads, 0, s>>>(b);
    RAFB200_CUDA(cudaGetLastError());
    return (int)RAFB200_OK;
  });
}

int rafb200_fuse_tensor(int k, const void* const* src, const int64_t* numel, const int64_t* offsets,
                        int elem_size, void* flat, void* stream) {
  RAFB200_REQUIRE(k >= 0 && elem_size > 0 && (k == 0 || (src && numel && offsets && flat)),
                  "rafb200_fuse_tensor: bad arguments");
  std::vector<void*> dst(k);
  for (int i = 0; i < k; ++i) dst[i] = static_cast<char*>(flat) + offsets[i] * elem_size;
  return group_copy(k, src, dst.data(), numel, elem_size, static_cast<cudaStream_t>(stream));
}

int rafb200_defuse_tensor(int k, void* const* dst, const int64_t* numel, const int64_t* offsets,
                          int elem_size, const void* flat, void* stream) {
  RAFB200_REQUIRE(k >= 0 && elem_size > 0 && (k == 0 || (dst && numel && offsets && flat)),
                  "rafb200_defuse_tensor: bad arguments");
  std::vector<const void*> src(k);
  for (int i = 0; i < k; ++i) src[i] = static_cast<const char*>(flat) + offsets[i] * elem_size;
  return group_copy(k, src.data(), dst, numel, elem_size, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
