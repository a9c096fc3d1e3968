// raf.op.lans as ONE persistent kernel.
//
// The reference runs four norm reductions and two element-wise stages as about
// fifty launches with a global dependency between them
// (src/op/dialect/cuda/kernels/multi_tensor_lans.cu:401-450).  Here the work of
// a call is a list of items (tensor, chunk, phase):
//   phase A  sum of squares of the (scaled) gradient chunk            -> ||g||
//   phase B  stage 1 on the chunk, results NOT stored: sums of squares of
//            p, update_m, update_g                                     -> norms
//   phase C  stage 1 again (bit-identical), then stage 2 with the trust
//            ratios; writes p, m, v and the model-dtype parameter copy.
// Blocks draw items from a ticket counter in list order.  An item depends only
// on items with smaller tickets (B of a tensor on all its A items, C on all its
// B items), and a ticket is only ever held by a running block, so the bounded
// waits below cannot deadlock whatever the number of resident blocks.  The
// host orders the list so that a tensor's C items follow its B items closely:
// the second read of g, p, m, v then comes out of L2 and HBM traffic approaches
// one read and one write per array.
//
// Norms: every chunk publishes its partial sums, the block that publishes the
// last partial of a tensor adds them up in a fixed order and releases a flag.
// Results are therefore bitwise reproducible run to run.
#include <algorithm>
#include <cmath>

#include "common.h"
#include "update_core.cuh"

namespace rafb200 {

void bias_corrections(float beta1, float beta2, int step, int bias_correction, float* bc1,
                      float* bc2);

constexpr int kPhaseA = 0, kPhaseB = 1, kPhaseC = 2;
constexpr unsigned kErrWaitA = 1, kErrWaitB = 2;

struct LansParams {
  const TensorDesc* descs;
  const Item* items;
  uint32_t nitems;
  LansHeader* hdr;
  LansCtl* ctl;
  float* part_a;  // [total_chunks]
  float* part_b;  // [3][total_chunks]
  uint32_t total_chunks;
  LansStage1 s1;
  float lr;
  const float* step_dev;
  int bias_correction;
  unsigned spin_limit;
};

// Bounded wait for *flag != 0.  Returns false when it gave up (or another
// block already reported an error).
__device__ __forceinline__ bool wait_flag(const unsigned* flag, LansHeader* hdr, unsigned code,
                                          uint32_t ticket, unsigned limit) {
  unsigned spins = 0, ns = 32;
  while (ld_acquire(flag) == 0) {
    __nanosleep(ns);
    if (ns < 1024) ns <<= 1;
    ++spins;
    if ((spins & 31u) == 0 && *reinterpret_cast<volatile unsigned*>(&hdr->error) != 0) return false;
    if (spins > limit) {
      if (atomicCAS(&hdr->error, 0u, code) == 0u) hdr->error_item = ticket;
      return false;
    }
  }
  return true;
}

template <typename GT, typename OT>
__global__ void __launch_bounds__(kBlockThreads, 4) lans_kernel(const LansParams P) {
  __shared__ float s_red[3 * (kBlockThreads / 32)];
  __shared__ uint32_t s_ticket;
  __shared__ int s_flag;
  __shared__ float s_bc[2];

  const int tid = threadIdx.x;
  Policies pol;
  pol.init();
  LansStage1 s1 = P.s1;
  if (P.step_dev != nullptr) {
    // step lives on the device as a 0-d fp32 tensor (python/raf/optim/lans.py:239):
    // same expression as the host code, evaluated in double.
    if (tid == 0) {
      float bc1 = 1.0f, bc2 = 1.0f;
      if (P.bias_correction == 1) {
        const int step = (int)(*P.step_dev);
        bc1 = (float)(1.0 - pow((double)s1.beta1, (double)step));
        bc2 = (float)(1.0 - pow((double)s1.beta2, (double)step));
      }
      s_bc[0] = bc1;
      s_bc[1] = bc2;
    }
    __syncthreads();
    s1.bc1 = s_bc[0];
    s1.bc2 = s_bc[1];
  }

  uint32_t next = 0;
  if (tid == 0) next = atomicAdd(&P.hdr->ticket, 1u);
  while (true) {
    if (tid == 0) s_ticket = next;
    __syncthreads();
    const uint32_t ticket = s_ticket;
    if (ticket >= P.nitems) break;
    // Draw the following ticket now: its latency hides behind this item.
    if (tid == 0) next = atomicAdd(&P.hdr->ticket, 1u);

    const Item item = P.items[ticket];
    const uint32_t t = item.tensor_phase & kTensorMask;
    const int phase = (int)(item.tensor_phase >> kPhaseShift);
    const TensorDesc d = P.descs[t];
    LansCtl* ctl = P.ctl + t;
    const ChunkView c = chunk_view(d, item.chunk, sizeof(GT), sizeof(OT));
    const GT* g = static_cast<const GT*>(c.g);
    const int len4 = c.aligned ? (c.len & ~(kVec - 1)) : 0;

    if (phase == kPhaseA) {
      float acc[1] = {0.f};
      for (int base = 0; base < len4; base += kUnroll * kPassElems) {
        F4 rg[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int e = base + u * kPassElems + tid * kVec;
          if (e < len4) rg[u] = Elem<GT>::template load4<kKeep>(g + e, pol);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int e = base + u * kPassElems + tid * kVec;
          if (e < len4) {
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
              float x = rg[u].x[j];
              if (s1.gscale != 1.0f) x = mul(x, s1.gscale);
              acc[0] = fmaf(x, x, acc[0]);
            }
          }
        }
      }
      for (int e = len4 + tid; e < c.len; e += kBlockThreads) {
        float x = Elem<GT>::to_f32(g[e]);
        if (s1.gscale != 1.0f) x = mul(x, s1.gscale);
        acc[0] = fmaf(x, x, acc[0]);
      }
      block_sum<1>(acc, s_red);
      if (tid == 0) {
        P.part_a[d.first_chunk + item.chunk] = acc[0];
        __threadfence();
        const unsigned old = atomicAdd(&ctl->arrived_a, 1u);
        s_flag = (old + 1u == d.nchunks);
      }
      __syncthreads();
      if (s_flag) {  // this block published the last partial of the tensor
        __threadfence();
        float tot[1] = {0.f};
        for (uint32_t i = tid; i < d.nchunks; i += kBlockThreads)
          tot[0] += __ldcg(P.part_a + d.first_chunk + i);
        block_sum<1>(tot, s_red);
        if (tid == 0) {
          ctl->norm[0] = sqrtf(tot[0]);
          __threadfence();
          st_release(&ctl->ready_a, 1u);
        }
      }
    } else {
      // B and C both need ||g|| (when gradients are normalised); C also the other three.
      if (tid == 0) {
        bool ok = true;
        if (s1.normalize) ok = wait_flag(&ctl->ready_a, P.hdr, kErrWaitA, ticket, P.spin_limit);
        if (ok && phase == kPhaseC)
          ok = wait_flag(&ctl->ready_b, P.hdr, kErrWaitB, ticket, P.spin_limit);
        s_flag = ok ? 0 : 1;
      }
      __syncthreads();
      if (s_flag) return;  // a bounded wait expired: the whole block leaves, nothing in flight
      const float gnorm = s1.normalize ? __ldcg(&ctl->norm[0]) : 0.f;

      if (phase == kPhaseB) {
        float acc[3] = {0.f, 0.f, 0.f};
        for (int base = 0; base < len4; base += kUnroll * kPassElems) {
          F4 rg[kUnroll], rp[kUnroll], rm[kUnroll], rv[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int e = base + u * kPassElems + tid * kVec;
            if (e < len4) {
              rg[u] = Elem<GT>::template load4<kKeep>(g + e, pol);
              rp[u] = Elem<float>::template load4<kKeep>(c.p + e, pol);
              rm[u] = Elem<float>::template load4<kKeep>(c.m + e, pol);
              rv[u] = Elem<float>::template load4<kKeep>(c.v + e, pol);
            }
          }
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int e = base + u * kPassElems + tid * kVec;
            if (e < len4) {
#pragma unroll
              for (int j = 0; j < kVec; ++j) {
                float um, ug, mm = rm[u].x[j], vv = rv[u].x[j];
                const float pp = rp[u].x[j];
                s1(rg[u].x[j], pp, mm, vv, gnorm, um, ug);
                acc[0] = fmaf(pp, pp, acc[0]);
                acc[1] = fmaf(um, um, acc[1]);
                acc[2] = fmaf(ug, ug, acc[2]);
              }
            }
          }
        }
        for (int e = len4 + tid; e < c.len; e += kBlockThreads) {
          float um, ug, mm = c.m[e], vv = c.v[e];
          const float pp = c.p[e];
          s1(Elem<GT>::to_f32(g[e]), pp, mm, vv, gnorm, um, ug);
          acc[0] = fmaf(pp, pp, acc[0]);
          acc[1] = fmaf(um, um, acc[1]);
          acc[2] = fmaf(ug, ug, acc[2]);
        }
        block_sum<3>(acc, s_red);
        if (tid == 0) {
          const uint32_t ci = d.first_chunk + item.chunk;
          P.part_b[ci] = acc[0];
          P.part_b[P.total_chunks + ci] = acc[1];
          P.part_b[2 * P.total_chunks + ci] = acc[2];
          __threadfence();
          const unsigned old = atomicAdd(&ctl->arrived_b, 1u);
          s_flag = (old + 1u == d.nchunks);
        }
        __syncthreads();
        if (s_flag) {
          __threadfence();
          float tot[3] = {0.f, 0.f, 0.f};
          for (uint32_t i = tid; i < d.nchunks; i += kBlockThreads) {
            const uint32_t ci = d.first_chunk + i;
            tot[0] += __ldcg(P.part_b + ci);
            tot[1] += __ldcg(P.part_b + P.total_chunks + ci);
            tot[2] += __ldcg(P.part_b + 2 * P.total_chunks + ci);
          }
          block_sum<3>(tot, s_red);
          if (tid == 0) {
            ctl->norm[1] = sqrtf(tot[0]);
            ctl->norm[2] = sqrtf(tot[1]);
            ctl->norm[3] = sqrtf(tot[2]);
            __threadfence();
            st_release(&ctl->ready_b, 1u);
          }
        }
      } else {  // phase C
        // multi_tensor_lans.cu:347-353
        const float pn = __ldcg(&ctl->norm[1]);
        const float umn = __ldcg(&ctl->norm[2]);
        const float ugn = __ldcg(&ctl->norm[3]);
        float ratio_m = (umn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, umn)) : P.lr;
        float ratio_g = (ugn != 0.0f && pn != 0.0f) ? mul(P.lr, fdiv(pn, ugn)) : P.lr;
        ratio_m = mul(ratio_m, s1.beta1);
        ratio_g = mul(ratio_g, s1.beta3);
        OT* out = static_cast<OT*>(c.out);
        for (int base = 0; base < len4; base += kUnroll * kPassElems) {
          F4 rg[kUnroll], rp[kUnroll], rm[kUnroll], rv[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int e = base + u * kPassElems + tid * kVec;
            if (e < len4) {
              rg[u] = Elem<GT>::template load4<kStream>(g + e, pol);
              rp[u] = Elem<float>::template load4<kStream>(c.p + e, pol);
              rm[u] = Elem<float>::template load4<kStream>(c.m + e, pol);
              rv[u] = Elem<float>::template load4<kStream>(c.v + e, pol);
            }
          }
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int e = base + u * kPassElems + tid * kVec;
            if (e < len4) {
#pragma unroll
              for (int j = 0; j < kVec; ++j) {
                float um, ug;
                s1(rg[u].x[j], rp[u].x[j], rm[u].x[j], rv[u].x[j], gnorm, um, ug);
                rp[u].x[j] = sub(sub(rp[u].x[j], mul(ratio_m, um)), mul(ratio_g, ug));  // :385
              }
              Elem<float>::template store4<kStream>(c.p + e, rp[u], pol);
              Elem<float>::template store4<kStream>(c.m + e, rm[u], pol);
              Elem<float>::template store4<kStream>(c.v + e, rv[u], pol);
              if (out) Elem<OT>::template store4<kStream>(out + e, rp[u], pol);
            }
          }
        }
        for (int e = len4 + tid; e < c.len; e += kBlockThreads) {
          float um, ug, mm = c.m[e], vv = c.v[e], pp = c.p[e];
          s1(Elem<GT>::to_f32(g[e]), pp, mm, vv, gnorm, um, ug);
          pp = sub(sub(pp, mul(ratio_m, um)), mul(ratio_g, ug));
          c.p[e] = pp;
          c.m[e] = mm;
          c.v[e] = vv;
          if (out) out[e] = Elem<OT>::from_f32(pp);
        }
      }
    }
    __syncthreads();  // s_ticket / s_flag are rewritten at the top of the loop
  }
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
    out.push_back(Item{((uint32_t)phase << kPhaseShift) | (uint32_t)cur.t, cur.c});
    cur.emitted++;
    if (++cur.c == nchunks[cur.t]) {
      if (done) (*done)[cur.t] = (int64_t)out.size();
      cur.c = 0;
      cur.t++;
      skip_empty(cur);
    }
  };
  if (!with_a) A.t = k;
  while (Cc.t < k) {
    const int64_t n = (int64_t)out.size();
    const bool a_ready = with_a && A.t < k;
    const bool b_ready = B.t < k && (!with_a || A.t > B.t);
    const bool c_ready = B.t > Cc.t;
    const bool b_slack_ok = b_ready && (B.c > 0 || !with_a || n - done_a[B.t] >= slack);
    const bool c_slack_ok = c_ready && (Cc.c > 0 || n - done_b[Cc.t] >= slack);
    const bool b_window_ok = (int64_t)(B.emitted - Cc.emitted) < window_chunks;
    const bool a_window_ok = (int64_t)(A.emitted - B.emitted) < window_chunks;
    if (c_slack_ok) emit(Cc, kPhaseC, nullptr);
    else if (b_slack_ok && b_window_ok) emit(B, kPhaseB, &done_b);
    else if (a_ready && a_window_ok) emit(A, kPhaseA, &done_a);
    else if (b_slack_ok) emit(B, kPhaseB, &done_b);
    else if (a_ready) emit(A, kPhaseA, &done_a);
    else if (b_ready) emit(B, kPhaseB, &done_b);
    else emit(Cc, kPhaseC, nullptr);  // c_ready must hold here
  }
  return out;
}

size_t lans_ctl_bytes(int k) { return 64 + sizeof(LansCtl) * (size_t)k; }

size_t lans_workspace_bytes(int k, uint32_t total_chunks) {
  size_t b = lans_ctl_bytes(k);
  b = (b + 255) & ~(size_t)255;
  b += sizeof(float) * 4 * (size_t)total_chunks;
  return (b + 255) & ~(size_t)255;
}

template <typename GT, typename OT>
static int launch_lans_t(const rafb200_tensor_list_s* l, const LansParams& P, cudaStream_t s) {
  static int occ[64] = {0};
  const int dev = (l->device >= 0 && l->device < 64) ? l->device : 0;
  if (occ[dev] == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, lans_kernel<GT, OT>, kBlockThreads, 0) !=
            cudaSuccess || n <= 0)
      n = 1;
    occ[dev] = n;
  }
  int64_t grid = (int64_t)l->sm_count * occ[dev];
  if (l->max_blocks > 0 && grid > l->max_blocks) grid = l->max_blocks;
  if (grid > (int64_t)P.nitems) grid = P.nitems;
  if (grid < 1) grid = 1;
  lans_kernel<GT, OT><<<(unsigned)grid, kBlockThreads, 0, s>>>(P);
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
  size_t off = (lans_ctl_bytes(list->k) + 255) & ~(size_t)255;
  P.part_a = reinterpret_cast<float*>(ws + off);
  P.part_b = P.part_a + list->total_chunks;
  P.total_chunks = list->total_chunks;
  P.s1.beta1 = beta1;
  P.s1.beta2 = beta2;
  P.s1.beta3 = (grad_averaging == 1) ? 1 - beta1 : 1.0f;  // lans.cc:106-109
  P.s1.one_minus_beta2 = 1 - beta2;
  P.s1.eps = eps;
  bias_corrections(beta1, beta2, step_dev ? 1 : step, bias_correction, &P.s1.bc1, &P.s1.bc2);
  P.s1.wd = weight_decay;
  P.s1.gscale = grad_scale;
  P.s1.mode = mode;
  P.s1.normalize = normalize_grad ? 1 : 0;
  P.lr = learning_rate;
  P.step_dev = step_dev;
  P.bias_correction = bias_correction;
  P.spin_limit = 4u << 20;  // x ~1 us per poll: a few seconds

  RAFB200_CUDA(cudaMemsetAsync(workspace, 0, lans_ctl_bytes(list->k), s));
  switch (list->g_dtype) {
    case RAFB200_F32: return launch_lans_g<float>(list, P, s);
    case RAFB200_F16: return launch_lans_g<__half>(list, P, s);
    default: return launch_lans_g<__nv_bfloat16>(list, P, s);
  }
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
      for (int j = 0; j < 4; ++j) norms_host[4 * t + j] = ctl[t].norm[j];
  }
  if (hdr->error != 0)
    return set_error(RAFB200_DEVICE_WAIT_EXPIRED,
                     "rafb200_lans: bounded wait %u expired at work item %u; results are invalid",
                     hdr->error, hdr->error_item);
  return RAFB200_OK;
}

}  // extern "C"
