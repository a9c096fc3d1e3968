// ZeRO plan (shard geometry, buckets) and the step driver:
// grouped reduce-scatter -> shard-local update -> grouped all-gather per bucket,
// collectives on the communication stream, updates on the compute stream.
#include <algorithm>
#include <cstring>
#include <memory>

#include "common.h"

struct rafb200_plan_s {
  int k = 0, n = 1, rank = 0;
  int64_t bucket_elems = 0;
  std::vector<int64_t> dim0, row_elems, shard_rows, shard_elems, padded_elems, numel;
  std::vector<int> bucket_of;
  int nbuckets = 0;
  int64_t total = 0, total_padded = 0, total_shard = 0;
};

namespace rafb200 {

struct Bucket {
  std::vector<int> tensors;
  rafb200_tensor_list_t list = nullptr;
  void* lans_ws = nullptr;
  size_t lans_ws_bytes = 0;
  cudaEvent_t rs_done = nullptr, upd_done = nullptr;
  // arguments of the grouped collectives, rebuilt on bind
  std::vector<const void*> rs_send;
  std::vector<void*> rs_recv;
  std::vector<int64_t> counts;
  std::vector<const void*> ag_send;
  std::vector<void*> ag_recv;
};

}  // namespace rafb200

struct rafb200_zero_s {
  rafb200_plan_s plan;
  rafb200_comm_t comm = nullptr;
  int n = 1, rank = 0;
  int g_dtype = 0, param_dtype = 0, optimizer = 0;
  std::vector<rafb200::Bucket> buckets;
  // staging for tensors whose dim 0 does not divide by n (raf.op.pad / strided_slice)
  std::vector<void*> stage_g, stage_p;
  std::vector<void*> grads, params;
  std::vector<float*> p, m, v;
  bool bound = false;
  cudaEvent_t ev_start = nullptr, ev_done = nullptr;
  int max_update_blocks = 0;
  int kernels_per_step = 0, collectives_per_step = 0;
};

using namespace rafb200;

extern "C" {

int rafb200_plan_create(int k, const int64_t* dim0, const int64_t* row_elems, int n_ranks,
                        int rank, int64_t bucket_elems, rafb200_plan_t* plan) {
  RAFB200_REQUIRE(plan, "rafb200_plan_create: NULL result pointer");
  *plan = nullptr;
  RAFB200_REQUIRE(k >= 0 && (k == 0 || (dim0 && row_elems)), "rafb200_plan_create: bad tensor table");
  RAFB200_REQUIRE(n_ranks >= 1 && rank >= 0 && rank < n_ranks,
                  "rafb200_plan_create: rank %d outside %d partitions", rank, n_ranks);
  auto pl = std::make_unique<rafb200_plan_s>();
  pl->k = k;
  pl->n = n_ranks;
  pl->rank = rank;
  pl->bucket_elems = bucket_elems;
  pl->dim0.assign(dim0, dim0 + k);
  pl->row_elems.assign(row_elems, row_elems + k);
  pl->shard_rows.resize(k);
  pl->shard_elems.resize(k);
  pl->padded_elems.resize(k);
  pl->numel.resize(k);
  pl->bucket_of.resize(k);
  int b = 0, open = 0;
  int64_t curr = 0;
  for (int i = 0; i < k; ++i) {
    RAFB200_REQUIRE(dim0[i] >= 0 && row_elems[i] >= 0, "rafb200_plan_create: negative shape, tensor %d", i);
    // partition_gradient.cc:191-197: d0/n + 1 rows per part when d0 % n != 0
    const int64_t rows = (dim0[i] % n_ranks == 0) ? dim0[i] / n_ranks : dim0[i] / n_ranks + 1;
    pl->shard_rows[i] = rows;
    pl->shard_elems[i] = rows * row_elems[i];
    pl->padded_elems[i] = rows * n_ranks * row_elems[i];
    pl->numel[i] = dim0[i] * row_elems[i];
    pl->total += pl->numel[i];
    pl->total_padded += pl->padded_elems[i];
    pl->total_shard += pl->shard_elems[i];
    // partition_gradient.cc:289-300 / group_allgather.cc:110-145: join while curr + size < bucket
    if (curr + pl->numel[i] < bucket_elems) {
      curr += pl->numel[i];
      open++;
    } else {
      if (open > 0) b++;
      curr = pl->numel[i];
      open = 1;
    }
    pl->bucket_of[i] = b;
  }
  pl->nbuckets = k > 0 ? b + 1 : 0;
  *plan = pl.release();
  return RAFB200_OK;
}

int rafb200_plan_destroy(rafb200_plan_t plan) {
  delete plan;
  return RAFB200_OK;
}

int rafb200_plan_num_buckets(rafb200_plan_t plan) { return plan ? plan->nbuckets : 0; }

int rafb200_plan_query(rafb200_plan_t plan, int64_t* shard_rows, int64_t* shard_elems,
                       int64_t* padded_elems, int* bucket_of) {
  RAFB200_REQUIRE(plan, "rafb200_plan_query: NULL plan");
  for (int i = 0; i < plan->k; ++i) {
    if (shard_rows) shard_rows[i] = plan->shard_rows[i];
    if (shard_elems) shard_elems[i] = plan->shard_elems[i];
    if (padded_elems) padded_elems[i] = plan->padded_elems[i];
    if (bucket_of) bucket_of[i] = plan->bucket_of[i];
  }
  return RAFB200_OK;
}

int rafb200_plan_totals(rafb200_plan_t plan, int64_t* elems, int64_t* padded_elems,
                        int64_t* shard_elems) {
  RAFB200_REQUIRE(plan, "rafb200_plan_totals: NULL plan");
  if (elems) *elems = plan->total;
  if (padded_elems) *padded_elems = plan->total_padded;
  if (shard_elems) *shard_elems = plan->total_shard;
  return RAFB200_OK;
}

// ---- step driver ----------------------------------------------------------------

int rafb200_zero_destroy(rafb200_zero_t z) {
  if (!z) return RAFB200_OK;
  for (auto& b : z->buckets) {
    if (b.list) rafb200_tensor_list_destroy(b.list);
    if (b.lans_ws) cudaFree(b.lans_ws);
    if (b.rs_done) cudaEventDestroy(b.rs_done);
    if (b.upd_done) cudaEventDestroy(b.upd_done);
  }
  for (void* ptr : z->stage_g)
    if (ptr) cudaFree(ptr);
  for (void* ptr : z->stage_p)
    if (ptr) cudaFree(ptr);
  if (z->ev_start) cudaEventDestroy(z->ev_start);
  if (z->ev_done) cudaEventDestroy(z->ev_done);
  delete z;
  return RAFB200_OK;
}

int rafb200_zero_create(rafb200_plan_t plan, rafb200_comm_t comm, int g_dtype, int param_dtype,
                        int optimizer, rafb200_zero_t* zero) {
  RAFB200_REQUIRE(zero, "rafb200_zero_create: NULL result pointer");
  *zero = nullptr;
  RAFB200_REQUIRE(plan && comm, "rafb200_zero_create: NULL plan or communicator");
  RAFB200_REQUIRE(dtype_valid(g_dtype) && dtype_valid(param_dtype), "rafb200_zero_create: bad dtype");
  RAFB200_REQUIRE(optimizer >= RAFB200_OPT_SGD && optimizer <= RAFB200_OPT_LANS,
                  "rafb200_zero_create: unknown optimizer %d", optimizer);
  RAFB200_REQUIRE(plan->n == rafb200_comm_size(comm) && plan->rank == rafb200_comm_rank(comm),
                  "rafb200_zero_create: plan is for rank %d of %d, communicator is rank %d of %d",
                  plan->rank, plan->n, rafb200_comm_rank(comm), rafb200_comm_size(comm));
  auto* z = new rafb200_zero_s();
  z->plan = *plan;
  z->comm = comm;
  z->n = plan->n;
  z->rank = plan->rank;
  z->g_dtype = g_dtype;
  z->param_dtype = param_dtype;
  z->optimizer = optimizer;
  const int k = plan->k;
  z->stage_g.assign(k, nullptr);
  z->stage_p.assign(k, nullptr);
  int rc = RAFB200_OK;
  do {
    // With a single rank there is nothing to overlap: one bucket, one launch.
    const int nb = (z->n == 1) ? (k > 0 ? 1 : 0) : plan->nbuckets;
    z->buckets.resize(nb);
    for (int i = 0; i < k; ++i) z->buckets[z->n == 1 ? 0 : plan->bucket_of[i]].tensors.push_back(i);
    for (auto& b : z->buckets) {
      std::vector<int64_t> numel;
      for (int i : b.tensors) numel.push_back(plan->shard_elems[i]);
      rc = rafb200_tensor_list_create((int)numel.size(), numel.data(), g_dtype, param_dtype, &b.list);
      if (rc != RAFB200_OK) break;
      if (optimizer == RAFB200_OPT_LANS) {
        b.lans_ws_bytes = rafb200_lans_workspace_bytes(b.list);
        if (cudaMalloc(&b.lans_ws, b.lans_ws_bytes) != cudaSuccess) {
          rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot allocate LANS workspace");
          break;
        }
      }
      if (cudaEventCreateWithFlags(&b.rs_done, cudaEventDisableTiming) != cudaSuccess ||
          cudaEventCreateWithFlags(&b.upd_done, cudaEventDisableTiming) != cudaSuccess) {
        rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot create events");
        break;
      }
    }
    if (rc != RAFB200_OK) break;
    if (cudaEventCreateWithFlags(&z->ev_start, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&z->ev_done, cudaEventDisableTiming) != cudaSuccess) {
      rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot create events");
      break;
    }
    for (int i = 0; i < k && z->n > 1; ++i) {
      if (plan->padded_elems[i] == plan->numel[i]) continue;
      if (cudaMalloc(&z->stage_g[i], (size_t)plan->padded_elems[i] * dtype_size(g_dtype)) != cudaSuccess ||
          cudaMalloc(&z->stage_p[i], (size_t)plan->padded_elems[i] * dtype_size(param_dtype)) != cudaSuccess) {
        rc = set_error(RAFB200_CUDA_ERROR, "rafb200_zero_create: cannot allocate padding buffers");
        break;
      }
      // The zero tail is written once: reduce-scatter only ever adds zeros to it.
      cudaMemset(z->stage_g[i], 0, (size_t)plan->padded_elems[i] * dtype_size(g_dtype));
    }
  } while (false);
  if (rc != RAFB200_OK) {
    rafb200_zero_destroy(z);
    return rc;
  }
  *zero = z;
  return RAFB200_OK;
}

int rafb200_zero_bind(rafb200_zero_t z, void* const* grads, void* const* params, float* const* p,
                      float* const* m, float* const* v) {
  RAFB200_REQUIRE(z, "rafb200_zero_bind: NULL state");
  const int k = z->plan.k;
  RAFB200_REQUIRE(k == 0 || (grads && params && p && m), "rafb200_zero_bind: NULL pointer table");
  RAFB200_REQUIRE(z->optimizer == RAFB200_OPT_SGD || v, "rafb200_zero_bind: v is required");
  z->grads.assign(grads, grads + k);
  z->params.assign(params, params + k);
  z->p.assign(p, p + k);
  z->m.assign(m, m + k);
  if (v) z->v.assign(v, v + k);
  else z->v.clear();
  const int gs = dtype_size(z->g_dtype), ps = dtype_size(z->param_dtype);
  z->kernels_per_step = 0;
  z->collectives_per_step = 0;
  for (auto& b : z->buckets) {
    const size_t nt = b.tensors.size();
    std::vector<const void*> lg(nt);
    std::vector<float*> lp(nt), lm(nt), lv(nt);
    std::vector<void*> lo(nt);
    b.rs_send.resize(nt);
    b.rs_recv.resize(nt);
    b.ag_send.resize(nt);
    b.ag_recv.resize(nt);
    b.counts.resize(nt);
    for (size_t j = 0; j < nt; ++j) {
      const int i = b.tensors[j];
      const int64_t se = z->plan.shard_elems[i];
      // Tensors that need padding live in staging buffers for the collectives.
      char* gbase = static_cast<char*>(z->stage_g[i] ? z->stage_g[i] : grads[i]);
      char* pbase = static_cast<char*>(z->stage_p[i] ? z->stage_p[i] : params[i]);
      RAFB200_REQUIRE(se == 0 || (gbase && pbase && p[i] && m[i]),
                      "rafb200_zero_bind: NULL buffer for tensor %d", i);
      char* gshard = gbase + (size_t)z->rank * se * gs;  // in-place reduce-scatter target
      char* pshard = pbase + (size_t)z->rank * se * ps;  // in-place all-gather source
      b.rs_send[j] = gbase;
      b.rs_recv[j] = gshard;
      b.ag_send[j] = pshard;
      b.ag_recv[j] = pbase;
      b.counts[j] = se;
      lg[j] = gshard;
      lp[j] = p[i];
      lm[j] = m[i];
      lv[j] = v ? v[i] : nullptr;
      lo[j] = pshard;
    }
    int rc = rafb200_tensor_list_bind(b.list, lg.data(), lp.data(), lm.data(), v ? lv.data() : nullptr,
                                      lo.data(), nullptr);
    if (rc != RAFB200_OK) return rc;
    if (rafb200_tensor_list_total_elems(b.list) > 0) z->kernels_per_step += 1;
    if (z->n > 1) z->collectives_per_step += 2 * (int)nt;
  }
  RAFB200_CUDA(cudaStreamSynchronize(nullptr));  // descriptor tables are in place
  z->bound = true;
  return RAFB200_OK;
}

int rafb200_zero_set_update_blocks(rafb200_zero_t z, int max_blocks) {
  RAFB200_REQUIRE(z && max_blocks >= 0, "rafb200_zero_set_update_blocks: bad arguments");
  z->max_update_blocks = max_blocks;
  for (auto& b : z->buckets) {
    int rc = rafb200_tensor_list_tune(b.list, b.list->window_elems, b.list->slack_items, max_blocks);
    if (rc != RAFB200_OK) return rc;
  }
  return RAFB200_OK;
}

int rafb200_zero_launch_counts(rafb200_zero_t z, int* kernels, int* collectives) {
  RAFB200_REQUIRE(z, "rafb200_zero_launch_counts: NULL state");
  if (kernels) *kernels = z->kernels_per_step;
  if (collectives) *collectives = z->collectives_per_step;
  return RAFB200_OK;
}

static int run_update(rafb200_zero_s* z, Bucket& b, const rafb200_hyper* h, int step, float gscale,
                      cudaStream_t s) {
  switch (z->optimizer) {
    case RAFB200_OPT_SGD:
      return rafb200_sgd_list(b.list, h->learning_rate, h->mu, h->weight_decay, gscale, s);
    case RAFB200_OPT_ADAM:
      return rafb200_adam(b.list, step, nullptr, h->learning_rate, h->beta1, h->beta2, h->eps,
                          h->bias_correction, h->weight_decay, h->mode, gscale, s);
    default:
      return rafb200_lans(b.list, step, nullptr, h->learning_rate, h->beta1, h->beta2, h->eps,
                          h->bias_correction, h->weight_decay, h->grad_averaging, h->mode,
                          h->normalize_grad, gscale, b.lans_ws, b.lans_ws_bytes, s);
  }
}

int rafb200_zero_step(rafb200_zero_t z, const rafb200_hyper* h, int step, void* compute_stream,
                      void* comm_stream) {
  RAFB200_REQUIRE(z && h, "rafb200_zero_step: NULL argument");
  RAFB200_REQUIRE(z->bound, "rafb200_zero_step: bind buffers first");
  RAFB200_REQUIRE(h->optimizer == z->optimizer, "rafb200_zero_step: optimizer differs from the one created");
  cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
  cudaStream_t ms = static_cast<cudaStream_t>(comm_stream);
  // A mean over ranks is a sum on the wire and a 1/n folded into the update's
  // gradient scale (the `divide` of partition_gradient.cc:274-279, fused).
  const float gscale = h->grad_scale * ((h->average && z->n > 1) ? 1.0f / (float)z->n : 1.0f);
  const int nb = (int)z->buckets.size();
  if (z->n == 1) {
    for (auto& b : z->buckets) {
      int rc = run_update(z, b, h, step, gscale, cs);
      if (rc != RAFB200_OK) return rc;
    }
    return RAFB200_OK;
  }
  const int gs = dtype_size(z->g_dtype), ps = dtype_size(z->param_dtype);
  // Gradients were produced on the compute stream.
  RAFB200_CUDA(cudaEventRecord(z->ev_start, cs));
  RAFB200_CUDA(cudaStreamWaitEvent(ms, z->ev_start, 0));
  auto reduce_scatter = [&](Bucket& b) -> int {
    for (int i : b.tensors)  // raf.op.pad: copy the unpadded rows in front of the zero tail
      if (z->stage_g[i])
        RAFB200_CUDA(cudaMemcpyAsync(z->stage_g[i], z->grads[i], (size_t)z->plan.numel[i] * gs,
                                     cudaMemcpyDeviceToDevice, ms));
    int rc = rafb200_group_reduce_scatter(z->comm, (int)b.tensors.size(), b.rs_send.data(),
                                          b.rs_recv.data(), b.counts.data(), z->g_dtype, "sum", ms);
    if (rc != RAFB200_OK) return rc;
    RAFB200_CUDA(cudaEventRecord(b.rs_done, ms));
    return RAFB200_OK;
  };
  int rc = nb > 0 ? reduce_scatter(z->buckets[0]) : RAFB200_OK;
  if (rc != RAFB200_OK) return rc;
  for (int bi = 0; bi < nb; ++bi) {
    Bucket& b = z->buckets[bi];
    if (bi + 1 < nb) {
      rc = reduce_scatter(z->buckets[bi + 1]);
      if (rc != RAFB200_OK) return rc;
    }
    RAFB200_CUDA(cudaStreamWaitEvent(cs, b.rs_done, 0));
    rc = run_update(z, b, h, step, gscale, cs);
    if (rc != RAFB200_OK) return rc;
    RAFB200_CUDA(cudaEventRecord(b.upd_done, cs));
    RAFB200_CUDA(cudaStreamWaitEvent(ms, b.upd_done, 0));
    rc = rafb200_group_allgather(z->comm, (int)b.tensors.size(), b.ag_send.data(), b.ag_recv.data(),
                                 b.counts.data(), z->param_dtype, ms);
    if (rc != RAFB200_OK) return rc;
    for (int i : b.tensors)  // strided_slice [0:dim0] + add(out=param): drop the padding rows
      if (z->stage_p[i])
        RAFB200_CUDA(cudaMemcpyAsync(z->params[i], z->stage_p[i], (size_t)z->plan.numel[i] * ps,
                                     cudaMemcpyDeviceToDevice, ms));
  }
  RAFB200_CUDA(cudaEventRecord(z->ev_done, ms));
  RAFB200_CUDA(cudaStreamWaitEvent(cs, z->ev_done, 0));
  return RAFB200_OK;
}

int rafb200_zero_step_host(rafb200_zero_t z, const rafb200_hyper* h, int step,
                           const void* const* grads_host, void* const* params_host,
                           void* compute_stream, void* comm_stream) {
  RAFB200_REQUIRE(z && h && grads_host && params_host, "rafb200_zero_step_host: NULL argument");
  RAFB200_REQUIRE(z->bound, "rafb200_zero_step_host: bind device buffers first");
  cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
  const int gs = dtype_size(z->g_dtype), ps = dtype_size(z->param_dtype);
  for (int i = 0; i < z->plan.k; ++i)
    if (z->plan.numel[i])
      RAFB200_CUDA(cudaMemcpyAsync(z->grads[i], grads_host[i], (size_t)z->plan.numel[i] * gs,
                                   cudaMemcpyHostToDevice, cs));
  int rc = rafb200_zero_step(z, h, step, compute_stream, comm_stream);
  if (rc != RAFB200_OK) return rc;
  for (int i = 0; i < z->plan.k; ++i)
    if (z->plan.numel[i])
      RAFB200_CUDA(cudaMemcpyAsync(params_host[i], z->params[i], (size_t)z->plan.numel[i] * ps,
                                   cudaMemcpyDeviceToHost, cs));
  return RAFB200_OK;
}

}  // extern "C"
