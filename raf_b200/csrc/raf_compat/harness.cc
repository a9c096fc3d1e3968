// C entry points that drive the b200 dialect (raf_dialect/b200_ops.cc) the way RAF's
// executors would: build the schema struct of a call from raw device pointers, dispatch by
// priority level, fulfil the OpEnv's requests, Execute.  Used by the tests through ctypes;
// not part of the product ABI (include/raf_b200.h).
#include <cstdio>
#include <cstring>

#include "../../schema/communication.h"
#include "../../schema/memory.h"
#include "../../schema/optimizer.h"
#include "../../schema/transform.h"
#include "raf/dialect.h"
#include "raf_compat.h"

using namespace raf;
using namespace raf::value;

namespace {
thread_local char g_err[1024] = "";
DLDataType DType(int code) {  // rafb200_dtype: 0 f32, 1 f16, 2 bf16
  if (code == 1) return DLDataType{kDLFloat, 16, 1};
  if (code == 2) return DLDataType{kDLBfloat, 16, 1};
  return DLDataType{kDLFloat, 32, 1};
}
Value Tensor(const void* data, int64_t n, int dtype) {
  return TensorValue::Assemble(const_cast<void*>(data), {n}, DType(dtype));
}
template <typename F>
int Guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    snprintf(g_err, sizeof(g_err), "%s", e.what());
    return 1;
  }
}
}  // namespace

#define RAFCOMPAT_API extern "C" __attribute__((visibility("default")))

RAFCOMPAT_API const char* rafcompat_last_error() { return g_err; }

// One line per registered dialect op: "<base op> <dialect> <dialect op> <level>\n".
RAFCOMPAT_API int rafcompat_list_ops(char* buf, size_t n) {
  std::string out;
  for (const auto& kv : op::OpDialect::Registry())
    for (const auto& e : kv.second.entries) {
      const bool has_maker = op::OpEnvMaker::Registry().count(e.dialect_op) != 0;
      out += kv.first + " " + e.dialect + " " + e.dialect_op + " " + std::to_string(e.plevel) +
             (has_maker ? " maker" : " no-maker") + "\n";
    }
  for (const auto& kv : op::Dialect::Registry())
    out += "dialect " + kv.first + (kv.second.is_enabled(DevType::kCUDA()) ? " cuda" : " -") + "\n";
  if (buf && n) snprintf(buf, n, "%s", out.c_str());
  return (int)out.size();
}

// raf.op.sgd(x, dx, v, learning_rate, mu) -> (v1, x1); v1 / x1 may alias v / x (the
// InplaceUpdate pass lets the VM allocate outputs in the inputs' buffers).
RAFCOMPAT_API int rafcompat_run_sgd(const float* x, const void* dx, int dx_dtype, const float* v, float* v1,
                                    float* x1, int64_t n, double lr, double mu, void* stream) {
  return Guard([&] {
    auto args = std::make_shared<op::schema::SgdArgs>();
    args->x = Tensor(x, n, 0);
    args->dx = Tensor(dx, n, dx_dtype);
    args->v = Tensor(v, n, 0);
    args->learning_rate = lr;
    args->mu = mu;
    auto call = op::CallValues::make({}, op::Attrs(args));
    std::vector<Value> outs = {Tensor(v1, n, 0), Tensor(x1, n, 0)};
    call->out = TupleValue::make(outs);
    compat::Executor ex(stream);
    ex.Run("raf.op.sgd", call);
  });
}

// raf.op.lans(tensor_list = [g.., p.., m.., v..], step (0-d fp32 on the device), ...): in place.
RAFCOMPAT_API int rafcompat_run_lans(int k, void* const* tensors, const int64_t* numel, int g_dtype,
                                     const float* step_dev, float lr, float beta1, float beta2, float eps,
                                     int bias_correction, float weight_decay, int grad_averaging, int mode,
                                     int normalize_grad, void* stream) {
  return Guard([&] {
    auto args = std::make_shared<op::schema::LansArgs>();
    for (int i = 0; i < 4 * k; ++i) args->tensor_list.push_back(Tensor(tensors[i], numel[i % k], i < k ? g_dtype : 0));
    args->step = TensorValue::Assemble(const_cast<float*>(step_dev), {}, DType(0));
    args->learning_rate = lr;
    args->beta1 = beta1;
    args->beta2 = beta2;
    args->eps = eps;
    args->bias_correction = bias_correction;
    args->weight_decay = weight_decay;
    args->grad_averaging = grad_averaging;
    args->mode = mode;
    args->normalize_grad = normalize_grad != 0;
    auto call = op::CallValues::make({}, op::Attrs(args));
    call->out = TupleValue::make(args->tensor_list);  // TRAFInplaceUpdate {0:0}
    compat::Executor ex(stream);
    ex.Run("raf.op.lans", call);
  });
}

RAFCOMPAT_API int rafcompat_run_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, void* stream) {
  return Guard([&] {
    auto args = std::make_shared<op::schema::CastArgs>();
    args->data = Tensor(src, n, src_dtype);
    auto call = op::CallValues::make({}, op::Attrs(args));
    call->out = Tensor(dst, n, dst_dtype);
    compat::Executor ex(stream);
    ex.Run("raf.op.cast", call);
  });
}

// fuse_tensor(data...) -> flat, then defuse_tensor(flat, sizes) -> outs: a round trip.
RAFCOMPAT_API int rafcompat_run_fuse_defuse(int k, void* const* src, void* const* dst, const int64_t* numel,
                                            void* flat, int dtype, void* stream) {
  return Guard([&] {
    int64_t total = 0;
    auto fa = std::make_shared<op::schema::FuseTensorArgs>();
    auto da = std::make_shared<op::schema::DefuseTensorArgs>();
    std::vector<Value> outs;
    for (int i = 0; i < k; ++i) {
      fa->data.push_back(Tensor(src[i], numel[i], dtype));
      outs.push_back(Tensor(dst[i], numel[i], dtype));
      da->sizes.push_back(numel[i]);
      total += numel[i];
    }
    compat::Executor ex(stream);
    auto fcall = op::CallValues::make({}, op::Attrs(fa));
    fcall->out = Tensor(flat, total, dtype);
    ex.Run("raf.op.fuse_tensor", fcall);
    da->data = Tensor(flat, total, dtype);
    auto dcall = op::CallValues::make({}, op::Attrs(da));
    dcall->out = TupleValue::make(outs);
    ex.Run("raf.op.defuse_tensor", dcall);
  });
}

// The collectives of the path on the communicator the caller names (nccl_comm NULL and
// size 1 = RAF's void communicator).  which: 0 _allreduce (in place on in[]), 1 _reduce_scatter,
// 2 _group_reduce_scatter, 3 _allgather, 4 _group_allgather.  numel_in / numel_out in elements.
RAFCOMPAT_API int rafcompat_run_collective(int which, int k, void* const* in, void* const* out,
                                           const int64_t* numel_in, const int64_t* numel_out, int dtype,
                                           const char* computation, void* nccl_comm, int size, int rank,
                                           void* stream) {
  return Guard([&] {
    std::vector<Value> ins, outs;
    for (int i = 0; i < k; ++i) {
      ins.push_back(Tensor(in[i], numel_in[i], dtype));
      outs.push_back(Tensor(out[i], numel_out[i], dtype));
    }
    compat::Executor ex(stream);
    ex.SetCommunicator(nccl_comm, size, rank);
    op::CallValues call;
    const char* name = "";
    if (which == 0) {
      auto a = std::make_shared<op::schema::AllreduceArgs>();
      a->x = ins;
      a->computation = computation;
      call = op::CallValues::make({}, op::Attrs(a));
      call->out = k == 1 ? ins[0] : Value(TupleValue::make(ins));
      name = "raf.op._allreduce";
    } else if (which == 1) {
      auto a = std::make_shared<op::schema::ReduceScatterArgs>();
      a->x = ins[0];
      a->computation = computation;
      call = op::CallValues::make({}, op::Attrs(a));
      call->out = outs[0];
      name = "raf.op._reduce_scatter";
    } else if (which == 2) {
      auto a = std::make_shared<op::schema::GroupReduceScatterArgs>();
      a->tensor_list = ins;
      a->computation = computation;
      call = op::CallValues::make({}, op::Attrs(a));
      call->out = TupleValue::make(outs);
      name = "raf.op._group_reduce_scatter";
    } else if (which == 3) {
      auto a = std::make_shared<op::schema::AllgatherArgs>();
      a->x = ins[0];
      a->axis = 0;
      call = op::CallValues::make({}, op::Attrs(a));
      call->out = outs[0];
      name = "raf.op._allgather";
    } else {
      auto a = std::make_shared<op::schema::GroupAllgatherArgs>();
      a->tensor_list = ins;
      a->axis = 0;
      a->out = outs;
      call = op::CallValues::make({}, op::Attrs(a));
      call->out = TupleValue::make(outs);
      name = "raf.op._group_allgather";
    }
    ex.Run(name, call);
  });
}
