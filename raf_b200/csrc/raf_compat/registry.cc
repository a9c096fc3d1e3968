// raf_compat: the pieces of RAF's runtime that live in .cc files there - schema field
// indices, dialect dispatch (src/impl/op.cc:127-215) and a minimal executor that fulfils an
// OpEnv's resource requests the way the interpreter does (src/impl/interpreter.cc:279-325):
// workspace from the device allocator, streams from a table indexed by tag, the
// communicator object from the caller.
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>

#include "raf/dialect.h"
#include "raf/nccl_communicator.h"
#include "raf/stream_pool.h"
#include "raf_compat.h"

namespace raf {
namespace op {

const std::vector<std::string>& SchemaFieldNames(const std::string& base_op) {
  // argument order of scripts/src_codegen/def_schema.py for the operators of the ZeRO path
  static const std::map<std::string, std::vector<std::string>> names = {
      {"raf.op.sgd", {"x", "dx", "v", "learning_rate", "mu"}},
      {"raf.op.lans",
       {"tensor_list", "step", "learning_rate", "beta1", "beta2", "eps", "bias_correction", "weight_decay",
        "grad_averaging", "mode", "normalize_grad"}},
      {"raf.op.cast", {"data", "dtype"}},
      {"raf.op.group_cast", {"tensor_list", "dtype"}},
      {"raf.op._allreduce", {"x", "computation", "rank_list"}},
      {"raf.op._allgather", {"x", "axis", "rank_list"}},
      {"raf.op._group_allgather", {"tensor_list", "axis", "out"}},
      {"raf.op._reduce_scatter", {"x", "computation", "rank_list"}},
      {"raf.op._group_reduce_scatter", {"tensor_list", "computation"}},
      {"raf.op.fuse_tensor", {"data"}},
      {"raf.op.defuse_tensor", {"data", "sizes", "shapes", "shape_indices"}},
  };
  static const std::vector<std::string> none;
  auto it = names.find(base_op);
  return it == names.end() ? none : it->second;
}

OpEnv* Dispatch(const std::string& base_op, const CallValues& call) {
  auto it = OpDialect::Registry().find(base_op);
  if (it == OpDialect::Registry().end()) return nullptr;
  for (const OpDialect::Entry& e : it->second.entries) {  // descending priority level
    auto d = Dialect::Registry().find(e.dialect);
    if (d == Dialect::Registry().end() || !d->second.is_enabled(call->device.device_type)) continue;
    auto mk = OpEnvMaker::Registry().find(e.dialect_op);
    if (mk == OpEnvMaker::Registry().end() || !mk->second.func) continue;
    std::unique_ptr<OpEnv> env(mk->second.func(call));
    if (env && !env->HasError()) return env.release();  // an OpEnv with errors: try the next dialect
  }
  return nullptr;
}

}  // namespace op

namespace ir {
op::FRAFSchemaFieldIndex Op::FieldIndexMap::operator[](const Op& op) const {
  const std::string base = op.name;
  return [base](const std::string& field) {
    const auto& names = op::SchemaFieldNames(base);
    for (size_t i = 0; i < names.size(); ++i)
      if (names[i] == field) return (int)i;
    CHECK(false) << "no field " << field << " in the schema of " << base;
    return -1;
  };
}
}  // namespace ir

namespace compat {

// Streams by tag, created on first use (src/impl/stream_pool.cc:53-98); tag 1 with index 0 is
// the stream the caller passed as "compute".
struct Executor::Impl {
  std::map<int, cudaStream_t> streams;
  std::vector<void*> workspaces;
  distributed::communicator::NCCLCommunicatorObj comm;
};

Executor::Executor(void* compute_stream) : impl_(new Impl()) {
  impl_->streams[stream_pool::StreamTagEnum::CudaCompute()] = static_cast<cudaStream_t>(compute_stream);
}
Executor::~Executor() {
  for (auto& kv : impl_->streams)
    if (kv.first != stream_pool::StreamTagEnum::CudaCompute()) cudaStreamDestroy(kv.second);
  for (void* w : impl_->workspaces) cudaFree(w);
  delete impl_;
}
void Executor::SetCommunicator(void* nccl_comm, int size, int rank) {
  impl_->comm.nccl_comm = nccl_comm;
  impl_->comm.size = impl_->comm.world_size = impl_->comm.local_size = size;
  impl_->comm.rank = impl_->comm.world_rank = impl_->comm.local_rank = rank;
}
void* Executor::StreamOf(int tag) {
  auto it = impl_->streams.find(tag);
  if (it != impl_->streams.end()) return it->second;
  cudaStream_t s = nullptr;
  CUDA_CALL(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  impl_->streams[tag] = s;
  return s;
}
void Executor::Fulfil(op::OpEnv* env) {
  auto req = env->GetRequests();
  for (auto& r : req->stream) *r.dest = StreamOf(r.tag_idx);
  for (auto& r : req->distributed) *r.dest = &impl_->comm;
  for (auto& r : req->workspace) {  // re-allocated before every Execute, as the VM does
    void* p = nullptr;
    CUDA_CALL(cudaMalloc(&p, r.nbytes > 0 ? (size_t)r.nbytes : 16));
    impl_->workspaces.push_back(p);
    *r.dest = p;
  }
}
void Executor::Run(const std::string& base_op, const op::CallValues& call) {
  std::unique_ptr<op::OpEnv> env(op::Dispatch(base_op, call));
  CHECK(env != nullptr) << "no dialect accepts " << base_op;
  Fulfil(env.get());
  env->Execute(call);
  // work on other streams than "compute" is joined before the caller looks at the results
  for (auto& kv : impl_->streams)
    if (kv.first != stream_pool::StreamTagEnum::CudaCompute()) CUDA_CALL(cudaStreamSynchronize(kv.second));
}

}  // namespace compat
}  // namespace raf
