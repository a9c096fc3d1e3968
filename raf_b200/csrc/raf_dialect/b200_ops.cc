// RAF-side glue of libraf_b200: an op dialect "b200" whose OpEnvs forward DLTensor pointers
// to the C ABI of include/raf_b200.h.  This file belongs INTO a RAF source tree
// (src/op/dialect/b200/b200_ops.cc) and is compiled by RAF's build, not by this package's:
// it needs RAF's headers (raf/op.h, raf/dialect.h, ...) and, through them, TVM.  It is kept
// here so that the integration described next to it can be applied by copying one file.
// Registration levels sit above the stock implementations (nccl 10, cuda.lans 20, tvm 10).
#include "raf/op.h"
#include "raf/dialect.h"
#include "raf/device_api.h"
#include "raf/stream_pool.h"
#include "raf/communicator.h"
#include "raf/nccl_communicator.h"
#include "../../schema/optimizer.h"
#include "../../schema/communication.h"
#include "../../schema/transform.h"
#include "../../schema/memory.h"
#include "raf_b200.h"

namespace raf { namespace op { namespace b200 {
using namespace raf::value;
using stream_pool::StreamTagEnum;

RAF_REGISTER_DIALECT("b200").set_enable(DevType::kCUDA());

static void Check(int status) { CHECK_EQ(status, RAFB200_OK) << rafb200_last_error(); }

static int DTypeOf(const DLTensor* t, std::vector<std::string>* err) {
  if (t->dtype.code == kDLFloat && t->dtype.bits == 32) return RAFB200_F32;
  if (t->dtype.code == kDLFloat && t->dtype.bits == 16) return RAFB200_F16;
  if (t->dtype.code == kDLBfloat && t->dtype.bits == 16) return RAFB200_BF16;
  err->push_back("b200: unsupported dtype");   // soft failure: dispatch tries the next dialect
  return RAFB200_F32;
}
static int64_t Numel(const DLTensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->shape[i];
  return n;
}

// ---- raf.op.lans  (replaces LansImpl, src/op/dialect/cuda/lans.cc:25-165) ------------------
class LansB200 : public OpEnv {
  rafb200_tensor_list_t list_{nullptr};
  void* workspace_{nullptr};
  size_t workspace_bytes_{0};
  void* stream_{nullptr};
  int k_{0};
  float lr_, beta1_, beta2_, eps_, wd_;
  int bias_correction_, grad_averaging_, mode_, normalize_grad_;

 public:
  explicit LansB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op.lans");
    auto args = cv->args.as<op::schema::LansArgs>();
    this->arg_indices = {fidx[base]("tensor_list"), fidx[base]("step")};
    lr_ = args->learning_rate; beta1_ = args->beta1; beta2_ = args->beta2; eps_ = args->eps;
    bias_correction_ = args->bias_correction; wd_ = args->weight_decay;
    grad_averaging_ = args->grad_averaging; mode_ = args->mode;
    normalize_grad_ = args->normalize_grad;
    CHECK_EQ(args->tensor_list.size() % 4, 0U);
    k_ = args->tensor_list.size() / 4;
    std::vector<int64_t> numel(k_);
    for (int i = 0; i < k_; ++i) {
      const DLTensor* t = ir::Downcast<TensorValue>(args->tensor_list[i]);
      numel[i] = Numel(t);
    }
    const DLTensor* g0 = ir::Downcast<TensorValue>(args->tensor_list[0]);
    Check(rafb200_tensor_list_create(k_, numel.data(), DTypeOf(g0, &error_msgs), RAFB200_F32, &list_));
    workspace_bytes_ = rafb200_lans_workspace_bytes(list_);
    RequestWorkspace(&workspace_, cv->device, workspace_bytes_);      // a few KB instead of 4*numel
    RequestStream(&stream_, cv->device, StreamTagEnum::CudaCompute());
  }
  ~LansB200() { rafb200_tensor_list_destroy(list_); }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200.lans")); }

  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::LansArgs>();
    Execute({TupleValue::make(ir::Array<Value>(args->tensor_list.begin(), args->tensor_list.end())),
             args->step}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    auto tuple = ir::Downcast<TupleValue>(inputs[0]);
    std::vector<const void*> g(k_);
    std::vector<float*> p(k_), m(k_), v(k_);
    for (int i = 0; i < k_; ++i) {
      g[i] = static_cast<const DLTensor*>(ir::Downcast<TensorValue>(tuple->fields[i]))->data;
      p[i] = static_cast<float*>(static_cast<const DLTensor*>(ir::Downcast<TensorValue>(tuple->fields[k_ + i]))->data);
      m[i] = static_cast<float*>(static_cast<const DLTensor*>(ir::Downcast<TensorValue>(tuple->fields[2 * k_ + i]))->data);
      v[i] = static_cast<float*>(static_cast<const DLTensor*>(ir::Downcast<TensorValue>(tuple->fields[3 * k_ + i]))->data);
    }
    const DLTensor* step = ir::Downcast<TensorValue>(inputs[1]);   // 0-d fp32 on the device
    Check(rafb200_tensor_list_bind(list_, g.data(), p.data(), m.data(), v.data(), nullptr, stream_));
    // The workspace pointer is re-filled by the VM before every Execute: read it here, never cache it.
    Check(rafb200_lans(list_, /*step=*/0, static_cast<const float*>(step->data), lr_, beta1_, beta2_,
                       eps_, bias_correction_, wd_, grad_averaging_, mode_, normalize_grad_,
                       /*grad_scale=*/1.0f, workspace_, workspace_bytes_, stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new LansB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, lans, 30);
RAF_OP_ENV_MAKER("raf.op.b200.lans", LansB200::make);

class SgdB200 : public OpEnv {
  void* stream_{nullptr};
  float lr_, mu_;
 public:
  explicit SgdB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op.sgd");
    auto args = cv->args.as<op::schema::SgdArgs>();
    this->arg_indices = {fidx[base]("x"), fidx[base]("dx"), fidx[base]("v")};
    lr_ = args->learning_rate; mu_ = args->mu;
    const DLTensor* x = args->x;
    if (!(x->dtype.code == kDLFloat && x->dtype.bits == 32)) error_msgs.push_back("b200.sgd: fp32 master only");
    RequestStream(&stream_, cv->device, StreamTagEnum::CudaCompute());
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200.sgd")); }
  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::SgdArgs>();
    Execute({args->x, args->dx, args->v}, cv->out);
  }
  void Execute(const std::vector<Value>& in, Value output) override {
    const DLTensor* x = ir::Downcast<TensorValue>(in[0]);
    const DLTensor* dx = ir::Downcast<TensorValue>(in[1]);
    const DLTensor* v = ir::Downcast<TensorValue>(in[2]);
    auto out = ir::Downcast<TupleValue>(output);                       // (v1, x1): note the order
    DLTensor* v1 = ir::Downcast<TensorValue>(out->fields[0]);
    DLTensor* x1 = ir::Downcast<TensorValue>(out->fields[1]);
    const int64_t n = Numel(x);
    auto s = static_cast<cudaStream_t>(stream_);
    if (v1->data != v->data) CUDA_CALL(cudaMemcpyAsync(v1->data, v->data, 4 * n, cudaMemcpyDeviceToDevice, s));
    if (x1->data != x->data) CUDA_CALL(cudaMemcpyAsync(x1->data, x->data, 4 * n, cudaMemcpyDeviceToDevice, s));
    Check(rafb200_sgd(static_cast<float*>(x1->data), dx->data, DTypeOf(dx, &error_msgs),
                      static_cast<float*>(v1->data), n, lr_, mu_, /*weight_decay=*/0.f,
                      /*grad_scale=*/1.f, /*out=*/nullptr, RAFB200_F32, stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new SgdB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, sgd, 20);
RAF_OP_ENV_MAKER("raf.op.b200.sgd", SgdB200::make);

class GroupReduceScatterB200 : public OpEnv {
  void* stream_{nullptr};
  void* communicator_{nullptr};
  rafb200_comm_t comm_{nullptr};
  std::string computation_;
 public:
  explicit GroupReduceScatterB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op._group_reduce_scatter");
    this->arg_indices = {fidx[base]("tensor_list")};
    RequestStream(&stream_, cv->device, StreamTagEnum::CudaCommunicate());
    RequestDistributed(&communicator_, "nccl", NullValue<Value>());
    computation_ = cv->args.as<op::schema::GroupReduceScatterArgs>()->computation;
  }
  ~GroupReduceScatterB200() { rafb200_comm_destroy(comm_); }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200._group_reduce_scatter")); }
  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::GroupReduceScatterArgs>();
    Execute({TupleValue::make(ir::Array<Value>(args->tensor_list.begin(), args->tensor_list.end()))}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    auto* c = reinterpret_cast<distributed::communicator::NCCLCommunicatorObj*>(communicator_);
    if (!comm_) Check(rafb200_comm_adopt(c->nccl_comm, c->size, c->rank, &comm_));
    auto in = ir::Downcast<TupleValue>(inputs[0]);
    auto out = ir::Downcast<TupleValue>(output);
    const int k = in->fields.size();
    std::vector<const void*> src(k);
    std::vector<void*> dst(k);
    std::vector<int64_t> count(k);                      // elements each rank RECEIVES
    int dtype = RAFB200_F32;
    for (int i = 0; i < k; ++i) {
      const DLTensor* x = ir::Downcast<TensorValue>(in->fields[i]);
      DLTensor* y = ir::Downcast<TensorValue>(out->fields[i]);
      src[i] = x->data; dst[i] = y->data; count[i] = Numel(y); dtype = DTypeOf(x, &error_msgs);
    }
    Check(rafb200_group_reduce_scatter(comm_, k, src.data(), dst.data(), count.data(), dtype,
                                       computation_.c_str(), stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new GroupReduceScatterB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, _group_reduce_scatter, 20);
RAF_OP_ENV_MAKER("raf.op.b200._group_reduce_scatter", GroupReduceScatterB200::make);

// ---- the remaining ops of the path: same three steps (parse the schema in the constructor,
// request stream / communicator, forward DLTensor::data in Execute) ---------------------------

// Shared by the collectives: RAF's communicator object, adopted once.
class CommEnv : public OpEnv {
 protected:
  void* stream_{nullptr};
  void* communicator_{nullptr};
  rafb200_comm_t comm_{nullptr};
  explicit CommEnv(const CallValues& cv, const Value& rank_list) {
    RequestStream(&stream_, cv->device, StreamTagEnum::CudaCommunicate());
    RequestDistributed(&communicator_, "nccl", rank_list);
  }
  ~CommEnv() { rafb200_comm_destroy(comm_); }
  rafb200_comm_t Comm() {
    if (!comm_) {
      auto* c = reinterpret_cast<distributed::communicator::NCCLCommunicatorObj*>(communicator_);
      Check(rafb200_comm_adopt(c->nccl_comm, c->size, c->rank, &comm_));
    }
    return comm_;
  }
};

class ReduceScatterB200 : public CommEnv {
  std::string computation_;
 public:
  explicit ReduceScatterB200(const CallValues& cv)
      : CommEnv(cv, cv->args.as<op::schema::ReduceScatterArgs>()->rank_list) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op._reduce_scatter");
    this->arg_indices = {fidx[base]("x")};
    computation_ = cv->args.as<op::schema::ReduceScatterArgs>()->computation;
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200._reduce_scatter")); }
  void Execute(const CallValues& cv) override {
    Execute({cv->args.as<op::schema::ReduceScatterArgs>()->x}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    const DLTensor* x = ir::Downcast<TensorValue>(inputs[0]);
    DLTensor* y = ir::Downcast<TensorValue>(output);
    Check(rafb200_reduce_scatter(Comm(), x->data, y->data, Numel(y), DTypeOf(x, &error_msgs),
                                 computation_.c_str(), stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new ReduceScatterB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, _reduce_scatter, 20);
RAF_OP_ENV_MAKER("raf.op.b200._reduce_scatter", ReduceScatterB200::make);

class AllGatherB200 : public CommEnv {
 public:
  explicit AllGatherB200(const CallValues& cv)
      : CommEnv(cv, cv->args.as<op::schema::AllgatherArgs>()->rank_list) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op._allgather");
    this->arg_indices = {fidx[base]("x")};
    // NCCL gathers on axis 0; python/raf/distributed/op.py:20-88 swaps other axes in and out.
    if (cv->args.as<op::schema::AllgatherArgs>()->axis != 0) error_msgs.push_back("b200._allgather: axis 0 only");
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200._allgather")); }
  void Execute(const CallValues& cv) override {
    Execute({cv->args.as<op::schema::AllgatherArgs>()->x}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    const DLTensor* x = ir::Downcast<TensorValue>(inputs[0]);
    DLTensor* y = ir::Downcast<TensorValue>(output);
    Check(rafb200_allgather(Comm(), x->data, y->data, Numel(x), DTypeOf(x, &error_msgs), stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new AllGatherB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, _allgather, 20);
RAF_OP_ENV_MAKER("raf.op.b200._allgather", AllGatherB200::make);

// _group_allgather writes into the caller's `out` tuple (TRAFInplaceUpdate {2:0}).
class GroupAllGatherB200 : public CommEnv {
 public:
  explicit GroupAllGatherB200(const CallValues& cv) : CommEnv(cv, NullValue<Value>()) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op._group_allgather");
    this->arg_indices = {fidx[base]("tensor_list"), fidx[base]("out")};
    if (cv->args.as<op::schema::GroupAllgatherArgs>()->axis != 0)
      error_msgs.push_back("b200._group_allgather: axis 0 only");
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200._group_allgather")); }
  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::GroupAllgatherArgs>();
    Execute({TupleValue::make(ir::Array<Value>(args->tensor_list.begin(), args->tensor_list.end())),
             TupleValue::make(ir::Array<Value>(args->out.begin(), args->out.end()))}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    auto in = ir::Downcast<TupleValue>(inputs[0]);
    auto out = ir::Downcast<TupleValue>(inputs[1]);
    const int k = in->fields.size();
    std::vector<const void*> src(k);
    std::vector<void*> dst(k);
    std::vector<int64_t> count(k);
    int dtype = RAFB200_F32;
    for (int i = 0; i < k; ++i) {
      const DLTensor* x = ir::Downcast<TensorValue>(in->fields[i]);
      DLTensor* y = ir::Downcast<TensorValue>(out->fields[i]);
      src[i] = x->data; dst[i] = y->data; count[i] = Numel(x); dtype = DTypeOf(x, &error_msgs);
    }
    Check(rafb200_group_allgather(Comm(), k, src.data(), dst.data(), count.data(), dtype, stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new GroupAllGatherB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, _group_allgather, 20);
RAF_OP_ENV_MAKER("raf.op.b200._group_allgather", GroupAllGatherB200::make);

// _allreduce is in place on every tensor of x (TRAFInplaceUpdate {0:0}); no packing workspace.
class AllReduceB200 : public CommEnv {
  std::string computation_;
 public:
  explicit AllReduceB200(const CallValues& cv)
      : CommEnv(cv, cv->args.as<op::schema::AllreduceArgs>()->rank_list) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op._allreduce");
    this->arg_indices = {fidx[base]("x")};
    computation_ = cv->args.as<op::schema::AllreduceArgs>()->computation;
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200._allreduce")); }
  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::AllreduceArgs>();
    Execute({TupleValue::make(ir::Array<Value>(args->x.begin(), args->x.end()))}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    auto in = ir::Downcast<TupleValue>(inputs[0]);
    for (size_t i = 0; i < in->fields.size(); ++i) {
      const DLTensor* x = ir::Downcast<TensorValue>(in->fields[i]);
      DLTensor* y = in->fields.size() == 1 ? static_cast<DLTensor*>(ir::Downcast<TensorValue>(output))
                                           : static_cast<DLTensor*>(ir::Downcast<TensorValue>(
                                                 ir::Downcast<TupleValue>(output)->fields[i]));
      Check(rafb200_allreduce(Comm(), x->data, y->data, Numel(x), DTypeOf(x, &error_msgs),
                              computation_.c_str(), stream_));
    }
  }
  static OpEnv* make(const CallValues& cv) { return new AllReduceB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, _allreduce, 20);
RAF_OP_ENV_MAKER("raf.op.b200._allreduce", AllReduceB200::make);

// cast / group_cast / fuse_tensor / defuse_tensor run on the compute stream.
class CastB200 : public OpEnv {
  void* stream_{nullptr};
 public:
  explicit CastB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op.cast");
    this->arg_indices = {fidx[base]("data")};
    RequestStream(&stream_, cv->device, StreamTagEnum::CudaCompute());
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200.cast")); }
  void Execute(const CallValues& cv) override { Execute({cv->args.as<op::schema::CastArgs>()->data}, cv->out); }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    const DLTensor* x = ir::Downcast<TensorValue>(inputs[0]);
    DLTensor* y = ir::Downcast<TensorValue>(output);
    Check(rafb200_cast(x->data, DTypeOf(x, &error_msgs), y->data, DTypeOf(y, &error_msgs), Numel(x), stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new CastB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, cast, 20);
RAF_OP_ENV_MAKER("raf.op.b200.cast", CastB200::make);

class GroupCastB200 : public OpEnv {
  void* stream_{nullptr};
 public:
  explicit GroupCastB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op.group_cast");
    this->arg_indices = {fidx[base]("tensor_list")};
    RequestStream(&stream_, cv->device, StreamTagEnum::CudaCompute());
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200.group_cast")); }
  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::GroupCastArgs>();
    Execute({TupleValue::make(ir::Array<Value>(args->tensor_list.begin(), args->tensor_list.end()))}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    auto in = ir::Downcast<TupleValue>(inputs[0]);
    auto out = ir::Downcast<TupleValue>(output);
    const int k = in->fields.size();
    if (k == 0) return;
    std::vector<const void*> src(k);
    std::vector<void*> dst(k);
    std::vector<int64_t> numel(k);
    for (int i = 0; i < k; ++i) {
      const DLTensor* x = ir::Downcast<TensorValue>(in->fields[i]);
      DLTensor* y = ir::Downcast<TensorValue>(out->fields[i]);
      src[i] = x->data; dst[i] = y->data; numel[i] = Numel(x);
    }
    const DLTensor* x0 = ir::Downcast<TensorValue>(in->fields[0]);
    const DLTensor* y0 = ir::Downcast<TensorValue>(out->fields[0]);
    Check(rafb200_group_cast(k, src.data(), DTypeOf(x0, &error_msgs), dst.data(), DTypeOf(y0, &error_msgs),
                             numel.data(), stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new GroupCastB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, group_cast, 20);
RAF_OP_ENV_MAKER("raf.op.b200.group_cast", GroupCastB200::make);

// fuse_tensor / defuse_tensor (replace CudaFuseTensor / CudaDefuseTensor,
// src/op/dialect/cuda/memory.cc:20-134): one launch instead of one copy per tensor.
class FuseTensorB200 : public OpEnv {
  void* stream_{nullptr};
 public:
  explicit FuseTensorB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op.fuse_tensor");
    this->arg_indices = {fidx[base]("data")};
    RequestStream(&stream_, cv->device, StreamTagEnum::MemCudaToCuda1());
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200.fuse_tensor")); }
  void Execute(const CallValues& cv) override {
    auto args = cv->args.as<op::schema::FuseTensorArgs>();
    Execute({TupleValue::make(ir::Array<Value>(args->data.begin(), args->data.end()))}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    auto in = ir::Downcast<TupleValue>(inputs[0]);
    DLTensor* flat = ir::Downcast<TensorValue>(output);
    const int k = in->fields.size();
    std::vector<const void*> src(k);
    std::vector<int64_t> numel(k), offset(k);
    int64_t at = 0;
    for (int i = 0; i < k; ++i) {
      const DLTensor* x = ir::Downcast<TensorValue>(in->fields[i]);
      src[i] = x->data; numel[i] = Numel(x); offset[i] = at; at += numel[i];
    }
    Check(rafb200_fuse_tensor(k, src.data(), numel.data(), offset.data(), flat->dtype.bits / 8, flat->data, stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new FuseTensorB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, fuse_tensor, 20);
RAF_OP_ENV_MAKER("raf.op.b200.fuse_tensor", FuseTensorB200::make);

class DefuseTensorB200 : public OpEnv {
  void* stream_{nullptr};
  std::vector<int64_t> sizes_;
 public:
  explicit DefuseTensorB200(const CallValues& cv) {
    static auto fidx = ir::Op::GetAttrMap<op::FRAFSchemaFieldIndex>("FRAFSchemaFieldIndex");
    static auto base = ir::Op::Get("raf.op.defuse_tensor");
    this->arg_indices = {fidx[base]("data")};
    sizes_ = cv->args.as<op::schema::DefuseTensorArgs>()->sizes;
    RequestStream(&stream_, cv->device, StreamTagEnum::MemCudaToCuda2());
  }
  std::string name() const override { return TruncateName(GetUniqueName("raf.op.b200.defuse_tensor")); }
  void Execute(const CallValues& cv) override {
    Execute({cv->args.as<op::schema::DefuseTensorArgs>()->data}, cv->out);
  }
  void Execute(const std::vector<Value>& inputs, Value output) override {
    const DLTensor* flat = ir::Downcast<TensorValue>(inputs[0]);
    auto out = ir::Downcast<TupleValue>(output);
    const int k = out->fields.size();
    std::vector<void*> dst(k);
    std::vector<int64_t> offset(k);
    int64_t at = 0;
    for (int i = 0; i < k; ++i) {
      DLTensor* y = ir::Downcast<TensorValue>(out->fields[i]);
      dst[i] = y->data; offset[i] = at; at += sizes_[i];
    }
    Check(rafb200_defuse_tensor(k, dst.data(), sizes_.data(), offset.data(), flat->dtype.bits / 8, flat->data, stream_));
  }
  static OpEnv* make(const CallValues& cv) { return new DefuseTensorB200(cv); }
};
RAF_REGISTER_DIALECT_OP(b200, defuse_tensor, 20);
RAF_OP_ENV_MAKER("raf.op.b200.defuse_tensor", DefuseTensorB200::make);

}}}  // namespace raf::op::b200
