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
}}}  // namespace raf::op::b200
