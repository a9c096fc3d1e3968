// raf_compat: OpEnv, CallValues, the OpEnv maker registry and resource requests
// (include/raf/op.h:33-101,331-334 and src/requests.h:15-49 of awslabs/raf), restated.
#pragma once
#include <cuda_runtime.h>

#include <functional>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "raf/value.h"

// ---- dmlc-style checks: a failed check throws (RAF: dmlc::Error up to Python) -----------
namespace raf {
namespace compat {
class CheckFailure {
 public:
  CheckFailure(const char* file, int line, const char* what) { os_ << file << ":" << line << ": check failed: " << what << " "; }
  [[noreturn]] ~CheckFailure() noexcept(false) { throw std::runtime_error(os_.str()); }
  std::ostringstream& stream() { return os_; }

 private:
  std::ostringstream os_;
};
}  // namespace compat
}  // namespace raf
#define CHECK(cond) \
  if (!(cond)) ::raf::compat::CheckFailure(__FILE__, __LINE__, #cond).stream()
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_NE(a, b) CHECK((a) != (b))
#define CUDA_CALL(expr)                                                        \
  do {                                                                         \
    cudaError_t e__ = (expr);                                                  \
    CHECK(e__ == cudaSuccess) << "CUDA: " << cudaGetErrorString(e__);          \
  } while (0)

namespace raf {
namespace op {

// The attribute object of a call: the schema struct of the operator (src/op/schema/*.h).
struct ArgsBase {
  virtual ~ArgsBase() = default;
};
class Attrs {
 public:
  Attrs() = default;
  explicit Attrs(std::shared_ptr<ArgsBase> p) : ptr_(std::move(p)) {}
  template <typename T>
  const T* as() const {
    return dynamic_cast<const T*>(ptr_.get());
  }

 private:
  std::shared_ptr<ArgsBase> ptr_;
};

// include/raf/op.h:33-57
struct CallValuesNode {
  value::Value callee;
  Attrs args;
  value::Value out;
  Device device;
};
class CallValues {
 public:
  static CallValues make(value::Value callee = {}, Attrs args = {}) {
    CallValues cv;
    cv.node_ = std::make_shared<CallValuesNode>();
    cv.node_->callee = callee;
    cv.node_->args = args;
    return cv;
  }
  CallValuesNode* operator->() const { return node_.get(); }

 private:
  std::shared_ptr<CallValuesNode> node_;
};

// src/requests.h:15-49: what an OpEnv asked for; the executor fills *dest.
struct Requests {
  struct WorkspaceRequest {
    void** dest;
    Device device;
    int64_t nbytes;
  };
  struct StreamRequest {
    void** dest;
    Device device;
    int tag_idx;
  };
  struct DistributedRequest {
    void** dest;
    std::string name;
    value::Value rank_list;
  };
  std::vector<WorkspaceRequest> workspace;
  std::vector<StreamRequest> stream;
  std::vector<DistributedRequest> distributed;
};

// include/raf/op.h:59-101
class OpEnv {
 public:
  OpEnv() : requests_(std::make_shared<Requests>()) {}
  virtual ~OpEnv() = default;
  virtual std::string name() const = 0;
  virtual void Execute(const CallValues& call) = 0;
  virtual void Execute(const std::vector<value::Value>& inputs, value::Value output) = 0;

  std::vector<std::string> error_msgs;
  bool HasError() { return !error_msgs.empty(); }

  void RequestWorkspace(void** dest, const Device& device, int64_t nbytes) {
    requests_->workspace.push_back({dest, device, nbytes});
  }
  void RequestStream(void** dest, const Device& device, int tag_idx) {
    requests_->stream.push_back({dest, device, tag_idx});
  }
  void RequestDistributed(void** dest, const std::string& name, const value::Value rank_list) {
    requests_->distributed.push_back({dest, name, rank_list});
  }
  std::shared_ptr<Requests> GetRequests() const { return requests_; }
  std::vector<int> arg_indices;

 private:
  std::shared_ptr<Requests> requests_;
};

using FMakeOpEnv = std::function<OpEnv*(const CallValues&)>;

// include/raf/op.h:103-130: name -> factory
class OpEnvMaker {
 public:
  static std::map<std::string, OpEnvMaker>& Registry() {
    static std::map<std::string, OpEnvMaker> r;
    return r;
  }
  static OpEnvMaker& GetOrCreate(const std::string& name) { return Registry()[name]; }
  OpEnvMaker& set_name(const std::string& n) {
    name = n;
    return *this;
  }
  OpEnvMaker& set_func(FMakeOpEnv f) {
    func = std::move(f);
    return *this;
  }
  std::string name;
  FMakeOpEnv func;
};

// FRAFSchemaFieldIndex: position of a named field in an operator's argument list
// (generated from scripts/src_codegen/def_schema.py in RAF).
using FRAFSchemaFieldIndex = std::function<int(const std::string&)>;

inline std::string GetUniqueName(const std::string& name) { return name; }
inline std::string TruncateName(const std::string& name) { return name.size() > 80 ? name.substr(0, 80) : name; }

}  // namespace op

namespace ir {
// ir::Op::Get / GetAttrMap as the glue uses them: an op is its name; the only attribute
// map asked for is the schema field index.
class Op {
 public:
  Op() = default;
  explicit Op(std::string n) : name(std::move(n)) {}
  static Op Get(const std::string& name) { return Op(name); }
  struct FieldIndexMap {
    op::FRAFSchemaFieldIndex operator[](const Op& op) const;
  };
  template <typename T>
  static FieldIndexMap GetAttrMap(const std::string&) {
    return FieldIndexMap();
  }
  std::string name;
};
}  // namespace ir

namespace op {
// argument names of the base operators, in schema order (def_schema.py:525-536,671-738 and
// the memory ops): filled by raf_compat/registry.cc
const std::vector<std::string>& SchemaFieldNames(const std::string& base_op);
}  // namespace op
}  // namespace raf

#define RAF_COMPAT_CONCAT_(a, b) a##b
#define RAF_COMPAT_CONCAT(a, b) RAF_COMPAT_CONCAT_(a, b)
#define RAF_OP_ENV_MAKER(OP_NAME, FOP_ENV_MAKER)                                        \
  static ::raf::op::OpEnvMaker& RAF_COMPAT_CONCAT(__make_OpEnvMaker, __COUNTER__) =     \
      ::raf::op::OpEnvMaker::GetOrCreate(OP_NAME).set_name(OP_NAME).set_func(FOP_ENV_MAKER)
