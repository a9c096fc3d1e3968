// raf_compat: a small stand-in for the part of RAF's headers that an op dialect touches.
//
// RAF itself cannot be built without its TVM submodule.  This directory restates, from
// RAF's public interface, just enough of the boundary types (values, call values, OpEnv,
// the three registration macros, resource requests, schema structs of the optimizer-step
// operators) for raf_dialect/b200_ops.cc to be compiled, type-checked and driven on fake
// DLTensors by the tests.  Names, members and call shapes follow include/raf/value.h,
// include/raf/op.h, include/raf/dialect.h and src/requests.h of awslabs/raf; the
// implementations are this repository's own and much simpler (no TVM object system: a
// Value is a shared pointer to a small tagged object).
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

// ---- dlpack subset (dlpack.h: DLDataTypeCode, DLDataType, DLDevice, DLTensor) ----------
enum DLDataTypeCode : uint8_t { kDLInt = 0, kDLUInt = 1, kDLFloat = 2, kDLBfloat = 4 };
struct DLDataType {
  uint8_t code;
  uint8_t bits;
  uint16_t lanes;
};
enum DLDeviceType : int32_t { kDLCPU = 1, kDLCUDA = 2 };
struct DLDevice {
  DLDeviceType device_type;
  int32_t device_id;
};
struct DLTensor {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
};

namespace raf {

// include/raf/device.h: DevType, Device
class DevType {
 public:
  static DevType kCPU() { return DevType(1); }
  static DevType kCUDA() { return DevType(2); }
  int code() const { return code_; }
  bool operator==(const DevType& o) const { return code_ == o.code_; }

 private:
  explicit DevType(int c) : code_(c) {}
  int code_;
};
struct Device {
  DevType device_type = DevType::kCUDA();
  int device_id = 0;
};

namespace value {

struct ValueObj {
  virtual ~ValueObj() = default;
};
// A tensor value owns its shape array; `data` belongs to whoever made the value.
struct TensorValueObj : ValueObj {
  DLTensor tensor{};
  std::vector<int64_t> shape;
};
class Value;
struct TupleValueObj : ValueObj {
  std::vector<Value> fields;
};

// include/raf/value.h:73: the base handle.  Converts to DLTensor* when it holds a tensor.
class Value {
 public:
  Value() = default;
  explicit Value(std::shared_ptr<ValueObj> p) : ptr_(std::move(p)) {}
  bool defined() const { return ptr_ != nullptr; }
  ValueObj* get() const { return ptr_.get(); }
  template <typename T>
  T* as_obj() const {
    return dynamic_cast<T*>(ptr_.get());
  }
  operator DLTensor*() const {
    auto* t = as_obj<TensorValueObj>();
    if (!t) throw std::runtime_error("raf_compat: value is not a tensor");
    return &t->tensor;
  }
  operator const DLTensor*() const { return static_cast<DLTensor*>(*this); }

 protected:
  std::shared_ptr<ValueObj> ptr_;
};

template <typename T>
inline T NullValue() {
  return T();
}

// include/raf/value.h:196-275
class TensorValue : public Value {
 public:
  TensorValue() = default;
  explicit TensorValue(const Value& v) : Value(v) {
    if (v.defined() && !v.as_obj<TensorValueObj>()) throw std::runtime_error("raf_compat: not a TensorValue");
  }
  // Wraps caller-owned device memory (what the executor does with the buffers it allocated).
  static TensorValue Assemble(void* data, const std::vector<int64_t>& shape, DLDataType dtype, int device_id = 0) {
    auto obj = std::make_shared<TensorValueObj>();
    obj->shape = shape;
    obj->tensor.data = data;
    obj->tensor.device = DLDevice{kDLCUDA, device_id};
    obj->tensor.ndim = (int32_t)shape.size();
    obj->tensor.dtype = dtype;
    obj->tensor.shape = obj->shape.data();
    obj->tensor.strides = nullptr;
    obj->tensor.byte_offset = 0;
    return TensorValue(Value(obj));
  }
};

class TupleValue : public Value {
 public:
  TupleValue() = default;
  explicit TupleValue(const Value& v) : Value(v) {
    if (v.defined() && !v.as_obj<TupleValueObj>()) throw std::runtime_error("raf_compat: not a TupleValue");
  }
  template <typename ArrayT>
  static TupleValue make(const ArrayT& fields) {
    auto obj = std::make_shared<TupleValueObj>();
    obj->fields.assign(fields.begin(), fields.end());
    return TupleValue(Value(obj));
  }
  TupleValueObj* operator->() const { return as_obj<TupleValueObj>(); }
};

}  // namespace value

namespace ir {
// tvm::runtime::Array<T> as far as the glue uses it: built from an iterator range.
template <typename T>
class Array {
 public:
  Array() = default;
  template <typename It>
  Array(It first, It last) : v_(first, last) {}
  typename std::vector<T>::const_iterator begin() const { return v_.begin(); }
  typename std::vector<T>::const_iterator end() const { return v_.end(); }
  size_t size() const { return v_.size(); }
  const T& operator[](size_t i) const { return v_[i]; }

 private:
  std::vector<T> v_;
};
template <typename T>
inline T Downcast(const value::Value& v) {
  return T(v);
}
}  // namespace ir
}  // namespace raf
