// raf_compat: fuse_tensor / defuse_tensor schemas (def_schema.py:829-841 -> src/op/schema/memory.h).
#pragma once
#include <cstdint>
#include <vector>
#include "raf/op.h"
namespace raf {
namespace op {
namespace schema {
struct FuseTensorArgs : ArgsBase {
  std::vector<value::Value> data;
};
struct DefuseTensorArgs : ArgsBase {
  value::Value data;
  std::vector<int64_t> sizes, shapes, shape_indices;
};
}  // namespace schema
}  // namespace op
}  // namespace raf
