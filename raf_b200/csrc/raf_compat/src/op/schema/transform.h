// raf_compat: cast / group_cast schemas (def_schema.py:525-536 -> src/op/schema/transform.h).
#pragma once
#include <string>
#include <vector>
#include "raf/op.h"
namespace raf {
namespace op {
namespace schema {
struct CastArgs : ArgsBase {
  value::Value data;
  std::string dtype;
};
struct GroupCastArgs : ArgsBase {
  std::vector<value::Value> tensor_list;
  std::string dtype;
};
}  // namespace schema
}  // namespace op
}  // namespace raf
