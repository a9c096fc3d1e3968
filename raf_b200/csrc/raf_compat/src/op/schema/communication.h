// raf_compat: schema structs of the collective operators of the ZeRO path
// (def_schema.py:699-738 -> src/op/schema/communication.h in RAF).
#pragma once
#include <string>
#include <vector>
#include "raf/op.h"
namespace raf {
namespace op {
namespace schema {
struct AllreduceArgs : ArgsBase {
  std::vector<value::Value> x;
  std::string computation = "sum";
  value::Value rank_list;
};
struct AllgatherArgs : ArgsBase {
  value::Value x;
  int axis = 0;
  value::Value rank_list;
};
struct GroupAllgatherArgs : ArgsBase {
  std::vector<value::Value> tensor_list;
  int axis = 0;
  std::vector<value::Value> out;
};
struct ReduceScatterArgs : ArgsBase {
  value::Value x;
  std::string computation = "sum";
  value::Value rank_list;
};
struct GroupReduceScatterArgs : ArgsBase {
  std::vector<value::Value> tensor_list;
  std::string computation = "sum";
};
}  // namespace schema
}  // namespace op
}  // namespace raf
