// raf_compat: schema structs of the optimizer operators (generated in RAF from
// scripts/src_codegen/def_schema.py:671-694 into src/op/schema/optimizer.h).
#pragma once
#include <vector>
#include "raf/op.h"
namespace raf {
namespace op {
namespace schema {
struct SgdArgs : ArgsBase {
  value::Value x, dx, v;
  double learning_rate = 0, mu = 0;
};
struct LansArgs : ArgsBase {
  std::vector<value::Value> tensor_list;
  value::Value step;
  float learning_rate = 0, beta1 = 0, beta2 = 0, eps = 0;
  int bias_correction = 0;
  float weight_decay = 0;
  int grad_averaging = 0, mode = 0;
  bool normalize_grad = false;
};
}  // namespace schema
}  // namespace op
}  // namespace raf
