// raf_compat: dialect and dialect-op registries (include/raf/dialect.h:28-243,
// src/impl/dialect.cc:37-147 of awslabs/raf), restated.
#pragma once
#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "raf/op.h"

namespace raf {
namespace op {

// A dialect is a name that is enabled for device types.
class Dialect {
 public:
  static std::map<std::string, Dialect>& Registry() {
    static std::map<std::string, Dialect> r;
    return r;
  }
  static Dialect& GetOrCreate(const std::string& name) { return Registry()[name]; }
  Dialect& set_name(const std::string& n) {
    name = n;
    return *this;
  }
  Dialect& set_enable(DevType dt) {
    enabled.push_back(dt.code());
    return *this;
  }
  bool is_enabled(DevType dt) const { return std::find(enabled.begin(), enabled.end(), dt.code()) != enabled.end(); }
  std::string name;
  std::vector<int> enabled;
};

// The implementations of one base operator, by dialect, ordered by priority level.
class OpDialect {
 public:
  struct Entry {
    std::string dialect;
    std::string dialect_op;
    int plevel;
  };
  static std::map<std::string, OpDialect>& Registry() {
    static std::map<std::string, OpDialect> r;
    return r;
  }
  static OpDialect& GetOrCreate(const std::string& base) { return Registry()[base]; }
  OpDialect& set_name(const std::string& n) {
    name = n;
    return *this;
  }
  // src/impl/dialect.cc:122-147: two dialects may not share a level on one base operator
  OpDialect& add_dialect(const std::string& dialect, const std::string& dialect_op, int plevel) {
    for (const Entry& e : entries) CHECK_NE(e.plevel, plevel) << "two dialect ops of " << name << " at level " << plevel;
    entries.push_back({dialect, dialect_op, plevel});
    std::sort(entries.begin(), entries.end(), [](const Entry& a, const Entry& b) { return a.plevel > b.plevel; });
    return *this;
  }
  std::string name;
  std::vector<Entry> entries;
};

// src/impl/op.cc:127-215: the first enabled dialect, by descending level, whose OpEnv
// reports no error.  `base_op` is e.g. "raf.op.lans".  Returns nullptr when none accepts.
OpEnv* Dispatch(const std::string& base_op, const CallValues& call);

}  // namespace op
}  // namespace raf

#define RAF_COMPAT_STRINGIZE(S) #S
#define RAF_REGISTER_DIALECT(DIALECT_NAME)                                              \
  static ::raf::op::Dialect& RAF_COMPAT_CONCAT(__make_Dialect, __COUNTER__) =           \
      ::raf::op::Dialect::GetOrCreate(DIALECT_NAME).set_name(DIALECT_NAME)
#define RAF_REGISTER_DIALECT_OP(DIALECT, OP, PLEVEL)                                    \
  static ::raf::op::OpDialect& RAF_COMPAT_CONCAT(__make_OpDialect, __COUNTER__) =       \
      ::raf::op::OpDialect::GetOrCreate(RAF_COMPAT_STRINGIZE(raf.op.OP))                \
          .set_name(RAF_COMPAT_STRINGIZE(raf.op.OP))                                    \
          .add_dialect(#DIALECT, RAF_COMPAT_STRINGIZE(raf.op.DIALECT.OP), PLEVEL)
