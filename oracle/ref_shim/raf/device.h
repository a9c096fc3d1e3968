/*
 * Stand-in for the one RAF header the reference's LANS kernel pulls in
 * (src/common/cuda_utils.h includes "raf/device.h").  The real header needs
 * TVM and dmlc-core, which are not vendored in the reference tree, so this
 * file declares just the names cuda_utils.h uses: CHECK, LOG(FATAL), the
 * DLPack type codes and a DType with a templated conversion operator.
 * Test infrastructure only; used by oracle/Makefile to build oracle/_ref.
 */
#pragma once
#include <cstdint>
#include <cstdlib>
#include <iostream>
#include <memory>
#include <sstream>
#include <type_traits>

namespace ref_shim {
class Sink {
 public:
  Sink(bool fatal, const char* file, int line) : fatal_(fatal) { os_ << file << ":" << line << ": "; }
  ~Sink() {
    if (fatal_) {
      std::cerr << os_.str() << std::endl;
      std::abort();
    }
  }
  template <typename T>
  Sink& operator<<(const T& v) {
    os_ << v;
    return *this;
  }

 private:
  bool fatal_;
  std::ostringstream os_;
};
}  // namespace ref_shim

#define FATAL 1
#define LOG(severity) ::ref_shim::Sink(true, __FILE__, __LINE__)
#define CHECK(cond) ::ref_shim::Sink(!(cond), __FILE__, __LINE__)

enum { kDLInt = 0, kDLUInt = 1, kDLFloat = 2, kDLBfloat = 4 };

namespace raf {
class DType {
 public:
  int code{kDLFloat};
  int bits{32};
  int lanes{1};
  const char* c_str() const { return "dtype"; }
  template <typename T>
  operator T() const;
};
}  // namespace raf
