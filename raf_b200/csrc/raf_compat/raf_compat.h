// raf_compat: a minimal executor for the tests - dispatch, fulfil the requests, Execute.
#pragma once
#include <string>

#include "raf/op.h"

namespace raf {
namespace compat {
class Executor {
 public:
  explicit Executor(void* compute_stream);
  ~Executor();
  Executor(const Executor&) = delete;
  // the communicator RequestDistributed hands out (size 1 = the void communicator)
  void SetCommunicator(void* nccl_comm, int size, int rank);
  void* StreamOf(int tag);
  void Fulfil(op::OpEnv* env);
  // Dispatch(base_op) -> requests -> Execute(call)
  void Run(const std::string& base_op, const op::CallValues& call);

 private:
  struct Impl;
  Impl* impl_;
};
}  // namespace compat
}  // namespace raf
