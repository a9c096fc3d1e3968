// raf_compat: the communicator object an OpEnv receives from RequestDistributed
// (include/raf/communicator.h:52-62 of awslabs/raf).
#pragma once
#include <string>
namespace raf {
namespace distributed {
namespace communicator {
struct CommunicatorObj {
  virtual ~CommunicatorObj() = default;
  int local_size = 1, local_rank = 0, size = 1, rank = 0, world_size = 1, world_rank = 0, root_rank = 0;
};
}  // namespace communicator
}  // namespace distributed
}  // namespace raf
