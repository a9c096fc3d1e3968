// raf_compat: include/raf/nccl_communicator.h:21-28 of awslabs/raf.  nccl_comm is an
// ncclComm_t; kept as void* so that this header needs no NCCL.
#pragma once
#include "raf/communicator.h"
namespace raf {
namespace distributed {
namespace communicator {
struct NCCLCommunicatorObj : CommunicatorObj {
  void* nccl_comm = nullptr;
};
}  // namespace communicator
}  // namespace distributed
}  // namespace raf
