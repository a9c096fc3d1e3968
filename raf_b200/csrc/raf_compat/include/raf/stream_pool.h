// raf_compat: stream tags (include/raf/stream_pool.h:22-66 of awslabs/raf).
#pragma once
namespace raf {
namespace stream_pool {
class StreamTagEnum {
 public:
  static int Reserved() { return 0; }
  static int CudaCompute() { return 1; }
  static int MemCpuToCuda() { return 2; }
  static int MemCudaToCpu() { return 3; }
  static int CudaCommunicate() { return 4; }
  static int MemCudaToCuda1() { return 5; }
  static int MemCudaToCuda2() { return 6; }
};
}  // namespace stream_pool
}  // namespace raf
