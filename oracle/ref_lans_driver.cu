/*
 * C entry point around the reference's own multi_tensor_lans_cuda<float>
 * (src/op/dialect/cuda/kernels/multi_tensor_lans.cu:401-450), which
 * oracle/Makefile compiles UNCHANGED from the reference tree next to this
 * file.  Test infrastructure: it lets the GPU tests and the benchmark run the
 * reference kernel on the same device buffers as this repository's kernels.
 *
 * The pointer list is laid out as the reference's host code builds it
 * (src/op/dialect/cuda/lans.cc:111-123): [g..., q..., p..., m..., v...].
 * q_layout 0 gives every tensor its own q region (a prefix sum of numels);
 * q_layout 1 reproduces lans.cc:116-119, q_i = q_buf + numels[i-1], whose
 * regions overlap for three or more tensors.
 */
#include <cuda_runtime.h>
#include <cmath>
#include <vector>

namespace raf {
namespace op {
namespace cuda {
template <typename T>
void multi_tensor_lans_cuda(int chunk_size, std::vector<T*> tensor_lists, const float lr,
                            const float beta1, const float beta2, const float epsilon,
                            const int bias_correction, const float bias_correction1,
                            const float bias_correction2, const float beta3,
                            const float weight_decay, const int grad_averaging, const int mode,
                            const bool normalize_grad, const std::vector<int> numels, void* stream,
                            float* output_per_tensor, float* grad_norm_tensor,
                            float* param_norm_tensor, float* update_m_norm, float* q_norm_tensor,
                            int max_chunks_per_tensor);
}
}  // namespace op
}  // namespace raf

extern "C" __attribute__((visibility("default"))) size_t ref_lans_workspace_floats(
    int k, const int* numels, int* max_chunks_out) {
  const int chunk = 65536;
  size_t total = 0;
  int max_chunks = 1;
  for (int i = 0; i < k; ++i) {
    total += (size_t)numels[i];
    int c = (numels[i] + chunk - 1) / chunk;
    if (c > max_chunks) max_chunks = c;
  }
  if (max_chunks_out) *max_chunks_out = max_chunks;
  /* q + chunk partials + four norm vectors (lans.cc:66,74-78) */
  return total + (size_t)k * max_chunks + 4 * (size_t)k;
}

/* Device pointers g/p/m/v[k]; workspace of ref_lans_workspace_floats() floats.
 * norms_out (device, 4*k floats, optional): g, p, update_m, update_g norms. */
extern "C" __attribute__((visibility("default"))) int ref_lans(
    int k, float* const* g, float* const* p, float* const* m, float* const* v, const int* numels,
    int step, float lr, float beta1, float beta2, float eps, int bias_correction,
    float weight_decay, int grad_averaging, int mode, int normalize_grad, float* workspace,
    int q_layout, float* norms_out, void* stream) {
  int max_chunks = 1;
  size_t total = ref_lans_workspace_floats(k, numels, &max_chunks) - (size_t)k * max_chunks - 4 * (size_t)k;
  float* q_buf = workspace;
  float* partials = q_buf + total;
  float* gn = partials + (size_t)k * max_chunks;
  float* pn = gn + k;
  float* umn = pn + k;
  float* qn = umn + k;

  float bc1 = 1.0f, bc2 = 1.0f; /* lans.cc:100-105 */
  if (bias_correction == 1) {
    bc1 = 1 - std::pow(beta1, step);
    bc2 = 1 - std::pow(beta2, step);
  }
  float beta3 = 1.0f; /* lans.cc:106-109 */
  if (grad_averaging == 1) beta3 = 1 - beta1;

  std::vector<int> nvec(numels, numels + k);
  std::vector<float*> tl;
  for (int i = 0; i < k; ++i) tl.push_back(g[i]);
  if (q_layout == 1) {
    tl.push_back(q_buf);
    for (int i = 1; i < k; ++i) tl.push_back(q_buf + numels[i - 1]);
  } else {
    size_t off = 0;
    for (int i = 0; i < k; ++i) {
      tl.push_back(q_buf + off);
      off += (size_t)numels[i];
    }
  }
  for (int i = 0; i < k; ++i) tl.push_back(p[i]);
  for (int i = 0; i < k; ++i) tl.push_back(m[i]);
  for (int i = 0; i < k; ++i) tl.push_back(v[i]);

  raf::op::cuda::multi_tensor_lans_cuda<float>(65536, tl, lr, beta1, beta2, eps, bias_correction,
                                               bc1, bc2, beta3, weight_decay, grad_averaging, mode,
                                               normalize_grad != 0, nvec, stream, partials, gn, pn,
                                               umn, qn, max_chunks);
  if (norms_out) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaMemcpyAsync(norms_out, gn, sizeof(float) * k, cudaMemcpyDeviceToDevice, s);
    cudaMemcpyAsync(norms_out + k, pn, sizeof(float) * k, cudaMemcpyDeviceToDevice, s);
    cudaMemcpyAsync(norms_out + 2 * k, umn, sizeof(float) * k, cudaMemcpyDeviceToDevice, s);
    cudaMemcpyAsync(norms_out + 3 * k, qn, sizeof(float) * k, cudaMemcpyDeviceToDevice, s);
  }
  return (int)cudaGetLastError();
}
