// tcgen05 / TMEM / TMA kernels (placeholder until the tensor path lands).
#include "common.cuh"

namespace lasp {

__device__ int32_t g_fault_word = 0;

cudaError_t read_fault_word(int32_t* host, bool clear, cudaStream_t st) {
  cudaError_t err = cudaMemcpyFromSymbolAsync(host, g_fault_word, sizeof(int32_t), 0, cudaMemcpyDeviceToHost, st);
  if (err != cudaSuccess) return err;
  err = cudaStreamSynchronize(st);
  if (err != cudaSuccess || !clear) return err;
  const int32_t zero = 0;
  err = cudaMemcpyToSymbolAsync(g_fault_word, &zero, sizeof(int32_t), 0, cudaMemcpyHostToDevice, st);
  if (err != cudaSuccess) return err;
  return cudaStreamSynchronize(st);
}

bool tensor_path_supported(const Dims&) { return false; }

cudaError_t tensor_chunk_states(const Dims&, const void*, const void*, const float*, float*, bool, cudaStream_t) {
  return cudaErrorNotSupported;
}
cudaError_t tensor_fwd_output(const Dims&, const void*, const void*, const void*, const float*,
                              const __nv_bfloat16*, void*, cudaStream_t) {
  return cudaErrorNotSupported;
}
cudaError_t tensor_bwd_grads(const Dims&, const void*, const void*, const void*, const void*, const float*,
                             const __nv_bfloat16*, const __nv_bfloat16*, void*, void*, void*, cudaStream_t) {
  return cudaErrorNotSupported;
}

}  // namespace lasp
