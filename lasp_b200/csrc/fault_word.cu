// The sticky per-device fault word: kernels set bits in it when one of their bounded waits runs out
// (see the kFault* codes in common.cuh) instead of spinning for ever; the host reads and clears it.
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

cudaError_t fault_word_address(int32_t** out) {
  static int32_t* cached[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!cached[dev]) {
    void* p = nullptr;
    if ((err = cudaGetSymbolAddress(&p, g_fault_word)) != cudaSuccess) return err;
    cached[dev] = static_cast<int32_t*>(p);
  }
  *out = cached[dev];
  return cudaSuccess;
}

}  // namespace lasp
