// Forward pass for callers that cannot allocate device memory.
//
// Some hosts of this library hand every byte of the GPU to a pool of their own
// at start-up (an inference server that pre-reserves the device), or call the
// operator from a section where cudaMalloc / cudaFree - which may synchronise
// the whole device - are not allowed (a latency-critical serving loop).  Such
// a caller has nowhere to get the chunk-state workspace from.  This file gives
// the forward pass a workspace that lives inside the library image: a
// file-scope __device__ array that every GPU loading the library holds until
// the process exits.
#include <mutex>

#include "common.cuh"

namespace {

// the workspace itself: LASP_B200_STATIC_SCRATCH_BYTES on every device
static __device__ __align__(256) unsigned char g_static_scratch[LASP_B200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
void* g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle for the runtime, not an
// address a kernel can use: the device address is asked for once per device,
// with that device current, and cached.
cudaError_t scratch_address(void** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> guard(g_setup_lock);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return err;
    if (!ptr) return cudaErrorInvalidSymbol;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int lasp_b200_forward_static(const lasp_problem* p, const lasp_fwd_args* a, void* stream) {
  if (!p || !a) return LASP_ERR_NULL;
  const int path = lasp_b200_resolve_path(p);  // full shape / dtype validation
  if (path < 0) return path;
  const size_t need = lasp_b200_fwd_workspace_bytes(p);
  if (need == 0 || need > (size_t)LASP_B200_STATIC_SCRATCH_BYTES) return LASP_ERR_TOO_LARGE;
  void* scratch = nullptr;
  if (scratch_address(&scratch) != cudaSuccess) return LASP_ERR_CUDA;
  lasp_fwd_args with_ws = *a;
  with_ws.ws = scratch;
  with_ws.ws_bytes = (size_t)LASP_B200_STATIC_SCRATCH_BYTES;
  // every chunk state the scan and the output kernel read is written by the
  // chunk-state kernel of this same call, so nothing has to be cleared first
  return lasp_b200_forward(p, &with_ws, stream);
}
