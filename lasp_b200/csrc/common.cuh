// Shared declarations of the lasp_b200 CUDA library (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lasp_b200.h"

namespace lasp {

// Workspace layout (forward and backward use the same one), with S = b*h*nc*d*e
// and nc the number of states kept per sequence.  The chunk-state phase writes
// the LOCAL states, the scan reads them and writes the PREFIX states (exclusive,
// seeded with the incoming rank state) that the output / gradient kernels read:
//   SIMT path        : one state per 64-token chunk, fp32 (b,h,nc,d,e):
//                      [0, S*4) prefix states, [S*4, 2*S*4) local states
//   TENSOR path      : one state per SPAN of `span` 128-token tiles (a few per
//                      sequence; inside a span the state lives on chip):
//                      [0, 4096)            words the CTAs of the fused kernels
//                                           synchronise through (zeroed once by
//                                           the caller, kept by the library)
//                      [4096, 4096 + S*4)   local states: fp32 span totals
//                      [4096 + S*4, + S*4)  prefix states: fp32 states at the span borders
// The running prefix inside the scan is always fp32.
constexpr int kSimtChunk = 64;    // the reference's block size
constexpr int kTensorTile = 128;  // one tcgen05 M=128 tile

struct Dims {
  int b, h, n, d, e;
  int chunk;  // tokens per state kept in the workspace
  int nc;     // states per sequence
  int dtype;
  int path;
  int walk;   // 1 on the tensor path: the state is carried on chip along a span of tiles
  int tiles;  // tensor path: 128-token tiles per sequence
  int span;   // tensor path: tiles per span (chunk = span * 128)
  int pitch_d, pitch_e;  // elements between the rows of consecutive tokens in q,k,dq,dk and in v,o,do,dv
  int qk_map;      // q and k enter as qk_scale * map(x): 0 identity, 1 elu(x) + 1
  float qk_scale;  // (1 when the caller left it 0)
};

inline bool has_qk_preprocessing(const Dims& m) { return m.qk_map != 0 || m.qk_scale != 1.f; }

// SM count of the current device (cached per device ordinal)
int sm_count();

inline size_t state_elems(const Dims& m) { return (size_t)m.b * m.h * m.nc * m.d * m.e; }

// Span states of the walk kernels are kept in global memory in "lane order": the float4 holding
// columns 4g..4g+3 of row r of a d x e state sits at float4 index g*d + r, so that the 32 rows a warp
// owns are contiguous for each of its accesses.  Rank states handed in and out by the caller stay
// row-major; `rows` > 0 on the elementwise kernels below selects the conversion (0 = plain row-major).
__host__ __device__ inline int lane_order_to_row_major(int f4, int rows, int cols) {
  const int g = f4 / rows, r = f4 - g * rows;
  return r * (cols / 4) + g;
}
constexpr size_t kWalkSyncBytes = 4096;
inline uint32_t* ws_walk_sync(void* ws) { return reinterpret_cast<uint32_t*>(ws); }
inline const uint32_t* ws_walk_sync(const void* ws) { return reinterpret_cast<const uint32_t*>(ws); }
inline float* ws_walk_totals(void* ws) { return reinterpret_cast<float*>(static_cast<char*>(ws) + kWalkSyncBytes); }
inline float* ws_walk_border(void* ws, const Dims& m) {
  return reinterpret_cast<float*>(static_cast<char*>(ws) + kWalkSyncBytes + state_elems(m) * 4);
}
inline const float* ws_walk_border(const void* ws, const Dims& m) {
  return reinterpret_cast<const float*>(static_cast<const char*>(ws) + kWalkSyncBytes + state_elems(m) * 4);
}
// where the chunk-state phase writes / where the scan writes and the output kernels read
inline float* ws_local(void* ws, const Dims& m) {
  return m.walk ? ws_walk_totals(ws) : reinterpret_cast<float*>(static_cast<char*>(ws) + state_elems(m) * 4);
}
inline float* ws_prefix(void* ws, const Dims& m) {
  return m.walk ? ws_walk_border(ws, m) : reinterpret_cast<float*>(ws);
}
inline const float* ws_prefix(const void* ws, const Dims& m) {
  return m.walk ? ws_walk_border(ws, m) : reinterpret_cast<const float*>(ws);
}
// bits of the sticky per-device fault word (fault_word.cu owns the word)
enum : int32_t {
  kFaultNone = 0,
  kFaultTmaWait = 1,   // a bounded wait on a TMA mbarrier ran out
  kFaultMmaWait = 2,   // a bounded wait on a tcgen05.commit mbarrier ran out
  kFaultRelayWait = 4, // a bounded wait on a peer's flag ran out (state relay)
  kFaultFlagWait = 8,  // a bounded wait on another CTA's flag ran out (fused kernels)
};
cudaError_t read_fault_word(int32_t* host, bool clear, cudaStream_t st);
// device address of the current device's fault word (for kernels in other translation units)
cudaError_t fault_word_address(int32_t** out);

// name of the host-side step that produced the last cudaError_t (for error text)
extern thread_local const char* g_failed_step;

// ---- launchers implemented in the .cu files (return cudaError_t) -----------
cudaError_t simt_chunk_states(const Dims& m, const void* a, const void* bten, const float* s, float* states,
                              bool backward, cudaStream_t st);
cudaError_t scan_states(const Dims& m, const float* s, const float* local, float* prefix, const float* x_in,
                        float* x_out, bool reverse, cudaStream_t st);
cudaError_t simt_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                            const float* prefix, void* o, cudaStream_t st);
cudaError_t simt_bwd_grads(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                           const float* s, const float* prefix, const float* suffix, void* dq, void* dk,
                           void* dv, cudaStream_t st);
cudaError_t state_combine(int b, int h, int d, int e, int n, const float* s, const float* x_in,
                          const float* x_local, float* x_out, cudaStream_t st);

// state relay (relay_kernels.cu)
cudaError_t exchange_scan(const Dims& m, const lasp_exchange_args& a, const float* local, float* prefix,
                          cudaStream_t st);

// tcgen05 path
bool tensor_path_supported(const Dims& m);

// tcgen05 path with the state carried on chip (walk_kernels.cu)
cudaError_t walk_span_totals(const Dims& m, const void* a, const void* bten, const float* s, float* totals,
                             bool reverse, cudaStream_t st);
cudaError_t walk_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                            const float* prefix, uint32_t* sync, void* o, cudaStream_t st);
cudaError_t walk_fwd_fused(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                           const float* x_in, float* x_out, uint32_t* sync, float* totals, float* prefix, void* o,
                           const lasp_exchange_args* link, cudaStream_t st);
cudaError_t walk_bwd_dq(const Dims& m, const void* q, const void* k, const void* v, const void* d_o, const float* s,
                        const float* prefix, const uint32_t* fwd_sync, void* dq, cudaStream_t st);
cudaError_t walk_bwd_dkv(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                         const float* s, const float* suffix, void* dk, void* dv, cudaStream_t st);
cudaError_t walk_bwd_dkv_fused(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                               const float* s, const float* x_in, float* x_out, uint32_t* sync, float* totals,
                               void* dk, void* dv, const lasp_exchange_args* link, cudaStream_t st);

}  // namespace lasp
