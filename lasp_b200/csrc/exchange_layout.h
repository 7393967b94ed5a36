// Index arithmetic of the state-exchange kernel (relay_kernels.cu), kept free of
// CUDA types so that the same functions run in the kernel and in the host-side
// protocol simulation of the test-suite.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define LASP_HD __host__ __device__ __forceinline__
#else
#define LASP_HD inline
#endif

namespace lasp {
namespace xl {

constexpr int kMaxRanks = 8;
constexpr int kSlices = 8;        // independently acknowledged slices of a state
constexpr int kGatherCtas = 16;   // CTAs per slice on the gathering side
constexpr int kPushTarget = 128;  // CTAs on the pushing side, shared among (destination, slice) pairs
constexpr int kAckStride = 32;    // acknowledgement words sit 128 bytes apart
constexpr int kThreads = 256;
constexpr int kVec = 4;           // floats per thread and access

// floats per slice: a multiple of kVec that covers elems in kSlices pieces
LASP_HD long long slice_len(long long elems) { return ((elems / kVec + kSlices - 1) / kSlices) * kVec; }

// [lo, hi) of part `part` of `parts` inside slice `slice`
LASP_HD void part_bounds(long long elems, int slice, int parts, int part, long long* lo, long long* hi) {
  const long long per = slice_len(elems);
  const long long slo = (long long)slice * per;
  long long shi = slo + per;
  if (shi > elems) shi = elems;
  const long long sub = ((per / kVec + parts - 1) / parts) * kVec;
  long long l = slo + (long long)part * sub, h = l + sub;
  if (h > shi) h = shi;
  if (l > shi) l = shi;
  *lo = l;
  *hi = h;
}

// CTAs per (destination, slice) for a rank with n_dst destinations
LASP_HD int push_parts(int n_dst) {
  if (n_dst <= 0) return 1;
  const int p = kPushTarget / (n_dst * kSlices);
  return p > 1 ? p : 1;
}
LASP_HD int push_ctas(int n_dst) { return n_dst * kSlices * push_parts(n_dst); }
LASP_HD int gather_ctas(int n_src) { return n_src > 0 ? kSlices * kGatherCtas : 0; }

// push CTA `block` -> destination index (0 = the next position), slice, part
LASP_HD void push_decode(int block, int parts, int* dst_index, int* slice, int* part) {
  *part = block % parts;
  *slice = (block / parts) % kSlices;
  *dst_index = block / (parts * kSlices);
}
// gather CTA index (block - push_ctas) -> slice, part
LASP_HD void gather_decode(int gi, int* slice, int* part) {
  *part = gi % kGatherCtas;
  *slice = gi / kGatherCtas;
}

// offset, in 8-byte {value, step} words, of element 0 of `source`'s state in a rank's slots
LASP_HD long long slot_offset(int parity, int ranks, int source, long long elems) {
  return ((long long)parity * ranks + source) * elems;
}
// index of the acknowledgement word for (position, slice) in a rank's ack array
LASP_HD int ack_index(int position, int slice) { return (position * kSlices + slice) * kAckStride; }

// A state that has to cross `hops` whole ranks of n tokens on its way arrives multiplied by
// exp(-s n hops).  Below exp(-kDecayCutoff) (about 1e-12, far under the resolution of the fp32 sum it
// would join) it is neither sent nor waited for; sender and receiver apply the same rule.
constexpr float kDecayCutoff = 27.6f;
LASP_HD bool reaches(float s_times_n, int hops) { return s_times_n * (float)hops <= kDecayCutoff; }

// a pusher may overwrite the slot of parity (step & 1) once the step two before has been acknowledged
LASP_HD bool needs_ack_wait(uint32_t step) { return step >= 3; }

}  // namespace xl
}  // namespace lasp
