// Exchange of the (b,h,d,e) fp32 KV / dKV state inside a sequence-parallel
// group over NVLink peer memory, and the reduction that feeds it.
//
// The reference passes the state rank to rank (recv, update, send), so the
// last of N ranks waits for N-1 serial hops.  The chain
//     X_in(r+1) = a X_in(r) + total(r),   a = exp(-s n) per head,
// has the closed form  X_in(r) = sum_{q<r} a^(r-1-q) total(q),  so one round is
// enough: every rank stores its own `total` straight into the receive slots of
// all ranks after it (plain peer stores through NVSwitch) and each rank sums
// what it received with the decay powers.  k_state_exchange does both halves in
// ONE launch: the first CTAs push, the others wait for the senders' flags and
// gather.  One NVLink latency per direction instead of N-1.
//
// There is no separate "data ready" flag and no system-wide fence on the path:
// every float travels in an 8-byte word together with the step number
// ({value, step}, written by one 16-byte store per two floats), and the receiver
// simply re-reads a word until it carries the current step.  Step numbers only
// grow and two sets of slots alternate with the step parity, so stale words are
// never mistaken for new ones; the receiver acknowledges a slot slice once it
// has summed it, so a sender never overwrites words that are still being read.
// Every wait is bounded: when it runs out the kernel sets kFaultRelayWait in the
// fault word and carries on (its output is then meaningless).
#include "common.cuh"
#include "exchange_layout.h"

namespace lasp {

namespace {

using namespace xl;

__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile(uint32_t* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// spins until *flag >= want (as a step number) or `limit` clocks pass
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, long long limit) {
  if ((int32_t)(ld_volatile(flag) - want) >= 0) return true;
  const long long t0 = clock64();
  while ((int32_t)(ld_volatile(flag) - want) < 0) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}

struct ExchangeParams {
  const float* total;           // local (b,h,d,e): this rank's own contribution
  float* x_in;                  // local (b,h,d,e) out: the incoming state (NULL: no sender before me)
  const float* s;               // h decay rates
  const uint2* my_slots;        // local: slots[parity][source][element] of {value, step} words
  uint32_t* src_acks[kMaxRanks];    // peer: ack words [me][slice] in each source's memory
  uint2* dst_slots[kMaxRanks];      // peer: each destination's slots
  const uint32_t* my_acks;      // local ack words [destination][slice]
  uint32_t* counters;           // local: [0] = last completed step, [1] = CTAs done, [2 + slice] = gather CTAs done
  int32_t* fault;
  int push_parts;               // CTAs per (destination, slice)
  int me;                       // my position in the chain order (0 = first sender)
  int n_src;                    // sources = positions 0..me-1
  int n_dst;                    // destinations = positions me+1..me+n_dst
  int ranks;                    // group size (slot stride)
  int h, de, n;
  long long elems;
  long long wait_clocks;
};

__global__ void __launch_bounds__(256) k_state_exchange(const ExchangeParams p) {
  const uint32_t step = p.counters[0] + 1;
  const int parity = step & 1;
  const int n_push = push_ctas(p.n_dst);
  if ((int)blockIdx.x < n_push) {
    // ---- push: my total -> slot [parity][me] of one destination, one slice part
    int di, slice, part;
    push_decode(blockIdx.x, p.push_parts, &di, &slice, &part);
    const int dst = p.me + 1 + di;
    long long lo, hi;
    part_bounds(p.elems, slice, p.push_parts, part, &lo, &hi);
    if (threadIdx.x == 0 && needs_ack_wait(step)) {
      // the slot was last used two steps ago: its reader must have acknowledged it
      if (!wait_flag(p.my_acks + ack_index(dst, slice), step - 2, p.wait_clocks)) atomicOr(p.fault, kFaultRelayWait);
    }
    __syncthreads();
    uint2* out = p.dst_slots[dst] + slot_offset(parity, p.ranks, p.me, p.elems);
    constexpr int kUnroll = 4;
    for (long long base = lo + (long long)threadIdx.x * 4; base < hi; base += 256 * 4 * kUnroll) {
      float4 t[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long el = base + (long long)u * 256 * 4;
        if (el < hi) t[u] = *reinterpret_cast<const float4*>(p.total + el);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long el = base + (long long)u * 256 * 4;
        if (el < hi) {
          st_volatile_v4(out + el, make_uint4(__float_as_uint(t[u].x), step, __float_as_uint(t[u].y), step));
          st_volatile_v4(out + el + 2, make_uint4(__float_as_uint(t[u].z), step, __float_as_uint(t[u].w), step));
        }
      }
    }
  } else if (p.x_in) {
    // ---- gather: x_in = sum_{q < me} a^(me-1-q) slot[parity][q], each word awaited until it carries `step`
    int slice, part;
    gather_decode(blockIdx.x - n_push, &slice, &part);
    long long lo, hi;
    part_bounds(p.elems, slice, kGatherCtas, part, &lo, &hi);
    const uint2* slots = p.my_slots + slot_offset(parity, p.ranks, 0, p.elems);
    bool late = false;
    for (long long el = lo + (long long)threadIdx.x * 4; el < hi; el += 256 * 4) {
      const float a = expf(-p.s[(el / p.de) % p.h] * (float)p.n);
      uint4 w0[kMaxRanks], w1[kMaxRanks];
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) {   // all sources' loads in flight together
        if (q < p.n_src) {
          w0[q] = ld_volatile_v4(slots + (long long)q * p.elems + el);
          w1[q] = ld_volatile_v4(slots + (long long)q * p.elems + el + 2);
        }
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) {   // Horner: acc = a * acc + slot[q]
        if (q < p.n_src) {
          if (!late && (w0[q].y != step || w0[q].w != step || w1[q].y != step || w1[q].w != step)) {
            const long long t0 = clock64();  // after one wait has run out this thread waits no more
            do {
              w0[q] = ld_volatile_v4(slots + (long long)q * p.elems + el);
              w1[q] = ld_volatile_v4(slots + (long long)q * p.elems + el + 2);
              if (clock64() - t0 > p.wait_clocks) {
                late = true;
                break;
              }
            } while (w0[q].y != step || w0[q].w != step || w1[q].y != step || w1[q].w != step);
          }
          acc.x = fmaf(a, acc.x, __uint_as_float(w0[q].x));
          acc.y = fmaf(a, acc.y, __uint_as_float(w0[q].z));
          acc.z = fmaf(a, acc.z, __uint_as_float(w1[q].x));
          acc.w = fmaf(a, acc.w, __uint_as_float(w1[q].z));
        }
      }
      *reinterpret_cast<float4*>(p.x_in + el) = acc;
    }
    if (late) atomicOr(p.fault, kFaultRelayWait);
    __syncthreads();
    // the last CTA of a slice to finish tells every source that the slice has been read
    if (threadIdx.x == 0) {
      if (atomicAdd(&p.counters[2 + slice], 1u) == (uint32_t)(kGatherCtas - 1)) {
        p.counters[2 + slice] = 0;
        for (int q = 0; q < p.n_src; ++q) st_volatile(p.src_acks[q] + ack_index(p.me, slice), step);
      }
    }
  }
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&p.counters[1], 1u) == (uint32_t)(gridDim.x - 1)) {
      p.counters[1] = 0;
      __threadfence();
      p.counters[0] = step;
    }
  }
}

// total[bh][el] = sum_c decay(chunks after c) * local[bh][c][el]; bf16 or fp32 local states
template <typename T>
__global__ void __launch_bounds__(128) k_state_total(const float* __restrict__ s, const T* __restrict__ local,
                                                     float* __restrict__ total, int h, int n, int de, int nc,
                                                     int chunk, int reverse, int lane_rows, int cols) {
  const int bh = blockIdx.y;
  const int el = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (el >= de) return;
  const float sh = s[bh % h];
  const float full = expf(-sh * (float)chunk);
  const float tail = expf(-sh * (float)(n - (nc - 1) * chunk));
  float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
  const T* base = local + (size_t)bh * nc * de + el;
  constexpr int kBatch = 8;
  for (int i0 = 0; i0 < nc; i0 += kBatch) {
    float4 loc[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = i0 + u;
      if (i < nc) {
        const T* src = base + (size_t)(reverse ? nc - 1 - i : i) * de;
        if constexpr (sizeof(T) == 4) {
          loc[u] = *reinterpret_cast<const float4*>(src);
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(src);
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          loc[u] = make_float4(a.x, a.y, b.x, b.y);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = i0 + u;
      if (i < nc) {
        const int c = reverse ? nc - 1 - i : i;
        const float dec = (c == nc - 1) ? tail : full;
        p.x = fmaf(dec, p.x, loc[u].x);
        p.y = fmaf(dec, p.y, loc[u].y);
        p.z = fmaf(dec, p.z, loc[u].z);
        p.w = fmaf(dec, p.w, loc[u].w);
      }
    }
  }
  const int ext = lane_rows > 0 ? lane_order_to_row_major(el / 4, lane_rows, cols) * 4 : el;
  *reinterpret_cast<float4*>(total + (size_t)bh * de + ext) = p;
}

}  // namespace

cudaError_t state_total(const Dims& m, const float* s, const void* local, float* total, bool reverse,
                        cudaStream_t st) {
  const int de = m.d * m.e;
  dim3 grid((de / 4 + 127) / 128, m.b * m.h);
  if (m.path == LASP_PATH_TENSOR && !m.walk)
    k_state_total<__nv_bfloat16><<<grid, 128, 0, st>>>(s, static_cast<const __nv_bfloat16*>(local), total, m.h, m.n,
                                                        de, m.nc, m.chunk, reverse ? 1 : 0, 0, m.e);
  else
    k_state_total<float><<<grid, 128, 0, st>>>(s, m.walk ? ws_walk_border(local, m) : static_cast<const float*>(local),
                                               total, m.h, m.n, de, m.nc, m.chunk, reverse ? 1 : 0, m.walk ? m.d : 0,
                                               m.e);
  return cudaGetLastError();
}

cudaError_t state_exchange(const lasp_exchange_args& a, cudaStream_t st) {
  ExchangeParams p;
  p.total = a.total;
  p.x_in = a.x_in;
  p.s = a.s;
  p.my_slots = static_cast<const uint2*>(a.my_slots);
  p.my_acks = a.my_acks;
  p.counters = a.counters;
  for (int i = 0; i < kMaxRanks; ++i) {
    p.src_acks[i] = a.peer_acks[i];
    p.dst_slots[i] = static_cast<uint2*>(a.peer_slots[i]);
  }
  cudaError_t err = fault_word_address(&p.fault);
  if (err != cudaSuccess) return err;
  p.me = a.position;
  p.n_src = a.position;
  p.n_dst = a.ranks - 1 - a.position;
  p.ranks = a.ranks;
  p.h = a.h;
  p.de = a.d * a.e;
  p.n = a.n;
  p.elems = (long long)a.b * a.h * a.d * a.e;
  p.wait_clocks = a.wait_clocks > 0 ? a.wait_clocks : 4000000000LL;  // about two seconds
  p.push_parts = push_parts(p.n_dst);
  const int ctas = push_ctas(p.n_dst) + gather_ctas(p.n_src);
  if (ctas == 0) return cudaSuccess;
  k_state_exchange<<<ctas, 256, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace lasp
