// Hand-over of the (b,h,d,e) fp32 KV / dKV state inside a sequence-parallel group over NVLink peer
// memory, fused with the reduction that feeds it and the scan that consumes it.
//
// The reference passes the state rank to rank (recv, update, send), so the last of N ranks waits for
// N-1 serial hops.  The chain
//     X_in(r+1) = a X_in(r) + total(r),   a = exp(-s n) per head,
// has the closed form  X_in(r) = sum_{q<r} a^(r-1-q) total(q),  so one round is enough: every rank
// stores its own `total` straight into the receive slots of the ranks after it (plain peer stores
// through NVSwitch) and each rank sums what it received with the decay powers.  A contribution whose
// decay power is below 1e-12 is neither sent nor awaited (exchange_layout.h), which for decaying heads
// leaves only the nearest ranks.  k_exchange_scan does everything in ONE launch per direction: the
// first CTAs reduce this rank's chunk states to its total and push it; the others wait for the
// senders' words, sum them and run the scan over the local chunk states with the result.
//
// There is no separate "data ready" flag and no system-wide fence on the path: every float travels
// in an 8-byte word together with the step number ({value, step}, written by one 16-byte store per two
// floats), and the receiver simply re-reads a word until it carries the current step.  Step numbers
// only grow and two sets of slots alternate with the step parity, so stale words are never mistaken
// for new ones; the receiver acknowledges a slot slice once it has summed it, so a sender never
// overwrites words that are still being read.  Every wait is bounded: when it runs out the kernel sets
// kFaultRelayWait in the fault word and makes the prefix states it writes NaN.
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
  const float* local;           // (b,h,nc,d*e) chunk states of this rank (read by both halves of the launch)
  float* prefix;                // (b,h,nc,d*e) out: exclusive prefix states seeded with the incoming rank state
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
  int h, de, n, nc, chunk, reverse;
  int n_push;                   // push CTAs of this launch (0: the launch only gathers and scans)
  int gathers;                  // 1: the launch has the gather + scan CTAs and completes the step
  long long elems;
  long long wait_clocks;
};

// this rank's own contribution to the outgoing state at four consecutive elements: the decayed sum of
// its chunk states (what the scan would hand on with a zero incoming state)
__device__ __forceinline__ float4 local_total(const ExchangeParams& p, long long el, float full, float tail) {
  const long long bh = el / p.de;
  const float* base = p.local + (size_t)bh * p.nc * p.de + (el - bh * p.de);
  float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int kBatch = 8;
  for (int i0 = 0; i0 < p.nc; i0 += kBatch) {
    float4 loc[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (i0 + u < p.nc) loc[u] = *reinterpret_cast<const float4*>(base + (size_t)(p.reverse ? p.nc - 1 - (i0 + u) : i0 + u) * p.de);
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (i0 + u < p.nc) {
        const int c = p.reverse ? p.nc - 1 - (i0 + u) : i0 + u;
        const float dec = (c == p.nc - 1) ? tail : full;
        t.x = fmaf(dec, t.x, loc[u].x), t.y = fmaf(dec, t.y, loc[u].y);
        t.z = fmaf(dec, t.z, loc[u].z), t.w = fmaf(dec, t.w, loc[u].w);
      }
  }
  return t;
}

// One launch per direction does the whole state hand-over of a rank: the first CTAs add up this rank's
// chunk states and store the total into the slots of the ranks after it; the others wait for what the
// ranks before stored here, sum it with the decay powers - that is the incoming rank state - and run
// the scan over the local chunk states with it (into a second array: both halves read the chunk states).
__global__ void __launch_bounds__(256) k_exchange_scan(const ExchangeParams p) {
  const uint32_t step = p.counters[0] + 1;
  const int parity = step & 1;
  const int n_push = p.n_push;
  const int last_len = p.n - (p.nc - 1) * p.chunk;
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
    for (long long el = lo + (long long)threadIdx.x * 4; el < hi; el += 256 * 4) {
      const float sh = p.s[(el / p.de) % p.h];
      if (!reaches(sh * (float)p.n, di)) continue;   // decayed to nothing on the way: the receiver does not wait for it
      const float4 t = local_total(p, el, expf(-sh * (float)p.chunk), expf(-sh * (float)last_len));
      st_volatile_v4(out + el, make_uint4(__float_as_uint(t.x), step, __float_as_uint(t.y), step));
      st_volatile_v4(out + el + 2, make_uint4(__float_as_uint(t.z), step, __float_as_uint(t.w), step));
    }
  } else {
    // ---- gather + scan
    int slice, part;
    gather_decode(blockIdx.x - n_push, &slice, &part);
    long long lo, hi;
    part_bounds(p.elems, slice, kGatherCtas, part, &lo, &hi);
    const uint2* slots = p.my_slots + slot_offset(parity, p.ranks, 0, p.elems);
    bool late = false;
    for (long long el = lo + (long long)threadIdx.x * 4; el < hi; el += 256 * 4) {
      const float sh = p.s[(el / p.de) % p.h];
      const float sn = sh * (float)p.n;
      const float a = expf(-sn);
      // incoming state = sum_{q < me} a^(me-1-q) slot[parity][q], each word awaited until it carries `step`
      uint4 w0[kMaxRanks], w1[kMaxRanks];
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) {   // all sources' loads in flight together
        if (q < p.n_src && reaches(sn, p.me - 1 - q)) {
          w0[q] = ld_volatile_v4(slots + (long long)q * p.elems + el);
          w1[q] = ld_volatile_v4(slots + (long long)q * p.elems + el + 2);
        }
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) {   // Horner: acc = a * acc + slot[q]
        if (q < p.n_src) {
          if (reaches(sn, p.me - 1 - q)) {
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
          } else {
            acc.x *= a, acc.y *= a, acc.z *= a, acc.w *= a;
          }
        }
      }
      if (late) {   // a state that did not arrive must not look like one that did
        const float nan = __int_as_float(0x7fc00000);
        acc = make_float4(nan, nan, nan, nan);
      }
      // exclusive scan of the local chunk states seeded with it
      const long long bh = el / p.de;
      const float* base = p.local + (size_t)bh * p.nc * p.de + (el - bh * p.de);
      float* out = p.prefix + (size_t)bh * p.nc * p.de + (el - bh * p.de);
      const float full = expf(-sh * (float)p.chunk), tail = expf(-sh * (float)last_len);
      constexpr int kBatch = 8;
      for (int i0 = 0; i0 < p.nc; i0 += kBatch) {
        float4 loc[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (i0 + u < p.nc) loc[u] = *reinterpret_cast<const float4*>(base + (size_t)(p.reverse ? p.nc - 1 - (i0 + u) : i0 + u) * p.de);
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (i0 + u < p.nc) {
            const int c = p.reverse ? p.nc - 1 - (i0 + u) : i0 + u;
            const float dec = (c == p.nc - 1) ? tail : full;
            *reinterpret_cast<float4*>(out + (size_t)c * p.de) = acc;
            acc.x = fmaf(dec, acc.x, loc[u].x), acc.y = fmaf(dec, acc.y, loc[u].y);
            acc.z = fmaf(dec, acc.z, loc[u].z), acc.w = fmaf(dec, acc.w, loc[u].w);
          }
      }
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
  // the launch that gathers completes the step (a push-only launch ahead of it belongs to the same step)
  if (threadIdx.x == 0 && p.gathers) {
    __threadfence();
    if (atomicAdd(&p.counters[1], 1u) == (uint32_t)(gridDim.x - 1)) {
      p.counters[1] = 0;
      __threadfence();
      p.counters[0] = step;
    }
  }
}

}  // namespace

cudaError_t exchange_scan(const Dims& m, const lasp_exchange_args& a, const float* local, float* prefix,
                          cudaStream_t st) {
  ExchangeParams p;
  p.local = local;
  p.prefix = prefix;
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
  p.h = m.h;
  p.de = m.d * m.e;
  p.n = m.n;
  p.nc = m.nc;
  p.chunk = m.chunk;
  p.reverse = a.reverse;
  p.elems = (long long)m.b * m.h * m.d * m.e;
  p.wait_clocks = a.wait_clocks > 0 ? a.wait_clocks : 20000000000LL;  // about ten seconds
  p.push_parts = push_parts(p.n_dst);
  p.n_push = (a.phase == LASP_EXCHANGE_GATHER) ? 0 : push_ctas(p.n_dst);
  p.gathers = a.phase != LASP_EXCHANGE_PUSH;
  const int ctas = p.n_push + (p.gathers ? kSlices * kGatherCtas : 0);
  if (ctas == 0) return cudaSuccess;   // a push-only launch of the rank that has nobody after it
  k_exchange_scan<<<ctas, 256, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace lasp
