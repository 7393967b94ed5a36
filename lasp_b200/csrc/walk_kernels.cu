// Tensor-core path (tcgen05 MMAs, accumulators in tensor memory, operands staged by TMA) with the
// running KV / dKV state kept ON CHIP.  bf16 inputs, fp32 accumulation, one rounding on store.
//
// A sequence of one (batch, head) is cut into 128-token tiles and the tiles into spans of `span`
// consecutive tiles; a span is the unit of work of a persistent CTA.  Per direction:
//
//   k_span_totals   T_span = sum over the span's tokens of decay * a_j b_j^T  (a,b = k,v or q,do)
//   (scan over the few span totals of a sequence: k_scan of simt_kernels.cu, seeded with the rank's
//    incoming state; gives every span its fp32 state at the span border)
//   k_walk_out      walks a span first to last tile with the d x e state in registers (fp32) and in
//                   shared memory (bf16 MMA operand):  OUT = (X Y^T . M) Z + diag(lambda^r) X op(P),
//                   then P <- lambda^C P + K^T diag(w) V.  Forward: (X,Y,Z,OUT) = (Q,K,V,O), op(P)=P;
//                   the same kernel gives dQ with (X,Y,Z,OUT) = (dO,V,K,dQ), op(P)=P^T.
//   k_walk_dkv      walks a span last to first tile with the suffix state Dn on chip: dK, dV.
//
// So K and V (Q and dO) are read twice per direction and nothing else is: no per-tile state is written
// to or read from global memory.  Every tile in shared memory is in the swizzled slab format of
// sm100.cuh; all buffers are 32 KB so that a tile's buffer can be reused for the decay-masked score
// tile and for the staging tile of the TMA store.  All waits are bounded (see tc_common.cuh).
#include <stdio.h>
#include <stdlib.h>

#include "exchange_layout.h"
#include "tc_common.cuh"

namespace lasp {

namespace {

using namespace tc;

#ifdef LASP_TRACE
__device__ long long g_trace[160 * 64];
#define TRACE(slot) do { if (blockIdx.x < 160 && (slot) < 64) g_trace[blockIdx.x * 64 + (slot)] = clock64(); } while (0)
__device__ __forceinline__ long long gtime() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define GTRACE(slot) do { if (blockIdx.x < 160) g_trace[blockIdx.x * 64 + (slot)] = gtime(); } while (0)
#else
#define TRACE(slot) do {} while (0)
#define GTRACE(slot) do {} while (0)
#endif

constexpr int kBuf = 32768;       // one shared-memory buffer: a 128 x 128 bf16 tile

// Two buffers of a double-buffered tile / two accumulators, addressed by arithmetic: an array of two pointers
// indexed by the tile's parity would live in local memory, and the tile loops look these up all the time.
struct BufPair {
  uint8_t* base;
  __device__ __forceinline__ uint8_t* operator[](int p) const { return base + p * kBuf; }
};
struct TmemPair {
  uint32_t base;
  __device__ __forceinline__ uint32_t operator[](int p) const { return base + p * 128; }
};
struct IntPair {
  int a, b;
  __device__ __forceinline__ int get(int p) const { return p ? b : a; }
  __device__ __forceinline__ void set(int p, int v) {
    if (p) b = v; else a = v;
  }
};
constexpr int kWorkers = 256;     // warps 2..9

// Global-memory image of a d x e span state in lane order (see common.cuh): this thread's part is row
// `row`, columns [col0, col0 + N).
template <int N, int ROWS, bool COHERENT>
__device__ __forceinline__ void load_state(const float* state, int row, int col0, float (&P)[N]) {
  const float4* src = reinterpret_cast<const float4*>(state) + (size_t)(col0 / 4) * ROWS + row;
#pragma unroll
  for (int q = 0; q < N / 4; ++q) {
    const float4 v = COHERENT ? __ldcg(src + (size_t)q * ROWS) : src[(size_t)q * ROWS];
    P[4 * q] = v.x, P[4 * q + 1] = v.y, P[4 * q + 2] = v.z, P[4 * q + 3] = v.w;
  }
}
template <int N, int ROWS>
__device__ __forceinline__ void fma_state(const float* state, int row, int col0, float dec, float (&P)[N]) {
  const float4* src = reinterpret_cast<const float4*>(state) + (size_t)(col0 / 4) * ROWS + row;
  float4 v[N / 4];
#pragma unroll
  for (int q = 0; q < N / 4; ++q) v[q] = __ldcg(src + (size_t)q * ROWS);   // written by another CTA of this launch
#pragma unroll
  for (int q = 0; q < N / 4; ++q) {
    P[4 * q] = fmaf(dec, v[q].x, P[4 * q]), P[4 * q + 1] = fmaf(dec, v[q].y, P[4 * q + 1]);
    P[4 * q + 2] = fmaf(dec, v[q].z, P[4 * q + 2]), P[4 * q + 3] = fmaf(dec, v[q].w, P[4 * q + 3]);
  }
}
template <int N, int ROWS>
__device__ __forceinline__ void store_state(float* state, int row, int col0, const float (&P)[N]) {
  float4* dst = reinterpret_cast<float4*>(state) + (size_t)(col0 / 4) * ROWS + row;
#pragma unroll
  for (int q = 0; q < N / 4; ++q) dst[(size_t)q * ROWS] = make_float4(P[4 * q], P[4 * q + 1], P[4 * q + 2], P[4 * q + 3]);
}
// 32 accumulator columns of this thread's row -> lane-order state
template <int ROWS>
__device__ __forceinline__ void store_state32(float* state, int row, int col0, const uint32_t (&r)[32]) {
  float4* dst = reinterpret_cast<float4*>(state) + (size_t)(col0 / 4) * ROWS + row;
#pragma unroll
  for (int q = 0; q < 8; ++q)
    dst[(size_t)q * ROWS] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                        __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
}


// ---------------------------------------------------------------------------
// span totals: totals[item][i][j] = sum_c w_c A[c][i] B[c][j] over the span's tokens
//   forward  (A,B) = (K,V):  w = lambda^(span end - position)      (decayed to the end of the span)
//   backward (A,B) = (Q,dO): w = lambda^(position - span start)    (decayed to the start of the span)
// Ten warps: warp 0 producer (three-stage ring of A,B tiles), warp 1 tensor-core issuer (accumulator
// double buffered over items), warps 2-5 scale the rows of A in place, warps 6-9 write the totals.
// ---------------------------------------------------------------------------
template <int D, int E>
__global__ void __launch_bounds__(320, 1) k_span_totals(const __grid_constant__ CUtensorMap map_a,
                                                        const __grid_constant__ CUtensorMap map_b,
                                                        const float* __restrict__ s, float* __restrict__ totals,
                                                        int h, int n, int tiles, int span, int nspans, int items,
                                                        int reverse, int32_t* fault) {
  constexpr int kStages = 3;
  constexpr int kA = C * D * 2, kB = C * E * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  // per stage: A then B (with D = 64 the M = 128 MMA reads on from A into B, which is valid memory)
  __shared__ uint64_t full[kStages], scaled[kStages], empty[kStages], acc_full[2], acc_free[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    dead = 0;
    for (int j = 0; j < kStages; ++j) {
      mbar_init(&full[j], 1);
      mbar_init(&scaled[j], 128);
      mbar_init(&empty[j], 1);
    }
    for (int j = 0; j < 2; ++j) {
      mbar_init(&acc_full[j], 1);
      mbar_init(&acc_free[j], 128);
    }
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 2) tmem_alloc(&tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  TileWalk w{items, nspans, span, tiles, 0, false, false};

  if (warp == 0) {
    if (lane == 0) {
      int g = 0;
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++g) {
        const int j = g % kStages, use = g / kStages;
        if (use >= 1) wait_or_fault(&empty[j], (use - 1) & 1, &dead, fault, kFaultMmaWait);
        uint8_t* sa = smem + j * (kA + kB);
        mbar_expect_tx(&full[j], kA + kB);
        tma_load_4d(sa, &map_a, &full[j], 0, w.t * C, 0, w.bh);
        tma_load_4d(sa + kA, &map_b, &full[j], 0, w.t * C, 0, w.bh);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int g = 0, li = -1;
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++g) {
        const int j = g % kStages, use = g / kStages;
        if (w.first_of_item()) {
          ++li;
          if (li >= 2) wait_or_fault(&acc_free[li & 1], ((li >> 1) - 1) & 1, &dead, fault, kFaultMmaWait);
        }
        wait_or_fault(&scaled[j], use & 1, &dead, fault, kFaultTmaWait);
        tc_fence_after_sync();
        uint8_t* sa = smem + j * (kA + kB);
        umma_gemm(tmem + 128 * (li & 1), Operand{smem_u32(sa), C, true}, Operand{smem_u32(sa + kA), C, true}, E, C / 16,
                  !w.first_of_item());
        umma_commit(&empty[j]);
        if (w.last_of_item()) umma_commit(&acc_full[li & 1]);
      }
    }
  } else if (warp < 6) {
    const int row = tid - 64;  // the token of the tile this thread scales
    int g = 0;
    for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++g) {
      const int j = g % kStages, use = g / kStages;
      const float sl2 = s[w.bh % h] * kLog2e;
      const int pos = w.t * C + row;
      const int dist = reverse ? pos - w.t0 * C : min(w.t1 * C, n) - pos;
      const float wt = decay_pow(sl2, max(dist, 0));  // rows past the end of the sequence are zero anyway
      wait_or_fault(&full[j], use & 1, &dead, fault, kFaultTmaWait);
      scale_row_pieces<D / 8>(smem + j * (kA + kB), row, 0, wt, lane);
      fence_async_smem();
      mbar_arrive(&scaled[j]);
    }
  } else {
    const int row = (warp & 3) * 32 + lane;  // tensor-memory lane = row of the state; warps 6..9 -> quarters 2,3,0,1
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int li = -1;
    for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next()) {
      if (!w.last_of_item()) continue;
      ++li;
      wait_or_fault(&acc_full[li & 1], (li >> 1) & 1, &dead, fault, kFaultMmaWait);
      tc_fence_after_sync();
      if (row < D) {
#pragma unroll
        for (int c0 = 0; c0 < E; c0 += 32) {
          uint32_t a[32];
          tmem_ld32(tmem + 128 * (li & 1) + lane_base + c0, a);
          tmem_ld_wait();
          store_state32<D>(totals + (size_t)w.it * D * E, row, c0, a);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_free[li & 1]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------
// flags between the CTAs of one launch (fused kernels)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// spins until *flag == want or `limit` clocks pass
__device__ __forceinline__ bool wait_flag_eq(const uint32_t* flag, uint32_t want, long long limit) {
  if (ld_volatile_u32(flag) == want) return true;
  const long long t0 = clock64();
  while (ld_volatile_u32(flag) != want) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}

// The peer-mapped buffers of a sequence-parallel group for one direction (word format, slots and
// acknowledgements as in relay_kernels.cu).  With a link the fused kernels hand the rank state over
// themselves: the CTA that owns the last span of a sequence (in walk order) stores the sequence's total
// into the slots of the ranks after this one as soon as the span totals exist, and every CTA adds what
// the ranks before stored here to its border state - one launch per direction computes AND exchanges.
struct Link {
  const uint2* my_slots;                 // local: slots[parity][source][element] of {value, step} words
  uint2* dst_slots[xl::kMaxRanks];       // peer: each destination's slots
  uint32_t* src_acks[xl::kMaxRanks];     // peer: acknowledgement words in each source's memory
  const uint32_t* my_acks;               // local acknowledgement words [destination]
  uint32_t* counters;                    // local: [0] = last completed step
  int ranks;                             // group size; 0 = no link
  int me;                                // this rank's place in the chain order
  long long wait_clocks;
};

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

// Where the two 16-byte halves of the four {value, step} words of float4 chunk g, row `row`, of a
// sequence sit among its slots (in words): per chunk two planes of ROWS x 16 bytes, so that the 32 rows
// of a warp write - and read - 512 contiguous bytes with each instruction.
template <int ROWS>
__device__ __forceinline__ size_t link_word(int g, int row, int plane) {
  return (size_t)g * ROWS * 4 + (size_t)plane * ROWS * 2 + (size_t)row * 2;
}

// This thread's part (row `row`, columns [col0, col0 + N)) of a sequence's outgoing total, dec * P + own,
// written over `own` (the total of the sequence's last span in walk order, which no other CTA reads).
template <int N, int ROWS>
__device__ __forceinline__ void link_make_total(float* own, int row, int col0, float dec, const float (&P)[N]) {
  float4* t = reinterpret_cast<float4*>(own) + (size_t)(col0 / 4) * ROWS + row;
#pragma unroll 4
  for (int q = 0; q < N / 4; ++q) {
    const float4 o = __ldcg(t + (size_t)q * ROWS);
    t[(size_t)q * ROWS] = make_float4(fmaf(dec, P[4 * q], o.x), fmaf(dec, P[4 * q + 1], o.y),
                                      fmaf(dec, P[4 * q + 2], o.z), fmaf(dec, P[4 * q + 3], o.w));
  }
}

// One CTA's share of the sending: of this thread's float4 chunks of the sequence's total, those whose index
// is `part` modulo `parts`, stored as {value, step} words into the slots of every rank after this one
// that the state still reaches.  All CTAs of a sequence send, each its share: one SM alone pushes slowly.
template <int N, int ROWS>
__device__ __forceinline__ void link_send_part(const Link& l, uint32_t step, long long elems, size_t seq_off, int row,
                                               int col0, const float* total, float sn, int part, int parts) {
  const float4* src = reinterpret_cast<const float4*>(total) + (size_t)(col0 / 4) * ROWS + row;
  const int n_dst = l.ranks - 1 - l.me;
#pragma unroll 4
  for (int q = 0; q < N / 4; ++q) {
    if ((col0 / 4 + q) % parts != part) continue;
    const float4 t = __ldcg(src + (size_t)q * ROWS);
    for (int di = 0; di < n_dst; ++di) {
      if (!xl::reaches(sn, di)) break;   // farther ranks are out of reach too
      uint2* out = l.dst_slots[l.me + 1 + di] + xl::slot_offset(step & 1, l.ranks, l.me, elems) + seq_off;
      st_volatile_v4(out + link_word<ROWS>(col0 / 4 + q, row, 0),
                     make_uint4(__float_as_uint(t.x), step, __float_as_uint(t.y), step));
      st_volatile_v4(out + link_word<ROWS>(col0 / 4 + q, row, 1),
                     make_uint4(__float_as_uint(t.z), step, __float_as_uint(t.w), step));
    }
  }
}

// The whole of this thread's part of the total, dec * P + own, straight from registers to the NEXT rank
// only (for sequences whose state reaches no farther: nothing to share out, no detour through memory).
template <int N, int ROWS>
__device__ __forceinline__ void link_send_next(const Link& l, uint32_t step, long long elems, size_t seq_off, int row,
                                               int col0, float dec, const float (&P)[N], const float* own) {
  const float4* src = reinterpret_cast<const float4*>(own) + (size_t)(col0 / 4) * ROWS + row;
  uint2* out = l.dst_slots[l.me + 1] + xl::slot_offset(step & 1, l.ranks, l.me, elems) + seq_off;
#pragma unroll 4
  for (int q = 0; q < N / 4; ++q) {
    const float4 o = __ldcg(src + (size_t)q * ROWS);
    const float4 t = make_float4(fmaf(dec, P[4 * q], o.x), fmaf(dec, P[4 * q + 1], o.y), fmaf(dec, P[4 * q + 2], o.z),
                                 fmaf(dec, P[4 * q + 3], o.w));
    st_volatile_v4(out + link_word<ROWS>(col0 / 4 + q, row, 0),
                   make_uint4(__float_as_uint(t.x), step, __float_as_uint(t.y), step));
    st_volatile_v4(out + link_word<ROWS>(col0 / 4 + q, row, 1),
                   make_uint4(__float_as_uint(t.z), step, __float_as_uint(t.w), step));
  }
}

// P += dec * sum over the ranks before this one of exp(-sn)^(hops) * their total of this sequence, each word
// awaited until it carries `step`.  Returns false when a wait ran out (P is then NaN).
template <int N, int ROWS>
__device__ __forceinline__ bool link_receive(const Link& l, uint32_t step, long long elems, size_t seq_off, int row,
                                             int col0, float dec, float (&P)[N], float sn) {
  bool late = false;
  for (int src = l.me - 1; src >= 0; --src) {
    const int hops = l.me - 1 - src;
    if (!xl::reaches(sn, hops)) break;   // farther ranks are out of reach too
    const float wgt = dec * expf(-sn * (float)hops);
    const uint2* in = l.my_slots + xl::slot_offset(step & 1, l.ranks, src, elems) + seq_off;
    // wait with pauses on this thread's last word before touching the rest: thousands of threads
    // re-reading all their words would only get in the way of the stores that are arriving
    {
      const uint2* p = in + link_word<ROWS>(col0 / 4 + N / 4 - 1, row, 1);
      const long long t0 = clock64();
      while (!late && ld_volatile_v4(p).w != step) {
        __nanosleep(100);
        if (clock64() - t0 > l.wait_clocks) late = true;
      }
    }
    constexpr int kBatch = 4;   // float4 chunks in flight
#pragma unroll
    for (int q0 = 0; q0 < N / 4; q0 += kBatch) {
      uint4 w0[kBatch], w1[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        w0[u] = ld_volatile_v4(in + link_word<ROWS>(col0 / 4 + q0 + u, row, 0));
        w1[u] = ld_volatile_v4(in + link_word<ROWS>(col0 / 4 + q0 + u, row, 1));
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (!late && (w0[u].y != step || w0[u].w != step || w1[u].y != step || w1[u].w != step)) {
          const long long t0 = clock64();   // after one wait has run out this thread waits no more
          do {
            w0[u] = ld_volatile_v4(in + link_word<ROWS>(col0 / 4 + q0 + u, row, 0));
            w1[u] = ld_volatile_v4(in + link_word<ROWS>(col0 / 4 + q0 + u, row, 1));
            if (clock64() - t0 > l.wait_clocks) {
              late = true;
              break;
            }
          } while (w0[u].y != step || w0[u].w != step || w1[u].y != step || w1[u].w != step);
        }
        const int j = 4 * (q0 + u);
        P[j] = fmaf(wgt, __uint_as_float(w0[u].x), P[j]);
        P[j + 1] = fmaf(wgt, __uint_as_float(w0[u].z), P[j + 1]);
        P[j + 2] = fmaf(wgt, __uint_as_float(w1[u].x), P[j + 2]);
        P[j + 3] = fmaf(wgt, __uint_as_float(w1[u].z), P[j + 3]);
      }
    }
  }
  if (late) {   // a state that did not arrive must not look like one that did
#pragma unroll
    for (int j = 0; j < N; ++j) P[j] = __int_as_float(0x7fc00000);
  }
  return !late;
}

// spins until *flag >= want (as a step number) or `limit` clocks pass
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, long long limit) {
  if ((int32_t)(ld_volatile_u32(flag) - want) >= 0) return true;
  const long long t0 = clock64();
  while ((int32_t)(ld_volatile_u32(flag) - want) < 0) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}

struct WalkArgs {
  const float* s;
  const float* p0;     // not fused: fp32 state of every span at its border, [items][D][E] (from the scan)
  float* p0_save;      // fused: where the border states are kept for the backward pass (may be NULL)
  float* totals;       // fused: span totals [items][D][E], exchanged between the CTAs of the launch
  uint32_t* sync;      // fused: [0] launch counter, [1] CTAs done, [kSyncFlags + item] "total written" flags,
                       // [kSyncFlags + kSyncSecondBank + sequence] "sequence total written" flags (4 KB in all)
  const float* x_in;   // fused: incoming rank state (b,h,d,e) or NULL
  float* x_out;        // fused: outgoing rank state (b,h,d,e) or NULL
  int h, n, tiles, span, nspans, items;
  float qk_scale;      // q and k enter as qk_scale * map(q), qk_scale * map(k)
  int elu;             // map = elu(x) + 1 (otherwise the identity)
  const void* raw;     // backward with a map or a scale: the raw q (dQ walk) or k (dK/dV walk) for the chain rule
  int raw_pitch;       // ... and its row pitch in elements
  int even;            // the tiles of a sequence are shared out evenly among its spans (see TileWalk); a fused
                       // forward records it in sync[kSyncEven], the dQ walk reads it from the forward's workspace
  const uint32_t* even_word;   // dQ: where the forward pass recorded how it cut the sequences (NULL: a.even)
  int all_totals;      // fused: the last span of a sequence computes its total too
  int coop;            // fused: every CTA has exactly one span and the CTAs synchronise (several spans per
                       // sequence, or a link)
  long long wait_clocks;
  int32_t* fault;
  Link link;           // fused: hand the rank state over inside the launch (link.ranks > 0)
};
constexpr int kSyncEven = 2;
constexpr int kSyncFlags = 32;
constexpr int kSyncSecondBank = 480;   // [kSyncFlags + kSyncSecondBank + sequence]: "the sequence's total is written"

// bf16 image of this thread's part of the state (row `row`, columns [col0, col0 + N)) in the operand tile
template <int N>
__device__ __forceinline__ void write_state_operand(uint8_t* tile, int rows, int row, int col0, const float (&P)[N]) {
#pragma unroll
  for (int j = 0; j < N; j += 8)
    *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + j, rows)) =
        make_uint4(pack_bf16(P[j], P[j + 1]), pack_bf16(P[j + 2], P[j + 3]), pack_bf16(P[j + 4], P[j + 5]),
                   pack_bf16(P[j + 6], P[j + 7]));
}

// ---------------------------------------------------------------------------
// walk, first to last tile:  OUT = (X Y^T . M) Z + diag(lambda^r) X op(P);  P <- lambda^C P + K^T diag(w) V
//
//   DQ = false: X,Y = Q,K (width D), Z,OUT = V,O (width E), op(P) = P
//   DQ = true : X,Y = dO,V (width E), Z,OUT = K,dQ (width D), op(P) = P^T
// P is the d x e state in both: fp32 in the registers of the eight worker warps (thread = one row and
// half of the columns) and bf16 in shared memory as the operand of X op(P).
//
// Shared memory: X, Y, Z double buffered and the state operand, seven 32 KB buffers.  A buffer's life
// inside a tile:  X: tile -> free after S and O2
//                 Y: tile -> (after S) rows scaled in place -> free after L -> staging tile of OUT
//                 Z: tile -> free after L and O1
// Tensor memory: S (two buffers; the masked scores are packed to bf16 over S itself and feed O1 as its A
// operand from tensor memory), O (X op(P), rows scaled by lambda^r in place, += S_m Z), L = the state update.
//   warp 0 (one lane)  producer: loads, and the TMA stores of the finished staging tiles
//   warp 1 (one lane)  tensor-core issuer
//   warps 2-9          mask, row scaling, state update, epilogue
//
// FUSED = false: the state of every span at its border comes from the scan (a.p0).
// FUSED = true : one launch does everything.  With more than one span per sequence every CTA has
//   exactly one span (a cooperative launch, all CTAs resident).  It first sums its own span,
//   T = sum_c lambda^(span end - c) k_c v_c^T, streaming K and V once through the Y and Z buffers, writes
//   T to global memory and raises a flag; then it adds up the totals of the spans before it (and the
//   incoming rank state) with their decays - that is its border state - and walks.  The K and V tiles
//   are read again by the walk (they are in L2 by then).  The last span of a sequence needs no total
//   unless a.all_totals; the outgoing rank state is the state after the last tile of the last span.
// ---------------------------------------------------------------------------
template <int D, int E, bool DQ, bool FUSED, bool PRE, bool LINK>
__global__ void __launch_bounds__(320, 1) k_walk_out(const __grid_constant__ CUtensorMap map_x,
                                                     const __grid_constant__ CUtensorMap map_y,
                                                     const __grid_constant__ CUtensorMap map_z,
                                                     const __grid_constant__ CUtensorMap map_out,
                                                     const __grid_constant__ WalkArgs a) {
  static_assert(!(DQ && FUSED), "dQ walks over states the forward pass kept");
  if (threadIdx.x == 0) GTRACE(56);
  constexpr int WX = DQ ? E : D;  // width of X and Y
  constexpr int WZ = DQ ? D : E;  // width of Z and OUT
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const BufPair sx{smem};
  const BufPair sy{smem + 2 * kBuf};
  const BufPair sz{smem + 4 * kBuf};
  uint8_t* sp = smem + 6 * kBuf;
  __shared__ uint64_t x_full[2], y_full[2], z_full[2], s_full[2], sm_ready[2], o_full[2], o2_full[2], staged[2];
  __shared__ uint64_t p_ready, l_free, o_free, ys_ready, o2s_ready, l_full;
  __shared__ uint64_t mapped[2];   // with a feature map: the workers have mapped the tile's X, Y (dQ: Z) in place
  __shared__ uint64_t ring_full[2], ring_scaled[2], ring_empty[2], sum_done;   // the span-total phase
  __shared__ uint32_t tmem_slot, step_s, step_x, even_s;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int32_t* fault = a.fault;
  // Thread 0 is also the producer: it asks for its first tiles before the CTA-wide barrier below, so that their
  // flight overlaps the rest of the set-up (what it issued is remembered in early_*; only its copy matters).
  bool early_ring = false;
  int early_x = 0;
  if (tid == 0) {
    dead = 0;
    // the words this launch reads from global memory, all in flight while the barriers are set up
    const uint32_t ev = a.even_word != nullptr ? ld_volatile_u32(a.even_word) : (uint32_t)a.even;
    uint32_t ss = 0, sx_ = 0;
    if constexpr (FUSED) {
      if (a.coop) ss = ld_volatile_u32(a.sync);
      if (LINK && a.link.ranks > 0) sx_ = ld_volatile_u32(a.link.counters);
    }
    for (int p = 0; p < 2; ++p) {
      mbar_init(&x_full[p], 1);
      mbar_init(&y_full[p], 1);
      mbar_init(&z_full[p], 1);
      mbar_init(&s_full[p], 1);
      mbar_init(&sm_ready[p], kWorkers);
      mbar_init(&o_full[p], 1);
      mbar_init(&o2_full[p], 1);
      mbar_init(&staged[p], kWorkers);
      mbar_init(&mapped[p], kWorkers);
      mbar_init(&ring_full[p], 1);
      mbar_init(&ring_scaled[p], kWorkers);
      mbar_init(&ring_empty[p], 1);
    }
    mbar_init(&p_ready, kWorkers);
    mbar_init(&l_free, kWorkers);
    mbar_init(&o_free, kWorkers);
    mbar_init(&ys_ready, kWorkers);
    mbar_init(&o2s_ready, kWorkers);
    mbar_init(&l_full, 1);
    mbar_init(&sum_done, 1);
    fence_mbar_init();
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_y);
    prefetch_tensormap(&map_z);
    prefetch_tensormap(&map_out);
    even_s = ev;
    if constexpr (FUSED) {
      step_s = a.coop ? ss + 1 : 0;                              // this launch among those on the workspace
      step_x = LINK && a.link.ranks > 0 ? sx_ + 1 : 0;           // this hand-over in the group
    }
    TileWalk w0{a.items, a.nspans, a.span, a.tiles, 0, false, ev != 0};
    if (w0.start(blockIdx.x, gridDim.x)) {
      const int sp0 = w0.it - w0.bh * a.nspans;
      if (FUSED && a.coop && (sp0 < a.nspans - 1 || a.all_totals)) {   // first stage of the span-total ring
        mbar_expect_tx(&ring_full[0], C * (WX + WZ) * 2);
        tma_load_4d(smem + 2 * kBuf, &map_y, &ring_full[0], 0, w0.t0 * C, 0, w0.bh);
        tma_load_4d(smem + 4 * kBuf, &map_z, &ring_full[0], 0, w0.t0 * C, 0, w0.bh);
        early_ring = true;
      } else {                                                          // X of the first tile of the walk
        mbar_expect_tx(&x_full[0], C * WX * 2);
        tma_load_4d(smem, &map_x, &x_full[0], 0, w0.t * C, 0, w0.bh);
        early_x = 1;
      }
    }
  }
  if (warp == 2) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (tid == 64) TRACE(0);
  if (tid == 64) GTRACE(57);
  const TmemPair t_s{tmem};
  const uint32_t t_o = tmem + 256, t_l = tmem + 384;
  TileWalk w{a.items, a.nspans, a.span, a.tiles, 0, false, even_s != 0};
  // the span-total phase: only with several spans per sequence, and then this CTA has one span
  bool sums = false;
  int sum_t0 = 0, sum_t1 = 0, my_bh = 0, my_sp = 0;
  if constexpr (FUSED) {
    if (a.coop && w.start(blockIdx.x, gridDim.x)) {
      my_bh = w.bh;
      my_sp = w.it - w.bh * a.nspans;
      sum_t0 = w.t0;
      sum_t1 = w.t1;
      sums = my_sp < a.nspans - 1 || a.all_totals;
    }
  }

  if (warp == 0) {
    if (lane == 0) {
      int x_issued = early_x;
      if (sums) {
        for (int t = sum_t0, g = 0; t < sum_t1; ++t, ++g) {
          const int j = g & 1;
          if (g >= 2) wait_or_fault(&ring_empty[j], ((g >> 1) - 1) & 1, &dead, fault, kFaultMmaWait);
          if (!(g == 0 && early_ring)) {
            mbar_expect_tx(&ring_full[j], C * (WX + WZ) * 2);
            tma_load_4d(sy[j], &map_y, &ring_full[j], 0, t * C, 0, my_bh);
            tma_load_4d(sz[j], &map_z, &ring_full[j], 0, t * C, 0, my_bh);
          }
          if (g == 1 || t == sum_t1 - 1) {
            // X of the first two tiles of the walk can come in during the sums - behind the first ring
            // stages, which every CTA of the launch asks for at the same moment and the sums wait for
            for (bool ok = x_issued == 0 && w.start(blockIdx.x, gridDim.x); ok && x_issued < 2; ok = w.next(), ++x_issued) {
              mbar_expect_tx(&x_full[x_issued], C * WX * 2);
              tma_load_4d(sx[x_issued], &map_x, &x_full[x_issued], 0, w.t * C, 0, w.bh);
            }
          }
        }
        wait_or_fault(&sum_done, 0, &dead, fault, kFaultMmaWait);   // the MMAs have read every ring stage
      }
      int i = 0;
      IntPair out_row{0, 0}, out_bh{0, 0};
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++i) {
        const int p = i & 1, u = i >> 1;
        if (i >= x_issued) {
          if (i >= 2) wait_or_fault(&o2_full[p], (u - 1) & 1, &dead, fault, kFaultMmaWait);  // S, O2 of tile i-2 read X
          mbar_expect_tx(&x_full[p], C * WX * 2);
          tma_load_4d(sx[p], &map_x, &x_full[p], 0, w.t * C, 0, w.bh);
        }
        if (i >= 2) wait_or_fault(&o_full[p], (u - 1) & 1, &dead, fault, kFaultMmaWait);     // L, O1 of tile i-2 read Z
        mbar_expect_tx(&z_full[p], C * WZ * 2);
        tma_load_4d(sz[p], &map_z, &z_full[p], 0, w.t * C, 0, w.bh);
        if (i >= 2) {
          // the output of tile i-2 is staged in Y's buffer: store it, then reuse the buffer
          wait_or_fault(&staged[p], (u - 1) & 1, &dead, fault, kFaultMmaWait);
          tma_store_4d(&map_out, sy[p], 0, out_row.get(p), 0, out_bh.get(p));
          bulk_commit();
          bulk_wait_read<0>();
        }
        mbar_expect_tx(&y_full[p], C * WX * 2);
        tma_load_4d(sy[p], &map_y, &y_full[p], 0, w.t * C, 0, w.bh);
        out_row.set(p, w.t * C);
        out_bh.set(p, w.bh);
      }
      for (int j = (i >= 2 ? i - 2 : 0); j < i; ++j) {   // the last two tiles
        const int p = j & 1, u = j >> 1;
        wait_or_fault(&staged[p], u & 1, &dead, fault, kFaultMmaWait);
        tma_store_4d(&map_out, sy[p], 0, out_row.get(p), 0, out_bh.get(p));
        bulk_commit();
      }
      bulk_wait_all<0>();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      if (sums) {
        for (int t = sum_t0, g = 0; t < sum_t1; ++t, ++g) {
          const int j = g & 1;
          wait_or_fault(&ring_scaled[j], (g >> 1) & 1, &dead, fault, kFaultTmaWait);
          tc_fence_after_sync();
          umma_gemm(t_l, Operand{smem_u32(sy[j]), C, true}, Operand{smem_u32(sz[j]), C, true}, E, C / 16, g > 0);
          umma_commit(&ring_empty[j]);
        }
        umma_commit(&sum_done);
      }
      int total = 0;
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next()) ++total;
      // Per tile: O2 = X op(P) as soon as the state operand exists; L once Y's rows are scaled; O1 = S_m Z
      // (S_m read from tensor memory) on top of the row-scaled O2 once both are ready; and S of the next
      // tile whenever its inputs are there, so that the next tile's mask never waits.
      auto issue_s = [&](int j) {
        const int q = j & 1;
        tc_fence_after_sync();
        umma_gemm(t_s[q], Operand{smem_u32(sx[q]), C, false}, Operand{smem_u32(sy[q]), C, false}, C, WX / 16, false);
        umma_commit(&s_full[q]);
      };
      const bool map_xy = PRE && a.elu && !DQ, map_z = PRE && a.elu && DQ;
      if (total > 0) {
        wait_or_fault(&x_full[0], 0, &dead, fault, kFaultTmaWait);
        wait_or_fault(&y_full[0], 0, &dead, fault, kFaultTmaWait);
        if (map_xy) wait_or_fault(&mapped[0], 0, &dead, fault, kFaultMmaWait);
        issue_s(0);
      }
      for (int i = 0; i < total; ++i) {
        const int p = i & 1, ph = (i >> 1) & 1, one = i & 1;
        const int q = (i + 1) & 1, uq = (i + 1) >> 1;
        // the four products of the tile go out as their inputs become ready, in whatever order that is
        bool need_o2 = true, need_l = true, need_o1 = true, need_s = i + 1 < total;
        const long long t0 = clock64();
        while ((need_o2 || need_l || need_o1 || need_s) && !dead) {
          // O1 = S_m Z on top of the row-scaled O2, the masked scores read from tensor memory.  It goes out
          // after L: the commit behind it then also covers L's reads of Y and Z, which is what frees them
          if (need_o1 && !need_o2 && !need_l && mbar_test_wait(&sm_ready[p], ph) && mbar_test_wait(&o2s_ready, one) &&
              mbar_test_wait(&z_full[p], ph) && (!map_z || mbar_test_wait(&mapped[p], ph))) {
            TRACE(32 + i * 5 + 3);
            tc_fence_after_sync();
            umma_gemm_ts(t_o, t_s[p], true, Operand{smem_u32(sz[p]), C, true}, WZ, true);
            umma_commit(&o_full[p]);
            need_o1 = false;
            continue;
          }
          // L = K^T diag(w) V (d x e), the scaled rows being Y's; the state update has read the previous L
          if (need_l && mbar_test_wait(&ys_ready, one) && mbar_test_wait(&z_full[p], ph) &&
              (!map_z || mbar_test_wait(&mapped[p], ph)) && (i < 1 || mbar_test_wait(&l_free, one ^ 1))) {
            TRACE(32 + i * 5 + 1);
            tc_fence_after_sync();
            if constexpr (!DQ)
              umma_gemm(t_l, Operand{smem_u32(sy[p]), C, true}, Operand{smem_u32(sz[p]), C, true}, E, C / 16, false);
            else
              umma_gemm(t_l, Operand{smem_u32(sz[p]), C, true}, Operand{smem_u32(sy[p]), C, true}, E, C / 16, false);
            umma_commit(&l_full);
            need_l = false;
            continue;
          }
          // O2 = X op(P): the state operand of this tile is written, the epilogue has drained O
          if (need_o2 && mbar_test_wait(&p_ready, one) && (i < 1 || mbar_test_wait(&o_free, one ^ 1))) {
            TRACE(32 + i * 5 + 0);
            tc_fence_after_sync();
            if constexpr (!DQ)  // X P: the state tile as [K = d rows] x [N = e columns]
              umma_gemm(t_o, Operand{smem_u32(sx[p]), C, false}, Operand{smem_u32(sp), D, true}, E, D / 16, false);
            else                // X P^T: the state tile as [N = d rows] x [K = e columns]
              umma_gemm(t_o, Operand{smem_u32(sx[p]), C, false}, Operand{smem_u32(sp), D, false}, D, E / 16, false);
            umma_commit(&o2_full[p]);
            need_o2 = false;
            continue;
          }
          // S of the next tile; S[q] held the masked scores of tile i-1: its O1 must have read them
          if (need_s && mbar_test_wait(&x_full[q], uq & 1) && mbar_test_wait(&y_full[q], uq & 1) &&
              (!map_xy || mbar_test_wait(&mapped[q], uq & 1)) && (i + 1 < 2 || mbar_test_wait(&o_full[q], (uq - 1) & 1))) {
            TRACE(32 + i * 5 + 2);
            issue_s(i + 1);
            need_s = false;
            continue;
          }
          if (clock64() - t0 > kWaitClocks) {
            dead = 1;
            atomicOr(fault, kFaultMmaWait);
          }
        }
      }
    }
  } else {
    const int cw = warp - 2;                     // 0..7
    const int row = (warp & 3) * 32 + lane;      // tensor-memory lane quarter of this warp
    const int half = cw >> 2;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    constexpr int kHalfE = E / 2;
    float P[kHalfE];  // this thread's part of the state: row `row`, columns [half * E/2, (half+1) * E/2)
    float sl2 = 0.f, lam = 1.f;
    // q and k enter as c * map(q), c * map(k): the map is applied to the tiles in shared memory, c is folded
    // into factors that exist anyway (dQ: the state already carries k's c)
    // (PRE = false: instantiations without any of this, for callers who bring q and k as they are)
    const float c = PRE ? a.qk_scale : 1.f;
    const float c_mask = DQ ? c : c * c, c_o2 = DQ ? 1.f : c;
    const bool elu = PRE && a.elu != 0;
    // brings tile j (buffers of parity j & 1) through the feature map once its loads have landed
    auto map_tile = [&](int j) {
      const int q = j & 1, uq = (j >> 1) & 1;
      if constexpr (!DQ) {
        wait_or_fault(&x_full[q], uq, &dead, fault, kFaultTmaWait);
        wait_or_fault(&y_full[q], uq, &dead, fault, kFaultTmaWait);
        scale_row_pieces<WX / 16, true>(sx[q], row, half * (WX / 16), 1.f, lane);
        scale_row_pieces<WX / 16, true>(sy[q], row, half * (WX / 16), 1.f, lane);
      } else {
        wait_or_fault(&z_full[q], uq, &dead, fault, kFaultTmaWait);
        scale_row_pieces<WZ / 16, true>(sz[q], row, half * (WZ / 16), 1.f, lane);
      }
      fence_async_smem();
      mbar_arrive(&mapped[q]);
    };
    if (sums) {
      // ---- this span's total, written where the CTAs of the later spans find it
      sl2 = a.s[my_bh % a.h] * kLog2e;
      const int span_end = min(sum_t1 * C, a.n);
      for (int t = sum_t0, g = 0; t < sum_t1; ++t, ++g) {
        const int j = g & 1;
        wait_or_fault(&ring_full[j], (g >> 1) & 1, &dead, fault, kFaultTmaWait);
        const float wt = c * decay_pow(sl2, max(span_end - (t * C + row), 0));
        if (elu)
          scale_row_pieces<WX / 16, true>(sy[j], row, half * (WX / 16), wt, lane);
        else
          scale_row_pieces<WX / 16>(sy[j], row, half * (WX / 16), wt, lane);
        fence_async_smem();
        mbar_arrive(&ring_scaled[j]);
      }
      wait_or_fault(&sum_done, 0, &dead, fault, kFaultMmaWait);
      if (tid == 64) TRACE(59);
      tc_fence_after_sync();
      if (row < D) {
#pragma unroll
        for (int c0 = 0; c0 < kHalfE; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_l + lane_base + half * kHalfE + c0, r);
          tmem_ld_wait();
          store_state32<D>(a.totals + (size_t)blockIdx.x * D * E, row, half * kHalfE + c0, r);
        }
      }
      tc_fence_before_sync();
      named_sync(1, kWorkers);   // every worker's part of the total is written ...
      if (tid == 64) {
        __threadfence();         // ... and visible to the other CTAs before the flag is
        st_volatile_u32(a.sync + kSyncFlags + blockIdx.x, step_s);
      }
      if (tid == 64) TRACE(60);
    }
    int total = 0;
    if (elu) {
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next()) ++total;
      if (total > 0) map_tile(0);
    }
    int i = 0;
    for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++i) {
      const int p = i & 1, ph = (i >> 1) & 1, one = i & 1;
      const int len = min(C, a.n - w.t * C);     // tokens really in the tile
      if (w.first_of_item()) {
        sl2 = a.s[w.bh % a.h] * kLog2e;
        lam = exp2f(-sl2);
      }
      if (tid == 64) TRACE(1 + i * 6 + 0);
      wait_or_fault(&s_full[p], ph, &dead, fault, kFaultMmaWait);
      wait_or_fault(&y_full[p], ph, &dead, fault, kFaultTmaWait);  // completed long ago: makes Y's bytes visible here
      if (tid == 64) TRACE(1 + i * 6 + 1);
      tc_fence_after_sync();
      // state chain first: scale Y's rows so that L can run under the mask
      scale_row_pieces<WX / 16>(sy[p], row, half * (WX / 16), c * decay_pow(sl2, max(len - row, 0)), lane);
      fence_async_smem();
      mbar_arrive(&ys_ready);
      if (tid == 64) TRACE(1 + i * 6 + 2);
      // masked scores, packed to bf16 in place: they are the A operand of O1 straight from tensor memory
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t packed[16];
        masked_pack32<false>(t_s[p] + lane_base + half * 64 + cc * 32, row, half * 64 + cc * 32, sl2, lam, packed, c_mask);
        tmem_st16(t_s[p] + lane_base + half * 64 + cc * 16, packed);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&sm_ready[p]);
      if (tid == 64) TRACE(1 + i * 6 + 3);
      if (elu && i + 1 < total) map_tile(i + 1);   // the next tile's S can then go out under this tile's work
      if (__builtin_expect(w.first_of_item(), 0)) {   // once per span: kept out of the tiles' straight-line code
        // the state at the span border (the score work above does not need it, so the wait for the other
        // CTAs' totals hides behind it); the O2 MMA that read the operand tile of the previous item has completed
        if constexpr (!FUSED) {
          if (row < D) load_state<kHalfE, D, false>(a.p0 + (size_t)w.it * D * E, row, half * kHalfE, P);
        } else {
          const int sp_idx = w.it - w.bh * a.nspans;
          const size_t mine = (size_t)row * E + half * kHalfE;
          // incoming rank state, decayed from the first token of the sequence to the first of the span
          if (a.x_in != nullptr && row < D) {
            const float dec = decay_pow(sl2, w.t0 * C);
            const float4* src = reinterpret_cast<const float4*>(a.x_in + (size_t)w.bh * D * E + mine);
#pragma unroll
            for (int j = 0; j < kHalfE / 4; ++j) {
              const float4 v = src[j];
              P[4 * j] = dec * v.x, P[4 * j + 1] = dec * v.y, P[4 * j + 2] = dec * v.z, P[4 * j + 3] = dec * v.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < kHalfE; ++j) P[j] = 0.f;
          }
          // totals of the spans before this one (each decayed to its own end); one thread per flag
          if (tid - 64 < sp_idx && !dead) {
            if (!wait_flag_eq(a.sync + kSyncFlags + w.bh * a.nspans + (tid - 64), step_s, a.wait_clocks)) {
              dead = 1;
              atomicOr(fault, kFaultFlagWait);
            }
          }
          named_sync(1, kWorkers);
          for (int j = 0; j < sp_idx; ++j) {   // each total is decayed to the end of its span
            if (row < D)
              fma_state<kHalfE, D>(a.totals + (size_t)(w.bh * a.nspans + j) * D * E, row, half * kHalfE,
                                   decay_pow(sl2, (w.t0 - w.span_t0(j + 1)) * C), P);
          }
          if (tid == 64) TRACE(61);
          if (LINK && a.link.ranks > 0) {
            // hand-over of the rank state inside the launch.  P holds the local part of the border state.
            const float sn = a.s[w.bh % a.h] * (float)a.n;
            const long long elems = (long long)(a.items / a.nspans) * D * E;
            const size_t seq_off = (size_t)w.bh * D * E;
            const int n_dst = a.link.ranks - 1 - a.link.me;
            if (n_dst > 0) {
              const int owner = w.bh * a.nspans + a.nspans - 1;   // the CTA that owns the end of the sequence
              const bool far = n_dst > 1 && xl::reaches(sn, 1);   // the state reaches beyond the next rank
              uint32_t* ready = a.sync + kSyncFlags + kSyncSecondBank + w.bh;
              if (w.it == owner && far) {
                // the sequence's total, lambda^(n - start) P + T, where the other CTAs of the sequence find it
                if (row < D)
                  link_make_total<kHalfE, D>(a.totals + (size_t)owner * D * E, row, half * kHalfE,
                                             decay_pow(sl2, a.n - w.t0 * C), P);
                named_sync(1, kWorkers);
                if (tid == 64) {
                  __threadfence();
                  st_volatile_u32(ready, step_s);
                }
              }
              if (far || w.it == owner) {
                // the readers of the ranks after this one have acknowledged the slots' previous use
                if (!dead) {
                  bool ok = true;
                  if (xl::needs_ack_wait(step_x) && tid - 64 < n_dst)
                    ok = wait_flag_ge(a.link.my_acks + xl::ack_index(a.link.me + 1 + (tid - 64), 0), step_x - 2,
                                      a.link.wait_clocks);
                  if (far && tid == 64 + xl::kMaxRanks && w.it != owner) ok = wait_flag_eq(ready, step_s, a.wait_clocks);
                  if (!ok) {
                    dead = 1;
                    atomicOr(fault, kFaultRelayWait);
                  }
                }
                named_sync(1, kWorkers);
                if (row < D) {
                  if (far)   // several destinations: every CTA of the sequence sends its share
                    link_send_part<kHalfE, D>(a.link, step_x, elems, seq_off, row, half * kHalfE,
                                              a.totals + (size_t)owner * D * E, sn, sp_idx, a.nspans);
                  else       // the next rank only: straight from the owner's registers
                    link_send_next<kHalfE, D>(a.link, step_x, elems, seq_off, row, half * kHalfE,
                                              decay_pow(sl2, a.n - w.t0 * C), P, a.totals + (size_t)owner * D * E);
                }
              }
            }
            if (tid == 64) TRACE(62);
            if (a.link.me > 0 && row < D) {
              // what the ranks before this one sent, decayed from the first token of the sequence to the span
              if (!link_receive<kHalfE, D>(a.link, step_x, elems, seq_off, row, half * kHalfE,
                                           decay_pow(sl2, w.t0 * C), P, sn))
                atomicOr(fault, kFaultRelayWait);
            }
            if (tid == 64) TRACE(55);
          }
        }
        if (row < D) write_state_operand<kHalfE>(sp, D, row, half * kHalfE, P);
        fence_async_smem();
        mbar_arrive(&p_ready);
        if constexpr (FUSED) {   // kept for the backward pass
          if (a.p0_save != nullptr && row < D) store_state<kHalfE, D>(a.p0_save + (size_t)w.it * D * E, row, half * kHalfE, P);
        }
      }
      // O2's rows take their decay lambda^row in tensor memory; O1 then accumulates on top
      wait_or_fault(&o2_full[p], ph, &dead, fault, kFaultMmaWait);
      tc_fence_after_sync();
      {
        const float qd = c_o2 * decay_pow(sl2, row);
#pragma unroll 1
        for (int cc = 0; cc < WZ / 64; ++cc) scale_tmem32(t_o + lane_base + half * (WZ / 2) + cc * 32, qd);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&o2s_ready);
      // state: P <- lambda^len P + L
      wait_or_fault(&l_full, one, &dead, fault, kFaultMmaWait);
      tc_fence_after_sync();
      if (row < D) {
        const float lam_c = decay_pow(sl2, len);
#pragma unroll
        for (int c0 = 0; c0 < kHalfE; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_l + lane_base + half * kHalfE + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) P[c0 + j] = fmaf(lam_c, P[c0 + j], __uint_as_float(r[j]));
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&l_free);
      if (!w.last_of_item()) {
        if (row < D) write_state_operand<kHalfE>(sp, D, row, half * kHalfE, P);
        fence_async_smem();
        mbar_arrive(&p_ready);
      } else if constexpr (FUSED) {
        // the state after the last tile of the sequence is the outgoing rank state
        if (a.x_out != nullptr && w.t == a.tiles - 1 && row < D) {
          float4* dst = reinterpret_cast<float4*>(a.x_out + (size_t)w.bh * D * E + (size_t)row * E + half * kHalfE);
#pragma unroll
          for (int q = 0; q < kHalfE / 4; ++q) dst[q] = make_float4(P[4 * q], P[4 * q + 1], P[4 * q + 2], P[4 * q + 3]);
        }
      }
      if (tid == 64) TRACE(1 + i * 6 + 4);
      // epilogue: OUT staged in Y's buffer (the L MMA has read the scaled rows)
      wait_or_fault(&o_full[p], ph, &dead, fault, kFaultMmaWait);
      tc_fence_after_sync();
      if (DQ && (elu || c != 1.f)) {
        // dq = dq' * c * map'(q), q read from the raw tensor (rows past the end of the sequence are not stored)
        const bool live = row < len;
        const __nv_bfloat16* raw =
            static_cast<const __nv_bfloat16*>(a.raw) + ((size_t)w.bh * a.n + (size_t)w.t * C + (live ? row : 0)) * a.raw_pitch;
#pragma unroll 1
        for (int cc = 0; cc < WZ / 64; ++cc) {
          const int col0 = half * (WZ / 2) + cc * 32;
          stage_row32_chain(t_o + lane_base + col0, sy[p], row, col0, raw, c, elu && live);
        }
      } else {
#pragma unroll 1
        for (int cc = 0; cc < WZ / 64; ++cc) {
          const int col0 = half * (WZ / 2) + cc * 32;
          stage_row32(t_o + lane_base + col0, kNoAcc, 0.f, sy[p], row, col0);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&o_free);
      fence_async_smem();
      mbar_arrive(&staged[p]);
      if (tid == 64) TRACE(1 + i * 6 + 5);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 64) TRACE(63);
  if (tid == 64) GTRACE(58);
  if (warp == 2) tmem_dealloc(tmem, 512);
  if constexpr (!DQ) {   // how this pass cut the sequences, for the dQ walk over the border states it leaves
    if (tid == 0 && blockIdx.x == 0 && a.sync != nullptr) st_volatile_u32(a.sync + kSyncEven, even_s);
  }
  if constexpr (FUSED) {
    // the last CTA to finish advances the launch counter: the flags of this launch are stale from then on;
    // with a link it also tells the ranks before this one that their words have been read (they may
    // overwrite them two hand-overs later) and completes the hand-over
    if (tid == 0 && a.coop) {
      __threadfence();
      if (atomicAdd(a.sync + 1, 1u) == gridDim.x - 1) {
        st_volatile_u32(a.sync + 1, 0u);
        __threadfence();
        st_volatile_u32(a.sync, step_s);
        if (LINK && a.link.ranks > 0) {
          for (int q = 0; q < a.link.me; ++q) st_volatile_u32(a.link.src_acks[q] + xl::ack_index(a.link.me, 0), step_x);
          st_volatile_u32(a.link.counters, step_x);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// walk, last to first tile, with the suffix state Dn (d x e) on chip:
//   dK = dS_m^T Q + diag(lambda^(len-c)) V Dn^T
//   dV = S_m^T dO + diag(lambda^(len-c)) K Dn
//   Dn <- lambda^len Dn + Q^T diag(lambda^r) dO          (len = tokens in the tile, 128 but for a ragged tail)
//
// Shared memory: Q, dO (single buffers), K, V (double buffered), the state operand: seven 32 KB buffers.
//   K : tile -> (after phase A) S_m  -> (after phase B) staging tile of dK
//   V : tile -> (after phase A) dS_m -> (after phase B) staging tile of dV
//   Dn: state operand -> (after phase A) row-scaled copy of Q for the state update -> new state operand
// Tensor memory, four 128-column regions:
//   T_S : S = Q K^T            -> (masked into shared memory) -> L = Q_s^T dO, the state update
//   T_dS: dS = dO V^T          -> (masked into shared memory)
//   T_dK: V Dn^T, rows scaled  -> += dS_m^T Q                  = dK
//   T_dV: K Dn, rows scaled    -> += S_m^T dO                  = dV
// Per tile the issuer runs phase A (four products), L as soon as the workers have copied Q and masked S,
// and phase B once dS is masked and the two state products are scaled; the workers update the state
// while phase B runs and then stage dK and dV for the TMA stores.
//
// FUSED: as in k_walk_out - the CTA first sums its span, T = sum_r lambda^(r - span start) q_r do_r^T,
// through the K and V buffers, publishes it, adds up the totals of the LATER spans of its sequence (and
// the incoming rank state) and walks; the outgoing rank state is the state after the first tile of the
// sequence.
// ---------------------------------------------------------------------------
template <int D, int E, bool FUSED, bool PRE, bool LINK>
__global__ void __launch_bounds__(320, 1) k_walk_dkv(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
    const __grid_constant__ WalkArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sq = smem;
  uint8_t* sdo = smem + kBuf;
  const BufPair sk{smem + 2 * kBuf};
  const BufPair sv{smem + 4 * kBuf};
  uint8_t* sdn = smem + 6 * kBuf;
  __shared__ uint64_t kv_full[2], staged[2];
  __shared__ uint64_t qdo_full, dn_ready, a_done, ms_ready, sm_ready, b_done, l_done, e_free, l_free;
  __shared__ uint64_t mapped;   // with a feature map: the workers have mapped the tile's Q and K in place
  __shared__ uint64_t ring_full[2], ring_scaled[2], ring_empty[2], sum_done;   // the span-total phase
  __shared__ uint32_t tmem_slot, step_s, step_x;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int32_t* fault = a.fault;
  // thread 0 is also the producer: its first loads go out before the CTA-wide barrier (see k_walk_out)
  bool early_ring = false, early_kv = false;
  if (tid == 0) {
    dead = 0;
    uint32_t ss = 0, sx_ = 0;   // in flight while the barriers are set up
    if constexpr (FUSED) {
      if (a.coop) ss = ld_volatile_u32(a.sync);
      if (LINK && a.link.ranks > 0) sx_ = ld_volatile_u32(a.link.counters);
    }
    for (int p = 0; p < 2; ++p) {
      mbar_init(&kv_full[p], 1);
      mbar_init(&staged[p], kWorkers);
      mbar_init(&ring_full[p], 1);
      mbar_init(&ring_scaled[p], kWorkers);
      mbar_init(&ring_empty[p], 1);
    }
    mbar_init(&qdo_full, 1);
    mbar_init(&mapped, kWorkers);
    mbar_init(&dn_ready, kWorkers);
    mbar_init(&a_done, 1);
    mbar_init(&ms_ready, kWorkers);
    mbar_init(&sm_ready, kWorkers);
    mbar_init(&b_done, 1);
    mbar_init(&l_done, 1);
    mbar_init(&e_free, kWorkers);
    mbar_init(&l_free, kWorkers);
    mbar_init(&sum_done, 1);
    fence_mbar_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    prefetch_tensormap(&map_do);
    prefetch_tensormap(&map_dk);
    prefetch_tensormap(&map_dv);
    if constexpr (FUSED) {
      step_s = a.coop ? ss + 1 : 0;                              // this launch among those on the workspace
      step_x = LINK && a.link.ranks > 0 ? sx_ + 1 : 0;           // this hand-over in the group
    }
    TileWalk w0{a.items, a.nspans, a.span, a.tiles, 0, true, a.even != 0};
    if (w0.start(blockIdx.x, gridDim.x)) {
      const int sp0 = w0.it - w0.bh * a.nspans;
      if (FUSED && a.coop && (sp0 > 0 || a.all_totals)) {   // first stage of the span-total ring: Q, dO
        mbar_expect_tx(&ring_full[0], C * (D + E) * 2);
        tma_load_4d(smem + 2 * kBuf, &map_q, &ring_full[0], 0, w0.t0 * C, 0, w0.bh);
        tma_load_4d(smem + 4 * kBuf, &map_do, &ring_full[0], 0, w0.t0 * C, 0, w0.bh);
        early_ring = true;
      } else {                                               // K, V of the first tile of the walk
        mbar_expect_tx(&kv_full[0], C * (D + E) * 2);
        tma_load_4d(smem + 2 * kBuf, &map_k, &kv_full[0], 0, w0.t * C, 0, w0.bh);
        tma_load_4d(smem + 4 * kBuf, &map_v, &kv_full[0], 0, w0.t * C, 0, w0.bh);
        early_kv = true;
      }
    }
  }
  if (warp == 2) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (tid == 64) TRACE(0);
  if (tid == 64) GTRACE(57);
  const uint32_t t_s = tmem, t_ds = tmem + 128, t_dk = tmem + 256, t_dv = tmem + 384;
  TileWalk w{a.items, a.nspans, a.span, a.tiles, 0, true, a.even != 0};
  bool sums = false;
  int sum_t0 = 0, sum_t1 = 0, my_bh = 0, my_sp = 0;
  if constexpr (FUSED) {
    if (a.coop && w.start(blockIdx.x, gridDim.x)) {
      my_bh = w.bh;
      my_sp = w.it - w.bh * a.nspans;
      sum_t0 = w.t0;
      sum_t1 = w.t1;
      sums = my_sp > 0 || a.all_totals;
    }
  }

  if (warp == 0) {
    if (lane == 0) {
      bool first_qdo_issued = false;
      if (sums) {
        for (int t = sum_t0, g = 0; t < sum_t1; ++t, ++g) {
          const int j = g & 1;
          if (g >= 2) wait_or_fault(&ring_empty[j], ((g >> 1) - 1) & 1, &dead, fault, kFaultMmaWait);
          if (!(g == 0 && early_ring)) {
            mbar_expect_tx(&ring_full[j], C * (D + E) * 2);
            tma_load_4d(sk[j], &map_q, &ring_full[j], 0, t * C, 0, my_bh);
            tma_load_4d(sv[j], &map_do, &ring_full[j], 0, t * C, 0, my_bh);
          }
          // Q, dO of the first tile of the walk can come in during the sums, behind the first ring stages
          if ((g == 1 || t == sum_t1 - 1) && !first_qdo_issued && w.start(blockIdx.x, gridDim.x)) {
            mbar_expect_tx(&qdo_full, C * (D + E) * 2);
            tma_load_4d(sq, &map_q, &qdo_full, 0, w.t * C, 0, w.bh);
            tma_load_4d(sdo, &map_do, &qdo_full, 0, w.t * C, 0, w.bh);
            first_qdo_issued = true;
          }
        }
        wait_or_fault(&sum_done, 0, &dead, fault, kFaultMmaWait);   // the MMAs have read every ring stage
      }
      int i = 0;
      IntPair out_row{0, 0}, out_bh{0, 0};
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++i) {
        const int p = i & 1, u = i >> 1;
        if (i >= 2) {
          // dK and dV of tile i-2 are staged in this parity's K and V buffers
          wait_or_fault(&staged[p], (u - 1) & 1, &dead, fault, kFaultMmaWait);
          tma_store_4d(&map_dk, sk[p], 0, out_row.get(p), 0, out_bh.get(p));
          tma_store_4d(&map_dv, sv[p], 0, out_row.get(p), 0, out_bh.get(p));
          bulk_commit();
          bulk_wait_read<0>();
        }
        if (!(i == 0 && early_kv)) {
          mbar_expect_tx(&kv_full[p], C * (D + E) * 2);
          tma_load_4d(sk[p], &map_k, &kv_full[p], 0, w.t * C, 0, w.bh);
          tma_load_4d(sv[p], &map_v, &kv_full[p], 0, w.t * C, 0, w.bh);
        }
        if (i >= 1) {   // Q, dO of tile i-1 are read: by phase B and by L
          wait_or_fault(&b_done, (i - 1) & 1, &dead, fault, kFaultMmaWait);
          wait_or_fault(&l_done, (i - 1) & 1, &dead, fault, kFaultMmaWait);
        }
        if (i >= 1 || !first_qdo_issued) {
          mbar_expect_tx(&qdo_full, C * (D + E) * 2);
          tma_load_4d(sq, &map_q, &qdo_full, 0, w.t * C, 0, w.bh);
          tma_load_4d(sdo, &map_do, &qdo_full, 0, w.t * C, 0, w.bh);
        }
        out_row.set(p, w.t * C);
        out_bh.set(p, w.bh);
      }
      for (int j = (i >= 2 ? i - 2 : 0); j < i; ++j) {   // the last two tiles
        const int p = j & 1, u = j >> 1;
        wait_or_fault(&staged[p], u & 1, &dead, fault, kFaultMmaWait);
        tma_store_4d(&map_dk, sk[p], 0, out_row.get(p), 0, out_bh.get(p));
        tma_store_4d(&map_dv, sv[p], 0, out_row.get(p), 0, out_bh.get(p));
        bulk_commit();
      }
      bulk_wait_all<0>();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      if (sums) {
        for (int t = sum_t0, g = 0; t < sum_t1; ++t, ++g) {
          const int j = g & 1;
          wait_or_fault(&ring_scaled[j], (g >> 1) & 1, &dead, fault, kFaultTmaWait);
          tc_fence_after_sync();
          umma_gemm(t_s, Operand{smem_u32(sk[j]), C, true}, Operand{smem_u32(sv[j]), C, true}, E, C / 16, g > 0);
          umma_commit(&ring_empty[j]);
        }
        umma_commit(&sum_done);
      }
      int i = 0;
      for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++i) {
        const int p = i & 1, ph = (i >> 1) & 1, one = i & 1;
        // phase A.  The state tile as [N = d rows] x [K = e columns] (V Dn^T) and as [K = d rows] x
        // [N = e columns] (K Dn); T_dK, T_dV were drained by the previous epilogue, T_S by the state update
        wait_or_fault(&kv_full[p], ph, &dead, fault, kFaultTmaWait);
        if (PRE && a.elu) wait_or_fault(&mapped, one, &dead, fault, kFaultMmaWait);
        wait_or_fault(&dn_ready, one, &dead, fault, kFaultMmaWait);
        if (i >= 1) {
          wait_or_fault(&e_free, one ^ 1, &dead, fault, kFaultMmaWait);
          wait_or_fault(&l_free, one ^ 1, &dead, fault, kFaultMmaWait);
        }
        tc_fence_after_sync();
        umma_gemm(t_dk, Operand{smem_u32(sv[p]), C, false}, Operand{smem_u32(sdn), D, false}, D, E / 16, false);
        umma_gemm(t_dv, Operand{smem_u32(sk[p]), C, false}, Operand{smem_u32(sdn), D, true}, E, D / 16, false);
        wait_or_fault(&qdo_full, one, &dead, fault, kFaultTmaWait);
        tc_fence_after_sync();
        umma_gemm(t_s, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sk[p]), C, false}, C, D / 16, false);
        umma_gemm(t_ds, Operand{smem_u32(sdo), C, false}, Operand{smem_u32(sv[p]), C, false}, C, E / 16, false);
        umma_commit(&a_done);
        // L = Q_s^T dO over S's columns: the scaled copy of Q is in the state operand's buffer, S is masked
        wait_or_fault(&ms_ready, one, &dead, fault, kFaultMmaWait);
        tc_fence_after_sync();
        umma_gemm(t_s, Operand{smem_u32(sdn), C, true}, Operand{smem_u32(sdo), C, true}, E, C / 16, false);
        umma_commit(&l_done);
        // phase B
        wait_or_fault(&sm_ready, one, &dead, fault, kFaultMmaWait);
        tc_fence_after_sync();
        umma_gemm(t_dk, Operand{smem_u32(sv[p]), C, true}, Operand{smem_u32(sq), C, true}, D, C / 16, true);    // += dS_m^T Q
        umma_gemm(t_dv, Operand{smem_u32(sk[p]), C, true}, Operand{smem_u32(sdo), C, true}, E, C / 16, true);   // += S_m^T dO
        umma_commit(&b_done);
      }
    }
  } else {
    const int cw = warp - 2;
    const int row = (warp & 3) * 32 + lane;
    const int half = cw >> 2;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    constexpr int kHalfE = E / 2;
    float Dn[kHalfE];  // this thread's part of the suffix state: row `row`, columns [half * E/2, (half+1) * E/2)
    float sl2 = 0.f, lam = 1.f;
    // q and k enter as c * map(q), c * map(k): the map is applied to the tiles in shared memory, c is folded
    // into factors that exist anyway
    // (PRE = false: instantiations without any of this, for callers who bring q and k as they are)
    const float c = PRE ? a.qk_scale : 1.f;
    const bool elu = PRE && a.elu != 0;
    if (sums) {
      sl2 = a.s[my_bh % a.h] * kLog2e;
      for (int t = sum_t0, g = 0; t < sum_t1; ++t, ++g) {
        const int j = g & 1;
        wait_or_fault(&ring_full[j], (g >> 1) & 1, &dead, fault, kFaultTmaWait);
        const float wt = c * decay_pow(sl2, (t - sum_t0) * C + row);
        if (elu)
          scale_row_pieces<D / 16, true>(sk[j], row, half * (D / 16), wt, lane);
        else
          scale_row_pieces<D / 16>(sk[j], row, half * (D / 16), wt, lane);
        fence_async_smem();
        mbar_arrive(&ring_scaled[j]);
      }
      wait_or_fault(&sum_done, 0, &dead, fault, kFaultMmaWait);
      if (tid == 64) TRACE(59);
      tc_fence_after_sync();
      if (row < D) {
#pragma unroll
        for (int c0 = 0; c0 < kHalfE; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_s + lane_base + half * kHalfE + c0, r);
          tmem_ld_wait();
          store_state32<D>(a.totals + (size_t)blockIdx.x * D * E, row, half * kHalfE + c0, r);
        }
      }
      tc_fence_before_sync();
      named_sync(1, kWorkers);   // every worker's part of the total is written ...
      if (tid == 64) {
        __threadfence();         // ... and visible to the other CTAs before the flag is
        st_volatile_u32(a.sync + kSyncFlags + blockIdx.x, step_s);
      }
      if (tid == 64) TRACE(60);
    }
    int i = 0;
    for (bool ok = w.start(blockIdx.x, gridDim.x); ok; ok = w.next(), ++i) {
      const int p = i & 1, one = i & 1;
      const int len = min(C, a.n - w.t * C);
      if (__builtin_expect(w.first_of_item(), 0)) {   // once per span: kept out of the tiles' straight-line code
        sl2 = a.s[w.bh % a.h] * kLog2e;
        lam = exp2f(-sl2);
        if constexpr (!FUSED) {
          if (row < D) load_state<kHalfE, D, false>(a.p0 + (size_t)w.it * D * E, row, half * kHalfE, Dn);
        } else {
          const int sp_idx = w.it - w.bh * a.nspans;
          const int span_end = min(w.t1 * C, a.n);
          const size_t mine = (size_t)row * E + half * kHalfE;
          // incoming rank state, decayed from the end of the sequence to the end of the span
          if (a.x_in != nullptr && row < D) {
            const float dec = decay_pow(sl2, a.n - span_end);
            const float4* src = reinterpret_cast<const float4*>(a.x_in + (size_t)w.bh * D * E + mine);
#pragma unroll
            for (int j = 0; j < kHalfE / 4; ++j) {
              const float4 v = src[j];
              Dn[4 * j] = dec * v.x, Dn[4 * j + 1] = dec * v.y, Dn[4 * j + 2] = dec * v.z, Dn[4 * j + 3] = dec * v.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < kHalfE; ++j) Dn[j] = 0.f;
          }
          // totals of the spans after this one (each decayed to its own start); one thread per flag
          if (tid - 64 < a.nspans - 1 - sp_idx && !dead) {
            if (!wait_flag_eq(a.sync + kSyncFlags + w.bh * a.nspans + sp_idx + 1 + (tid - 64), step_s, a.wait_clocks)) {
              dead = 1;
              atomicOr(fault, kFaultFlagWait);
            }
          }
          named_sync(1, kWorkers);
          for (int j = sp_idx + 1; j < a.nspans; ++j) {   // each total is decayed to the start of its span
            if (row < D)
              fma_state<kHalfE, D>(a.totals + (size_t)(w.bh * a.nspans + j) * D * E, row, half * kHalfE,
                                   decay_pow(sl2, (w.span_t0(j) - w.t1) * C), Dn);
          }
          if (LINK && a.link.ranks > 0) {
            // hand-over of the rank state inside the launch.  Dn holds the local part of the border state.
            const float sn = a.s[w.bh % a.h] * (float)a.n;
            const long long elems = (long long)(a.items / a.nspans) * D * E;
            const size_t seq_off = (size_t)w.bh * D * E;
            const int n_dst = a.link.ranks - 1 - a.link.me;
            if (n_dst > 0) {
              const int owner = w.bh * a.nspans;   // the CTA that owns the start of the sequence
              const bool far = n_dst > 1 && xl::reaches(sn, 1);   // the state reaches beyond the next rank
              uint32_t* ready = a.sync + kSyncFlags + kSyncSecondBank + w.bh;
              if (w.it == owner && far) {
                // the sequence's total, lambda^(span end) Dn + T, where the other CTAs of the sequence find it
                if (row < D)
                  link_make_total<kHalfE, D>(a.totals + (size_t)owner * D * E, row, half * kHalfE,
                                             decay_pow(sl2, span_end), Dn);
                named_sync(1, kWorkers);
                if (tid == 64) {
                  __threadfence();
                  st_volatile_u32(ready, step_s);
                }
              }
              if (far || w.it == owner) {
                // the readers of the ranks after this one in the chain order (the ranks BEFORE it in the
                // sequence) have acknowledged the slots' previous use
                if (!dead) {
                  bool ok = true;
                  if (xl::needs_ack_wait(step_x) && tid - 64 < n_dst)
                    ok = wait_flag_ge(a.link.my_acks + xl::ack_index(a.link.me + 1 + (tid - 64), 0), step_x - 2,
                                      a.link.wait_clocks);
                  if (far && tid == 64 + xl::kMaxRanks && w.it != owner) ok = wait_flag_eq(ready, step_s, a.wait_clocks);
                  if (!ok) {
                    dead = 1;
                    atomicOr(fault, kFaultRelayWait);
                  }
                }
                named_sync(1, kWorkers);
                if (row < D) {
                  if (far)
                    link_send_part<kHalfE, D>(a.link, step_x, elems, seq_off, row, half * kHalfE,
                                              a.totals + (size_t)owner * D * E, sn, sp_idx, a.nspans);
                  else
                    link_send_next<kHalfE, D>(a.link, step_x, elems, seq_off, row, half * kHalfE,
                                              decay_pow(sl2, span_end), Dn, a.totals + (size_t)owner * D * E);
                }
              }
            }
            if (a.link.me > 0 && row < D) {
              // what came from the ranks after this one in the sequence, decayed from its end to the span's
              if (!link_receive<kHalfE, D>(a.link, step_x, elems, seq_off, row, half * kHalfE,
                                           decay_pow(sl2, a.n - span_end), Dn, sn))
                atomicOr(fault, kFaultRelayWait);
            }
          }
        }
        // the phase-A MMAs that read the operand tile of the previous item have completed (a_done was waited for)
        if (row < D) write_state_operand<kHalfE>(sdn, D, row, half * kHalfE, Dn);
        fence_async_smem();
        mbar_arrive(&dn_ready);
      }
      if (tid == 64) TRACE(1 + i * 6 + 0);
      if (elu) {   // Q and K of this tile through the feature map before any product reads them
        wait_or_fault(&kv_full[p], (i >> 1) & 1, &dead, fault, kFaultTmaWait);
        wait_or_fault(&qdo_full, one, &dead, fault, kFaultTmaWait);
        scale_row_pieces<D / 16, true>(sk[p], row, half * (D / 16), 1.f, lane);
        scale_row_pieces<D / 16, true>(sq, row, half * (D / 16), 1.f, lane);
        fence_async_smem();
        mbar_arrive(&mapped);
      }
      wait_or_fault(&a_done, one, &dead, fault, kFaultMmaWait);
      wait_or_fault(&qdo_full, one, &dead, fault, kFaultTmaWait);  // completed long ago: makes Q's bytes visible here
      if (tid == 64) TRACE(1 + i * 6 + 1);
      tc_fence_after_sync();
      // row-scaled copy of Q over the state operand (phase A has read it), then S_m over the K tile
      {
        const float qd = c * decay_pow(sl2, row);
        constexpr int kPieces = D / 16;
        uint4 v[kPieces];
#pragma unroll
        for (int q = 0; q < kPieces; ++q) {
          const int piece = half * kPieces + ((q + lane) & (kPieces - 1));
          v[q] = *reinterpret_cast<const uint4*>(sq + (piece >> 3) * C * 128 + row * 128 + (piece & 7) * 16);
        }
#pragma unroll
        for (int q = 0; q < kPieces; ++q) {
          const int piece = half * kPieces + ((q + lane) & (kPieces - 1));
          uint32_t* u = reinterpret_cast<uint32_t*>(&v[q]);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u[t]));
            u[t] = pack_bf16(f.x * qd, f.y * qd);
          }
          *reinterpret_cast<uint4*>(sdn + (piece >> 3) * C * 128 + row * 128 + (piece & 7) * 16) = v[q];
        }
      }
      // S_m over the K tile, then dS_m (times Q's c) over the V tile: one piece of code for the four blocks (the
      // tile loop runs the faster the less code it spans)
#pragma unroll 1
      for (int u = 0; u < 4; ++u) {
        const int col0 = half * 64 + (u & 1) * 32;
        if (u == 2) {   // S_m is complete: the state update's product can go out
          fence_async_smem();
          tc_fence_before_sync();
          mbar_arrive(&ms_ready);
        }
        masked_store32((u < 2 ? t_s : t_ds) + lane_base + col0, (u < 2 ? sk : sv)[p], row, col0, sl2, lam,
                       u < 2 ? c * c : c);
      }
      if (tid == 64) TRACE(1 + i * 6 + 2);
      const float kd = decay_pow(sl2, max(len - row, 0));
      // the two state products take their row decay in place (32 columns at a time, dK's blocks then dV's)
#pragma unroll 1
      for (int u = 0; u < D / 64 + E / 64; ++u) {
        const bool dv_part = u >= D / 64;
        const int cc = dv_part ? u - D / 64 : u;
        scale_tmem32((dv_part ? t_dv + half * (E / 2) : t_dk + half * (D / 2)) + lane_base + cc * 32, dv_part ? kd * c : kd);
      }
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&sm_ready);
      if (tid == 64) TRACE(1 + i * 6 + 3);
      // state: Dn <- lambda^len Dn + L, while phase B runs
      wait_or_fault(&l_done, one, &dead, fault, kFaultMmaWait);
      tc_fence_after_sync();
      if (row < D) {
        const float lam_len = decay_pow(sl2, len);
#pragma unroll
        for (int c0 = 0; c0 < kHalfE; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_s + lane_base + half * kHalfE + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) Dn[c0 + j] = fmaf(lam_len, Dn[c0 + j], __uint_as_float(r[j]));
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&l_free);
      if (!w.last_of_item()) {
        if (row < D) write_state_operand<kHalfE>(sdn, D, row, half * kHalfE, Dn);
        fence_async_smem();
        mbar_arrive(&dn_ready);
      } else if constexpr (FUSED) {
        // the state after the first tile of the sequence is the outgoing rank state
        if (a.x_out != nullptr && w.t == 0 && row < D) {
          float4* dst = reinterpret_cast<float4*>(a.x_out + (size_t)w.bh * D * E + (size_t)row * E + half * kHalfE);
#pragma unroll
          for (int q = 0; q < kHalfE / 4; ++q) dst[q] = make_float4(Dn[4 * q], Dn[4 * q + 1], Dn[4 * q + 2], Dn[4 * q + 3]);
        }
      }
      if (tid == 64) TRACE(1 + i * 6 + 4);
      // epilogue: dK and dV staged over S_m and dS_m (both read by phase B)
      wait_or_fault(&b_done, one, &dead, fault, kFaultMmaWait);
      tc_fence_after_sync();
      if (elu || c != 1.f) {
        // dk = dk' * c * map'(k), k read from the raw tensor (rows past the end of the sequence are not stored)
        const bool live = row < len;
        const __nv_bfloat16* raw =
            static_cast<const __nv_bfloat16*>(a.raw) + ((size_t)w.bh * a.n + (size_t)w.t * C + (live ? row : 0)) * a.raw_pitch;
#pragma unroll 1
        for (int cc = 0; cc < D / 64; ++cc) {
          const int col0 = half * (D / 2) + cc * 32;
          stage_row32_chain(t_dk + lane_base + col0, sk[p], row, col0, raw, c, elu && live);
        }
      }
      // dV's blocks, and dK's too unless the chain rule above has staged them: one loop
#pragma unroll 1
      for (int u = (elu || c != 1.f) ? D / 64 : 0; u < D / 64 + E / 64; ++u) {
        const bool dv_part = u >= D / 64;
        const int cc = dv_part ? u - D / 64 : u;
        const int col0 = half * ((dv_part ? E : D) / 2) + cc * 32;
        stage_row32((dv_part ? t_dv : t_dk) + lane_base + col0, kNoAcc, 0.f, (dv_part ? sv : sk)[p], row,
                    col0);
      }
      tc_fence_before_sync();
      mbar_arrive(&e_free);
      fence_async_smem();
      mbar_arrive(&staged[p]);
      if (tid == 64) TRACE(1 + i * 6 + 5);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 64) TRACE(63);
  if (tid == 64) GTRACE(58);
  if (warp == 2) tmem_dealloc(tmem, 512);
  if constexpr (FUSED) {
    if (tid == 0 && a.coop) {
      __threadfence();
      if (atomicAdd(a.sync + 1, 1u) == gridDim.x - 1) {
        st_volatile_u32(a.sync + 1, 0u);
        __threadfence();
        st_volatile_u32(a.sync, step_s);
        if (LINK && a.link.ranks > 0) {
          for (int q = 0; q < a.link.me; ++q) st_volatile_u32(a.link.src_acks[q] + xl::ack_index(a.link.me, 0), step_x);
          st_volatile_u32(a.link.counters, step_x);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename F>
cudaError_t opt_in_smem(F* fn, size_t bytes) {
  cudaError_t err = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) g_failed_step = "cudaFuncSetAttribute(max dynamic shared memory)";
  return err;
}

cudaError_t seq_map(CUtensorMap* map, const void* base, const Dims& m, int width, int pitch, const char* what) {
  cudaError_t err = make_seq_tile_map(map, base, (uint64_t)m.b * m.h, (uint64_t)m.n, (uint32_t)width, C, (uint32_t)pitch);
  if (err != cudaSuccess) {
    static thread_local char text[160];
    snprintf(text, sizeof(text), "tensor map (%s): CUresult %d, base %p, b*h %d, n %d, width %d", what,
             last_encode_result(), base, m.b * m.h, m.n, width);
    g_failed_step = text;
  }
  return err;
}

cudaError_t launched(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) g_failed_step = what;
  return err;
}

int grid_for(int items) {
  const int sms = sm_count();
  return items < sms ? items : sms;
}

template <int D, int E>
cudaError_t launch_span_totals(const Dims& m, const void* a, const void* bten, const float* s, float* totals,
                               bool reverse, cudaStream_t st) {
  CUtensorMap ma, mb;
  cudaError_t err;
  if ((err = seq_map(&ma, a, m, D, m.pitch_d, "span totals, first operand")) != cudaSuccess) return err;
  if ((err = seq_map(&mb, bten, m, E, m.pitch_e, "span totals, second operand")) != cudaSuccess) return err;
  int32_t* fault = nullptr;
  if ((err = fault_word_address(&fault)) != cudaSuccess) return err;
  const size_t smem = (size_t)3 * C * (D + E) * 2 + 1024;
  if ((err = opt_in_smem(k_span_totals<D, E>, smem)) != cudaSuccess) return err;
  const int items = m.b * m.h * m.nc;
  k_span_totals<D, E><<<grid_for(items), 320, smem, st>>>(ma, mb, s, totals, m.h, m.n, m.tiles, m.span, m.nc, items,
                                                          reverse ? 1 : 0, fault);
  return launched("launch of the span-total kernel");
}

// The CTAs of a fused launch wait for one another's totals.  They are at most one per SM (the host side
// checks), so all of them become resident as soon as whatever ran before has drained; their waits are
// bounded all the same and report through the fault word.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), int grid, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(320);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr long long kFlagWaitClocks = 1000000000LL;   // about half a second

template <int D, int E, bool DQ, bool FUSED, bool PRE, bool LINK>
cudaError_t launch_walk_out_pre(const Dims& m, const void* x, const void* y, const void* z, void* out, WalkArgs a,
                            cudaStream_t st) {
  constexpr int WX = DQ ? E : D, WZ = DQ ? D : E;
  CUtensorMap mx, my, mz, mo;
  cudaError_t err;
  if ((err = seq_map(&mx, x, m, WX, DQ ? m.pitch_e : m.pitch_d, DQ ? "do" : "q")) != cudaSuccess) return err;
  if ((err = seq_map(&my, y, m, WX, DQ ? m.pitch_e : m.pitch_d, DQ ? "v" : "k")) != cudaSuccess) return err;
  if ((err = seq_map(&mz, z, m, WZ, DQ ? m.pitch_d : m.pitch_e, DQ ? "k" : "v")) != cudaSuccess) return err;
  if ((err = seq_map(&mo, out, m, WZ, DQ ? m.pitch_d : m.pitch_e, DQ ? "dq" : "o")) != cudaSuccess) return err;
  if ((err = fault_word_address(&a.fault)) != cudaSuccess) return err;
  const size_t smem = (size_t)7 * kBuf + 1024;
  if ((err = opt_in_smem(k_walk_out<D, E, DQ, FUSED, PRE, LINK>, smem)) != cudaSuccess) return err;
  a.h = m.h, a.n = m.n, a.tiles = m.tiles, a.span = m.span, a.nspans = m.nc, a.items = m.b * m.h * m.nc;
  a.wait_clocks = kFlagWaitClocks;
  a.qk_scale = m.qk_scale, a.elu = m.qk_map, a.raw_pitch = m.pitch_d;
  const bool waits = FUSED && (m.nc > 1 || a.link.ranks > 0);   // CTAs wait for one another: one span each, all resident
  a.coop = waits ? 1 : 0;
  if (waits) a.even = 1;
  if (a.link.ranks > 0 && a.link.me < a.link.ranks - 1) a.all_totals = 1;   // the sequence totals are sent on
  if (waits && a.items > sm_count()) {
    g_failed_step = "fused walk kernel: more spans than SMs";
    return cudaErrorInvalidConfiguration;
  }
  if ((err = launch_kernel(k_walk_out<D, E, DQ, FUSED, PRE, LINK>, grid_for(a.items), smem, st, mx, my, mz, mo, a)) !=
      cudaSuccess) {
    g_failed_step = "launch of a walk kernel";
    return err;
  }
  return launched(DQ ? "launch of the dq walk kernel" : "launch of the forward walk kernel");
}

template <int D, int E, bool FUSED, bool PRE, bool LINK>
cudaError_t launch_walk_dkv_pre(const Dims& m, const void* q, const void* k, const void* v, const void* d_o, void* dk,
                            void* dv, WalkArgs a, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mdo, mdk, mdv;
  cudaError_t err;
  if ((err = seq_map(&mq, q, m, D, m.pitch_d, "q")) != cudaSuccess) return err;
  if ((err = seq_map(&mk, k, m, D, m.pitch_d, "k")) != cudaSuccess) return err;
  if ((err = seq_map(&mv, v, m, E, m.pitch_e, "v")) != cudaSuccess) return err;
  if ((err = seq_map(&mdo, d_o, m, E, m.pitch_e, "do")) != cudaSuccess) return err;
  if ((err = seq_map(&mdk, dk, m, D, m.pitch_d, "dk")) != cudaSuccess) return err;
  if ((err = seq_map(&mdv, dv, m, E, m.pitch_e, "dv")) != cudaSuccess) return err;
  if ((err = fault_word_address(&a.fault)) != cudaSuccess) return err;
  a.raw = k;   // for the chain rule of a folded k preprocessing
  const size_t smem = (size_t)7 * kBuf + 1024;
  if ((err = opt_in_smem(k_walk_dkv<D, E, FUSED, PRE, LINK>, smem)) != cudaSuccess) return err;
  a.h = m.h, a.n = m.n, a.tiles = m.tiles, a.span = m.span, a.nspans = m.nc, a.items = m.b * m.h * m.nc;
  a.wait_clocks = kFlagWaitClocks;
  a.qk_scale = m.qk_scale, a.elu = m.qk_map, a.raw_pitch = m.pitch_d;
  const bool waits = FUSED && (m.nc > 1 || a.link.ranks > 0);
  a.coop = waits ? 1 : 0;
  if (waits) a.even = 1;
  if (a.link.ranks > 0 && a.link.me < a.link.ranks - 1) a.all_totals = 1;
  if (waits && a.items > sm_count()) {
    g_failed_step = "fused walk kernel: more spans than SMs";
    return cudaErrorInvalidConfiguration;
  }
  if ((err = launch_kernel(k_walk_dkv<D, E, FUSED, PRE, LINK>, grid_for(a.items), smem, st, mq, mk, mv, mdo, mdk, mdv, a)) !=
      cudaSuccess) {
    g_failed_step = "launch of the dk/dv walk kernel";
    return err;
  }
  return launched("launch of the dk/dv walk kernel");
}

// the instantiations with the q,k preprocessing only where it is asked for: the others keep the short code
template <int D, int E, bool DQ, bool FUSED>
cudaError_t launch_walk_out(const Dims& m, const void* x, const void* y, const void* z, void* out, WalkArgs a,
                            cudaStream_t st) {
  // ... and the hand-over code only in the launches of a sequence-parallel rank
  const bool linked = a.link.ranks > 0;
  if (has_qk_preprocessing(m)) {
    if constexpr (FUSED) {
      return linked ? launch_walk_out_pre<D, E, DQ, true, true, true>(m, x, y, z, out, a, st)
                    : launch_walk_out_pre<D, E, DQ, true, true, false>(m, x, y, z, out, a, st);
    } else if constexpr (DQ) {
      return launch_walk_out_pre<D, E, true, false, true, false>(m, x, y, z, out, a, st);
    }
    g_failed_step = "q,k preprocessing is not part of the phase-by-phase schedule";
    return cudaErrorInvalidValue;
  }
  if constexpr (FUSED) {
    if (linked) return launch_walk_out_pre<D, E, DQ, true, false, true>(m, x, y, z, out, a, st);
  }
  return launch_walk_out_pre<D, E, DQ, FUSED, false, false>(m, x, y, z, out, a, st);
}
template <int D, int E, bool FUSED>
cudaError_t launch_walk_dkv(const Dims& m, const void* q, const void* k, const void* v, const void* d_o, void* dk,
                            void* dv, WalkArgs a, cudaStream_t st) {
  const bool linked = a.link.ranks > 0;
  if (has_qk_preprocessing(m)) {
    if constexpr (FUSED) {
      return linked ? launch_walk_dkv_pre<D, E, true, true, true>(m, q, k, v, d_o, dk, dv, a, st)
                    : launch_walk_dkv_pre<D, E, true, true, false>(m, q, k, v, d_o, dk, dv, a, st);
    }
    g_failed_step = "q,k preprocessing is not part of the phase-by-phase schedule";
    return cudaErrorInvalidValue;
  }
  if constexpr (FUSED) {
    if (linked) return launch_walk_dkv_pre<D, E, true, false, true>(m, q, k, v, d_o, dk, dv, a, st);
  }
  return launch_walk_dkv_pre<D, E, FUSED, false, false>(m, q, k, v, d_o, dk, dv, a, st);
}

}  // namespace

#define LASP_DISPATCH_DE(m, CALL)                                        \
  do {                                                                    \
    if ((m).d == 128 && (m).e == 128) return CALL(128, 128);              \
    if ((m).d == 128 && (m).e == 64) return CALL(128, 64);                \
    if ((m).d == 64 && (m).e == 128) return CALL(64, 128);                \
    if ((m).d == 64 && (m).e == 64) return CALL(64, 64);                  \
    return cudaErrorInvalidValue;                                         \
  } while (0)

cudaError_t walk_span_totals(const Dims& m, const void* a, const void* bten, const float* s, float* totals,
                             bool reverse, cudaStream_t st) {
#define LASP_CALL(DD, EE) launch_span_totals<DD, EE>(m, a, bten, s, totals, reverse, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

cudaError_t walk_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                            const float* prefix, uint32_t* sync, void* o, cudaStream_t st) {
  WalkArgs a = {};
  a.s = s, a.p0 = prefix, a.sync = sync;   // sync: only the word that says how the sequences were cut
#define LASP_CALL(DD, EE) launch_walk_out<DD, EE, false, false>(m, q, k, v, o, a, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

// the walk kernels' view of the caller's peer-mapped buffers (NULL: no link)
static Link make_link(const lasp_exchange_args* x) {
  Link l = {};
  if (x == nullptr) return l;
  l.my_slots = static_cast<const uint2*>(x->my_slots);
  l.my_acks = x->my_acks;
  l.counters = x->counters;
  for (int i = 0; i < xl::kMaxRanks; ++i) {
    l.src_acks[i] = x->peer_acks[i];
    l.dst_slots[i] = static_cast<uint2*>(x->peer_slots[i]);
  }
  l.ranks = x->ranks;
  l.me = x->position;
  l.wait_clocks = x->wait_clocks > 0 ? x->wait_clocks : 20000000000LL;   // about ten seconds
  return l;
}

cudaError_t walk_fwd_fused(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                           const float* x_in, float* x_out, uint32_t* sync, float* totals, float* prefix, void* o,
                           const lasp_exchange_args* link, cudaStream_t st) {
  WalkArgs a = {};
  a.link = make_link(link);
  a.s = s, a.x_in = x_in, a.x_out = x_out, a.sync = sync, a.totals = totals, a.p0_save = prefix;
#define LASP_CALL(DD, EE) launch_walk_out<DD, EE, false, true>(m, q, k, v, o, a, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

cudaError_t walk_bwd_dq(const Dims& m, const void* q, const void* k, const void* v, const void* d_o, const float* s,
                        const float* prefix, const uint32_t* fwd_sync, void* dq, cudaStream_t st) {
  WalkArgs a = {};
  a.s = s, a.p0 = prefix, a.even_word = fwd_sync + kSyncEven;   // cut the sequences as the forward pass did
  a.raw = q;                                                    // for the chain rule of a folded q preprocessing
#define LASP_CALL(DD, EE) launch_walk_out<DD, EE, true, false>(m, d_o, v, k, dq, a, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

cudaError_t walk_bwd_dkv(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                         const float* s, const float* suffix, void* dk, void* dv, cudaStream_t st) {
  WalkArgs a = {};
  a.s = s, a.p0 = suffix;
#define LASP_CALL(DD, EE) launch_walk_dkv<DD, EE, false>(m, q, k, v, d_o, dk, dv, a, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

cudaError_t walk_bwd_dkv_fused(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                               const float* s, const float* x_in, float* x_out, uint32_t* sync, float* totals,
                               void* dk, void* dv, const lasp_exchange_args* link, cudaStream_t st) {
  WalkArgs a = {};
  a.link = make_link(link);
  a.s = s, a.x_in = x_in, a.x_out = x_out, a.sync = sync, a.totals = totals;
#define LASP_CALL(DD, EE) launch_walk_dkv<DD, EE, true>(m, q, k, v, d_o, dk, dv, a, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

#ifdef LASP_TRACE
extern "C" __attribute__((visibility("default"))) int lasp_b200_debug_trace(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_trace, sizeof(long long) * 160 * 64);
}
#endif

}  // namespace lasp
