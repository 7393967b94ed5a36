// Tensor-core path: tcgen05 MMAs with accumulators in tensor memory, operands
// staged in shared memory by TMA.  bf16 inputs, fp32 accumulation, one rounding
// on store.  The unit of work is a tile: one 128-token chunk of one (batch, head).
//
// Every tile in shared memory is in the swizzled slab format of sm100.cuh, so a
// tile loaded once serves both as a K-major operand (rows = M/N) and as an
// MN-major operand (rows = K).  The decay mask is applied between MMAs on the
// way from tensor memory back to shared memory (S -> S_m as bf16).
//
//   k_tc_chunk_states      one CTA per tile: (decay-scaled K)^T V or (decay-scaled Q)^T dO
//   k_tc_chunk_states_v2   the same as a persistent pipeline (gated, see below)
//   k_tc_fwd_output        persistent: O = S_m V + diag(lambda^r) Q P
//   k_tc_bwd_grads         persistent: dQ, dK, dV
//
// All waits are bounded; a wait that runs out sets a bit in g_fault_word and the
// CTA skips its remaining waits, frees its tensor memory and exits.
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "sm100.cuh"

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

namespace {

using namespace sm100;

constexpr int C = kTensorTile;  // 128 tokens per tile

// bounded wait that records a fault once and makes later waits of the CTA no-ops
__device__ __forceinline__ void wait_or_fault(uint64_t* bar, uint32_t parity, volatile int* dead, int32_t code) {
  if (*dead) return;
  if (!mbar_wait(bar, parity)) {
    *dead = 1;
    atomicOr(&g_fault_word, code);
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

// acc (32 columns) *= f, in tensor memory
__device__ __forceinline__ void scale_tmem32(uint32_t taddr, float f) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
  tmem_st32(taddr, r);
}

// out_row[col0 .. col0+31] = bf16(acc1 + f * acc2)  (acc2 skipped when taddr2 == 0xFFFFFFFF)
__device__ __forceinline__ void store_row32(uint32_t taddr1, uint32_t taddr2, float f, __nv_bfloat16* out_row,
                                            int col0) {
  uint32_t a[32];
  tmem_ld32(taddr1, a);
  if (taddr2 != 0xFFFFFFFFu) {
    uint32_t b[32];
    tmem_ld32(taddr2, b);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) a[j] = __float_as_uint(fmaf(f, __uint_as_float(b[j]), __uint_as_float(a[j])));
  } else {
    tmem_ld_wait();
  }
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 v = make_uint4(pack_bf16(__uint_as_float(a[j]), __uint_as_float(a[j + 1])),
                         pack_bf16(__uint_as_float(a[j + 2]), __uint_as_float(a[j + 3])),
                         pack_bf16(__uint_as_float(a[j + 4]), __uint_as_float(a[j + 5])),
                         pack_bf16(__uint_as_float(a[j + 6]), __uint_as_float(a[j + 7])));
    *reinterpret_cast<uint4*>(out_row + col0 + j) = v;
  }
}

// tile[row][col0 .. col0+31] = bf16(acc1 + f * acc2) into a swizzled staging tile of C rows
// (acc2 skipped when taddr2 == 0xFFFFFFFF); a TMA store then moves the tile out
__device__ __forceinline__ void stage_row32(uint32_t taddr1, uint32_t taddr2, float f, uint8_t* tile, int row,
                                            int col0) {
  uint32_t a[32];
  tmem_ld32(taddr1, a);
  if (taddr2 != 0xFFFFFFFFu) {
    uint32_t b[32];
    tmem_ld32(taddr2, b);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) a[j] = __float_as_uint(fmaf(f, __uint_as_float(b[j]), __uint_as_float(a[j])));
  } else {
    tmem_ld_wait();
  }
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 v = make_uint4(pack_bf16(__uint_as_float(a[j]), __uint_as_float(a[j + 1])),
                         pack_bf16(__uint_as_float(a[j + 2]), __uint_as_float(a[j + 3])),
                         pack_bf16(__uint_as_float(a[j + 4]), __uint_as_float(a[j + 5])),
                         pack_bf16(__uint_as_float(a[j + 6]), __uint_as_float(a[j + 7])));
    *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + j, C)) = v;
  }
}

// ---------------------------------------------------------------------------
// chunk states: out[i][j] = sum_c w_c A[c][i] B[c][j]   (A = K or Q, B = V or dO)
// ---------------------------------------------------------------------------
template <int D, int E, bool PDL>
__global__ void __launch_bounds__(128) k_tc_chunk_states(const __grid_constant__ CUtensorMap map_a,
                                                         const __grid_constant__ CUtensorMap map_b,
                                                         const float* __restrict__ s,
                                                         __nv_bfloat16* __restrict__ states, int h, int n, int nc,
                                                         int backward) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sa = smem;               // C x D  (followed by sb: with D = 64 the M = 128 MMA reads on into sb)
  uint8_t* sb = smem + C * D * 2;   // C x E
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const float sh = s[bh % h];
  if (tid == 0) {
    dead = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 128);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if constexpr (PDL) {
    // inputs may come from the kernel ahead and the states may still be read by it
    grid_dependency_wait();
    if (tid == 0) grid_launch_dependents();
  }
  const uint32_t tmem = tmem_slot;
  const int row0 = bh * n + chunk * C;
  if (tid == 0) {
    mbar_expect_tx(&bar_load, C * (D + E) * 2);
    tma_load_3d(sa, &map_a, &bar_load, 0, row0, 0);
    tma_load_3d(sb, &map_b, &bar_load, 0, row0, 0);
  }
  wait_or_fault(&bar_load, 0, &dead, kFaultTmaWait);
  // scale row `tid` of A by its decay weight, in place (chunks of a row stay in the row under the swizzle)
  {
    const float w = backward ? expf(-sh * (float)tid) : expf(-sh * (float)(C - tid));
#pragma unroll
    for (int slab = 0; slab < D / 64; ++slab) {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int j = (jj + lane) & 7;  // spread the 16-byte chunks of a quarter warp over the banks
        uint4* p = reinterpret_cast<uint4*>(sa + slab * C * 128 + tid * 128 + j * 16);
        uint4 v = *p;
        uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          __nv_bfloat162 hh = *reinterpret_cast<__nv_bfloat162*>(&u[t]);
          float2 f = __bfloat1622float2(hh);
          u[t] = pack_bf16(f.x * w, f.y * w);
        }
        *p = v;
      }
    }
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && !dead) {
    tc_fence_after_sync();
    const Operand a{smem_u32(sa), C, true}, b{smem_u32(sb), C, true};
    umma_gemm(tmem, a, b, E, C / 16, false);
    umma_commit(&bar_mma);
  }
  wait_or_fault(&bar_mma, 0, &dead, kFaultMmaWait);
  tc_fence_after_sync();
  if (tid < D) {
    __nv_bfloat16* out = states + ((size_t)bh * nc + chunk) * D * E + (size_t)tid * E;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll
    for (int c0 = 0; c0 < E; c0 += 32) store_row32(tmem + lane_base + c0, 0xFFFFFFFFu, 0.f, out, c0);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// ---------------------------------------------------------------------------
// chunk states, persistent variant (selected with LASP_B200_CHUNK_STATES_V2=1 until verified on a GPU)
//
// Same arithmetic as k_tc_chunk_states.  One CTA per SM walks over tiles; ten warps in four roles:
//   warp 0 (one lane)  producer: A and B tiles into a two-stage ring
//   warp 1 (one lane)  tensor-core issuer, accumulators double buffered (2 x 128 columns)
//   warps 2-5          scale the rows of A by their decay weights in place (row = thread)
//   warps 6-9          accumulator -> bf16 -> swizzled staging tile -> one TMA store per tile
// so the loads of tile i+1, the row scaling of tile i+1 and the store of tile i-1 overlap the MMA of tile i.
// ---------------------------------------------------------------------------
template <int D, int E>
__global__ void __launch_bounds__(320, 1) k_tc_chunk_states_v2(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b,
                                                               const __grid_constant__ CUtensorMap map_out,
                                                               const float* __restrict__ s, int h, int n, int nc,
                                                               int num_tiles, int backward) {
  constexpr int kA = C * D * 2, kB = C * E * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  // per stage: A then B (with D = 64 the M = 128 MMA reads on from A into B, which is valid memory)
  uint8_t* sa[2] = {smem, smem + kA + kB};
  uint8_t* sb[2] = {smem + kA, smem + 2 * kA + kB};
  uint8_t* so = smem + 2 * (kA + kB);   // D x E staging tile
  __shared__ uint64_t full[2], scaled[2], mma_done[2], t_free[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    dead = 0;
    for (int j = 0; j < 2; ++j) {
      mbar_init(&full[j], 1);
      mbar_init(&scaled[j], 128);
      mbar_init(&mma_done[j], 1);
      mbar_init(&t_free[j], 128);
    }
    fence_mbar_init();
  }
  if (warp == 2) tmem_alloc(&tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int i = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
        const int bh = t / nc, chunk = t - bh * nc, row0 = bh * n + chunk * C, j = i & 1;
        if (i >= 2) wait_or_fault(&mma_done[j], ((i - 2) >> 1) & 1, &dead, kFaultMmaWait);  // stage j has been read
        mbar_expect_tx(&full[j], kA + kB);
        tma_load_3d(sa[j], &map_a, &full[j], 0, row0, 0);
        tma_load_3d(sb[j], &map_b, &full[j], 0, row0, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int i = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
        const int j = i & 1, ph = (i >> 1) & 1;
        if (i >= 2) wait_or_fault(&t_free[j], ((i - 2) >> 1) & 1, &dead, kFaultMmaWait);  // accumulator j drained
        wait_or_fault(&scaled[j], ph, &dead, kFaultTmaWait);
        tc_fence_after_sync();
        umma_gemm(tmem + 128 * j, Operand{smem_u32(sa[j]), C, true}, Operand{smem_u32(sb[j]), C, true}, E, C / 16,
                  false);
        umma_commit(&mma_done[j]);
      }
    }
  } else if (warp < 6) {
    const int row = tid - 64;   // 0..127: the token of the tile this thread scales
    int i = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
      const int bh = t / nc, j = i & 1, ph = (i >> 1) & 1;
      const float sh = s[bh % h];
      const float w = backward ? expf(-sh * (float)row) : expf(-sh * (float)(C - row));
      wait_or_fault(&full[j], ph, &dead, kFaultTmaWait);
#pragma unroll
      for (int slab = 0; slab < D / 64; ++slab) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int c16 = (jj + lane) & 7;  // spread the 16-byte chunks of a quarter warp over the banks
          uint4* p = reinterpret_cast<uint4*>(sa[j] + slab * C * 128 + row * 128 + c16 * 16);
          uint4 v = *p;
          uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u[q]));
            u[q] = pack_bf16(f.x * w, f.y * w);
          }
          *p = v;
        }
      }
      fence_async_smem();
      mbar_arrive(&scaled[j]);
    }
  } else {
    const int row = (warp & 3) * 32 + lane;   // tensor-memory lane = row of the state; warps 6..9 -> quarters 2,3,0,1
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const bool leader = (warp == 6 && lane == 0);
    int i = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
      const int j = i & 1, ph = (i >> 1) & 1;
      wait_or_fault(&mma_done[j], ph, &dead, kFaultMmaWait);
      tc_fence_after_sync();
      if (leader) bulk_wait_read<0>();   // the previous tile's store has read the staging tile
      named_sync(2, 128);
      if (row < D) {
#pragma unroll
        for (int c0 = 0; c0 < E; c0 += 32) {
          uint32_t a[32];
          tmem_ld32(tmem + 128 * j + lane_base + c0, a);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 32; q += 8) {
            const uint4 v = make_uint4(pack_bf16(__uint_as_float(a[q]), __uint_as_float(a[q + 1])),
                                       pack_bf16(__uint_as_float(a[q + 2]), __uint_as_float(a[q + 3])),
                                       pack_bf16(__uint_as_float(a[q + 4]), __uint_as_float(a[q + 5])),
                                       pack_bf16(__uint_as_float(a[q + 6]), __uint_as_float(a[q + 7])));
            *reinterpret_cast<uint4*>(so + tile_offset(row, c0 + q, D)) = v;
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&t_free[j]);
      fence_async_smem();
      named_sync(2, 128);
      if (leader) {
        tma_store_3d(&map_out, so, 0, t * D, 0);   // state tile t = (bh * nc + chunk)
        bulk_commit();
      }
    }
    if (leader) bulk_wait_all<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------
// forward output: O = S_m V + diag(lambda^r) Q P      (persistent, pipelined)
//
// One CTA per SM walks over tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...
// Ten warps in three roles, synchronised only through mbarriers:
//   warp 0 (one lane)  producer: TMA loads of Q, P (single buffers) and K, V
//                      (two buffers each), issued as soon as a buffer is free
//   warp 1 (one lane)  tensor-core issuer: S = Q K^T and O2 = Q P, then, once
//                      S_m is in shared memory, O1 = S_m V over S's columns
//   warps 2-9          S -> decay mask -> S_m (bf16, over the K buffer);
//                      epilogue O = O1 + lambda^r O2 -> global
// Tensor memory is double buffered (256 columns per tile parity), so the loads
// and the first MMAs of tile i+1 overlap the mask and epilogue work of tile i.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float decay_pow(float sl2, int k) { return exp2f(-sl2 * (float)k); }

// Tensor-memory accumulator (32 columns at `taddr`, this thread's lane = row) ->
// decay-masked bf16 in a K-major swizzled tile:
//   out[row][col] = [row >= col] lambda^(row-col) acc[col].
// The factor is built from the right-most unmasked column leftwards by repeated
// multiplication with lambda, so it can only underflow towards the far columns.
__device__ __forceinline__ void masked_store32(uint32_t taddr, uint8_t* tile, int row, int col0, float sl2,
                                               float lam) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
  tmem_ld_wait();
  const int first = min(row, col0 + 31);  // right-most column of this group with row >= col
  float f = decay_pow(sl2, row - first);
  float m[32];
#pragma unroll
  for (int j = 31; j >= 0; --j) {
    const bool live = (col0 + j) <= row;
    m[j] = live ? __uint_as_float(r[j]) * f : 0.f;
    f = live ? f * lam : f;
  }
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const uint4 v = make_uint4(pack_bf16(m[j], m[j + 1]), pack_bf16(m[j + 2], m[j + 3]), pack_bf16(m[j + 4], m[j + 5]),
                               pack_bf16(m[j + 6], m[j + 7]));
    *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + j, C)) = v;
  }
}

constexpr float kLog2e = 1.4426950408889634f;

template <int D, int E, bool PDL>
__global__ void __launch_bounds__(320, 1) k_tc_fwd_output(const __grid_constant__ CUtensorMap map_q,
                                                          const __grid_constant__ CUtensorMap map_k,
                                                          const __grid_constant__ CUtensorMap map_v,
                                                          const __grid_constant__ CUtensorMap map_p,
                                                          const __grid_constant__ CUtensorMap map_o,
                                                          const float* __restrict__ s, int h, int n, int nc,
                                                          int num_tiles) {
  constexpr int kQ = C * D * 2, kP = D * E * 2, kK = C * C * 2 /* K, then S_m; C >= D */, kV = C * E * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sq = smem;
  uint8_t* sp = sq + kQ;
  uint8_t* sk[2] = {sp + kP, sp + kP + kK};
  uint8_t* sv[2] = {sp + kP + 2 * kK, sp + kP + 2 * kK + kV};
  uint8_t* so = sv[1] + kV;  // C x E staging tile of the output
  __shared__ uint64_t qp_full, p_full, k_full[2], v_full[2], s_full[2], sm_ready[2], o_full[2], t_free[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    dead = 0;
    mbar_init(&qp_full, 1);
    mbar_init(&p_full, 1);   // used by the dependent-launch variant only: P arrives apart from Q
    for (int p = 0; p < 2; ++p) {
      mbar_init(&k_full[p], 1);
      mbar_init(&v_full[p], 1);
      mbar_init(&s_full[p], 1);
      mbar_init(&sm_ready[p], 256);
      mbar_init(&o_full[p], 1);
      mbar_init(&t_free[p], 256);
    }
    fence_mbar_init();
  }
  if (warp == 2) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int i = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
        const int bh = t / nc, chunk = t - bh * nc, row0 = bh * n + chunk * C, p = i & 1;
        if (i >= 2) wait_or_fault(&o_full[p], ((i - 2) >> 1) & 1, &dead, kFaultMmaWait);  // K/S_m, V of tile i-2 read
        mbar_expect_tx(&k_full[p], kQ);
        tma_load_3d(sk[p], &map_k, &k_full[p], 0, row0, 0);
        mbar_expect_tx(&v_full[p], kV);
        tma_load_3d(sv[p], &map_v, &v_full[p], 0, row0, 0);
        if (i >= 1) wait_or_fault(&s_full[(i - 1) & 1], ((i - 1) >> 1) & 1, &dead, kFaultMmaWait);  // Q, P read
        if constexpr (!PDL) {
          mbar_expect_tx(&qp_full, kQ + kP);
          tma_load_3d(sq, &map_q, &qp_full, 0, row0, 0);
          tma_load_3d(sp, &map_p, &qp_full, 0, (bh * nc + chunk) * D, 0);
        } else {
          // q, k, v are older than the chain of launches this kernel belongs to and may be read at once;
          // the prefix states are written by the scan just ahead: wait for it before the first P load
          mbar_expect_tx(&qp_full, kQ);
          tma_load_3d(sq, &map_q, &qp_full, 0, row0, 0);
          if (i == 0) {
            grid_dependency_wait();
            grid_launch_dependents();
          }
          mbar_expect_tx(&p_full, kP);
          tma_load_3d(sp, &map_p, &p_full, 0, (bh * nc + chunk) * D, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int i = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
        const int p = i & 1, ph2 = (i >> 1) & 1;
        const uint32_t t_s = tmem + 256 * p, t_o2 = t_s + 128;
        if (i >= 2) wait_or_fault(&t_free[p], ((i - 2) >> 1) & 1, &dead, kFaultMmaWait);
        wait_or_fault(&qp_full, i & 1, &dead, kFaultTmaWait);
        wait_or_fault(&k_full[p], ph2, &dead, kFaultTmaWait);
        tc_fence_after_sync();
        umma_gemm(t_s, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sk[p]), C, false}, C, D / 16, false);
        if constexpr (PDL) {
          wait_or_fault(&p_full, i & 1, &dead, kFaultTmaWait);
          tc_fence_after_sync();
        }
        umma_gemm(t_o2, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sp), D, true}, E, D / 16, false);
        umma_commit(&s_full[p]);
        wait_or_fault(&sm_ready[p], ph2, &dead, kFaultMmaWait);
        wait_or_fault(&v_full[p], ph2, &dead, kFaultTmaWait);
        tc_fence_after_sync();
        umma_gemm(t_s, Operand{smem_u32(sk[p]), C, false}, Operand{smem_u32(sv[p]), C, true}, E, C / 16, false);
        umma_commit(&o_full[p]);
      }
    }
  } else {
    const int cw = warp - 2;                       // 0..7
    const int row = (warp & 3) * 32 + lane;        // tensor-memory lane quarter of this warp
    const int half = cw >> 2;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int i = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
      const int bh = t / nc, chunk = t - bh * nc, row0 = bh * n + chunk * C, p = i & 1, ph2 = (i >> 1) & 1;
      const uint32_t t_s = tmem + 256 * p, t_o2 = t_s + 128;
      const float sl2 = s[bh % h] * kLog2e;
      const float lam = exp2f(-sl2);
      wait_or_fault(&s_full[p], ph2, &dead, kFaultMmaWait);
      tc_fence_after_sync();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col0 = half * 64 + cc * 32;
        masked_store32(t_s + lane_base + col0, sk[p], row, col0, sl2, lam);
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&sm_ready[p]);
      wait_or_fault(&o_full[p], ph2, &dead, kFaultMmaWait);
      tc_fence_after_sync();
      // the staging tile is free once the previous tile's store has read it
      if (cw == 0 && lane == 0) {
        bulk_wait_read<0>();
        if constexpr (PDL) {
          if (i == 0) grid_dependency_wait();   // the output may still be read by a kernel ahead
        }
      }
      named_sync(1, 256);
      const float qd = decay_pow(sl2, row);
#pragma unroll
      for (int cc = 0; cc < E / 64; ++cc) {
        const int col0 = half * (E / 2) + cc * 32;
        stage_row32(t_s + lane_base + col0, t_o2 + lane_base + col0, qd, so, row, col0);
      }
      tc_fence_before_sync();
      mbar_arrive(&t_free[p]);
      fence_async_smem();
      named_sync(1, 256);
      if (cw == 0 && lane == 0) {
        tma_store_3d(&map_o, so, 0, row0, 0);
        bulk_commit();
      }
    }
    if (cw == 0 && lane == 0) bulk_wait_all<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// backward: dQ = dS_m K + diag(lambda^r) dO P^T
//           dK = dS_m^T Q + diag(lambda^(C-c)) V Dn^T
//           dV = S_m^T dO + diag(lambda^(C-c)) K Dn          (persistent)
//
// Seven shared-memory tiles (Q, K, V, dO, Dn, dS_m, P -> S_m) and all 512
// tensor-memory columns are in use, so tiles cannot be double buffered; what
// overlaps is the next tile's six loads with this tile's epilogue.
//   warp 0 (one lane)  producer: as soon as the last MMAs of tile i have
//                      completed, loads tile i+1 into the same buffers
//   warp 1 (one lane)  tensor-core issuer.  Phase A: S = Q K^T (T0),
//                      dS = dO V^T (T1), dO P^T (T2), V Dn^T (T3).  Phase B,
//                      after the warps below: T2 += dS_m K, T3 += dS_m^T Q,
//                      T0 = S_m^T dO, T1 = K Dn
//   warps 2-9          S, dS -> decay mask -> S_m, dS_m in shared memory; T2, T3
//                      scaled by their row decays in place; epilogue dQ = T2,
//                      dK = T3, dV = T0 + lambda^(C-c) T1, staged one after the
//                      other through the dS_m tile and stored by TMA
// ---------------------------------------------------------------------------
template <int D, int E, bool PDL>
__global__ void __launch_bounds__(320, 1) k_tc_bwd_grads(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_dn,
    const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ CUtensorMap map_dk,
    const __grid_constant__ CUtensorMap map_dv, const float* __restrict__ s, int h, int n, int nc, int num_tiles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sq = smem;                   // C x D
  uint8_t* sk = sq + C * D * 2;         // C x D
  uint8_t* sv = sk + C * D * 2;         // C x E
  uint8_t* sdo = sv + C * E * 2;        // C x E
  uint8_t* sdn = sdo + C * E * 2;       // D x E  suffix state
  uint8_t* sds = sdn + D * E * 2;       // C x C  dS_m, then the staging tile of the epilogue
  uint8_t* sp = sds + C * C * 2;        // D x E  prefix state, then S_m (C x C)
  __shared__ uint64_t bar_in, bar_st, a_done, sm_ready, b_done, t_free;
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    dead = 0;
    mbar_init(&bar_in, 1);
    mbar_init(&bar_st, 1);
    mbar_init(&a_done, 1);
    mbar_init(&sm_ready, 256);
    mbar_init(&b_done, 1);
    mbar_init(&t_free, 256);
    fence_mbar_init();
  }
  if (warp == 2) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t t0 = tmem, t1 = tmem + 128, t2 = tmem + 256, t3 = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      int i = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
        const int bh = t / nc, chunk = t - bh * nc, row0 = bh * n + chunk * C;
        if (i >= 1) wait_or_fault(&b_done, (i - 1) & 1, &dead, kFaultMmaWait);  // every buffer of tile i-1 is read
        mbar_expect_tx(&bar_in, 2 * C * (D + E) * 2);
        tma_load_3d(sq, &map_q, &bar_in, 0, row0, 0);
        tma_load_3d(sk, &map_k, &bar_in, 0, row0, 0);
        tma_load_3d(sdo, &map_do, &bar_in, 0, row0, 0);
        tma_load_3d(sv, &map_v, &bar_in, 0, row0, 0);
        if constexpr (PDL) {
          // q, k, v, do are older than the chain of launches this kernel belongs to; the suffix states are
          // written by the scan just ahead: wait for it before the first state load
          if (i == 0) {
            grid_dependency_wait();
            grid_launch_dependents();
          }
        }
        mbar_expect_tx(&bar_st, 2 * D * E * 2);
        tma_load_3d(sp, &map_p, &bar_st, 0, (bh * nc + chunk) * D, 0);
        tma_load_3d(sdn, &map_dn, &bar_st, 0, (bh * nc + chunk) * D, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int i = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
        const uint32_t ph = i & 1;
        if (i >= 1) wait_or_fault(&t_free, (i - 1) & 1, &dead, kFaultMmaWait);  // epilogue of tile i-1 has drained T0..T3
        wait_or_fault(&bar_in, ph, &dead, kFaultTmaWait);
        tc_fence_after_sync();
        umma_gemm(t0, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sk), C, false}, C, D / 16, false);
        umma_gemm(t1, Operand{smem_u32(sdo), C, false}, Operand{smem_u32(sv), C, false}, C, E / 16, false);
        wait_or_fault(&bar_st, ph, &dead, kFaultTmaWait);
        tc_fence_after_sync();
        // state tiles as K-major B operands: rows = d (N), columns = e (K)
        umma_gemm(t2, Operand{smem_u32(sdo), C, false}, Operand{smem_u32(sp), D, false}, D, E / 16, false);
        umma_gemm(t3, Operand{smem_u32(sv), C, false}, Operand{smem_u32(sdn), D, false}, D, E / 16, false);
        umma_commit(&a_done);
        wait_or_fault(&sm_ready, ph, &dead, kFaultMmaWait);
        tc_fence_after_sync();
        umma_gemm(t2, Operand{smem_u32(sds), C, false}, Operand{smem_u32(sk), C, true}, D, C / 16, true);
        umma_gemm(t3, Operand{smem_u32(sds), C, true}, Operand{smem_u32(sq), C, true}, D, C / 16, true);
        umma_gemm(t0, Operand{smem_u32(sp), C, true}, Operand{smem_u32(sdo), C, true}, E, C / 16, false);
        umma_gemm(t1, Operand{smem_u32(sk), C, false}, Operand{smem_u32(sdn), D, true}, E, D / 16, false);
        umma_commit(&b_done);
      }
    }
  } else {
    const int cw = warp - 2;
    const int row = (warp & 3) * 32 + lane;
    const int half = cw >> 2;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const bool leader = (cw == 0 && lane == 0);
    int i = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++i) {
      const int bh = t / nc, chunk = t - bh * nc, row0 = bh * n + chunk * C;
      const uint32_t ph = i & 1;
      const float sl2 = s[bh % h] * kLog2e;
      const float lam = exp2f(-sl2);
      wait_or_fault(&a_done, ph, &dead, kFaultMmaWait);
      tc_fence_after_sync();
      // the previous tile's last store must have read the staging tile before dS_m lands in it
      if (leader) bulk_wait_read<0>();
      named_sync(1, 256);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col0 = half * 64 + cc * 32;
        masked_store32(t0 + lane_base + col0, sp, row, col0, sl2, lam);    // S_m over the prefix-state tile
        masked_store32(t1 + lane_base + col0, sds, row, col0, sl2, lam);   // dS_m
      }
      const float qd = decay_pow(sl2, row), kd = decay_pow(sl2, C - row);
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int col0 = half * (D / 2) + cc * 32;
        scale_tmem32(t2 + lane_base + col0, qd);
        scale_tmem32(t3 + lane_base + col0, kd);
      }
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&sm_ready);
      wait_or_fault(&b_done, ph, &dead, kFaultMmaWait);
      tc_fence_after_sync();
      // epilogue: three output tiles, one after the other through the staging tile
      if constexpr (PDL) {
        if (leader && i == 0) grid_dependency_wait();   // the outputs may still be read by a kernel ahead
      }
#pragma unroll
      for (int which = 0; which < 3; ++which) {
        if (which > 0) {
          if (leader) bulk_wait_read<0>();
          named_sync(1, 256);
        }
        const int width = which < 2 ? D : E;
        for (int cc = 0; cc < width / 64; ++cc) {
          const int col0 = half * (width / 2) + cc * 32;
          if (which == 0) stage_row32(t2 + lane_base + col0, 0xFFFFFFFFu, 0.f, sds, row, col0);
          else if (which == 1) stage_row32(t3 + lane_base + col0, 0xFFFFFFFFu, 0.f, sds, row, col0);
          else stage_row32(t0 + lane_base + col0, t1 + lane_base + col0, kd, sds, row, col0);
        }
        if (which == 2) {
          tc_fence_before_sync();
          mbar_arrive(&t_free);
        }
        fence_async_smem();
        named_sync(1, 256);
        if (leader) {
          tma_store_3d(which == 0 ? &map_dq : which == 1 ? &map_dk : &map_dv, sds, 0, row0, 0);
          bulk_commit();
        }
      }
    }
    if (leader) bulk_wait_all<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 512);
}


bool chunk_states_v2_enabled() {
  static const bool on = [] {
    const char* v = getenv("LASP_B200_CHUNK_STATES_V2");
    return v && v[0] == '1';
  }();
  return on;
}

// Launch with or without the programmatic-stream-serialization attribute (see grid_dependency_wait in sm100.cuh).
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool chained,
                   Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename F>
cudaError_t opt_in_smem(F* fn, size_t bytes) {
  cudaError_t err = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) g_failed_step = "cudaFuncSetAttribute(max dynamic shared memory)";
  return err;
}

cudaError_t tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t width, uint32_t box_rows,
                     const char* what) {
  cudaError_t err = make_tile_map(map, base, rows, width, box_rows);
  if (err != cudaSuccess) {
    static thread_local char text[160];
    snprintf(text, sizeof(text), "%s: CUresult %d, base %p, rows %llu, width %u, box rows %u", what,
             last_encode_result(), base, (unsigned long long)rows, width, box_rows);
    g_failed_step = text;
  }
  return err;
}

cudaError_t launched(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) g_failed_step = what;
  return err;
}

struct Maps {
  CUtensorMap m[6];
};

template <int D, int E>
cudaError_t launch_chunk_states(const Dims& m, const void* a, const void* bten, const float* s,
                                __nv_bfloat16* states, bool backward, bool chained, cudaStream_t st) {
  CUtensorMap ma, mb;
  const uint64_t rows = (uint64_t)m.b * m.h * m.n;
  cudaError_t err = tile_map(&ma, a, rows, D, C, "tensor map (chunk-state A)");
  if (err != cudaSuccess) return err;
  if ((err = tile_map(&mb, bten, rows, E, C, "tensor map (chunk-state B)")) != cudaSuccess) return err;
  const size_t smem = (size_t)C * (D + E) * 2 + 1024;
  if (chunk_states_v2_enabled() && !chained) {
    CUtensorMap mo;
    if ((err = tile_map(&mo, states, (uint64_t)m.b * m.h * m.nc * D, E, D, "tensor map (chunk states)")) != cudaSuccess)
      return err;
    const size_t smem2 = (size_t)(2 * C * (D + E) + D * E) * 2 + 1024;
    if ((err = opt_in_smem(k_tc_chunk_states_v2<D, E>, smem2)) != cudaSuccess) return err;
    const int tiles = m.nc * m.b * m.h;
    const int ctas = tiles < sm_count() ? tiles : sm_count();
    k_tc_chunk_states_v2<D, E><<<ctas, 320, smem2, st>>>(ma, mb, mo, s, m.h, m.n, m.nc, tiles, backward ? 1 : 0);
    return launched("launch of the persistent chunk-state kernel");
  }
  dim3 grid(m.nc, m.b * m.h);
  if (chained) {
    if ((err = opt_in_smem(k_tc_chunk_states<D, E, true>, smem)) != cudaSuccess) return err;
    if ((err = launch(k_tc_chunk_states<D, E, true>, grid, dim3(128), smem, st, true, ma, mb, s, states, m.h, m.n, m.nc,
                      backward ? 1 : 0)) != cudaSuccess) {
      g_failed_step = "launch of the chunk-state kernel";
      return err;
    }
    return launched("launch of the chunk-state kernel");
  }
  if ((err = opt_in_smem(k_tc_chunk_states<D, E, false>, smem)) != cudaSuccess) return err;
  k_tc_chunk_states<D, E, false><<<grid, 128, smem, st>>>(ma, mb, s, states, m.h, m.n, m.nc, backward ? 1 : 0);
  return cudaGetLastError();
}

template <int D, int E>
cudaError_t launch_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                              const __nv_bfloat16* prefix, void* o, bool chained, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mp;
  const uint64_t rows = (uint64_t)m.b * m.h * m.n;
  cudaError_t err;
  if ((err = tile_map(&mq, q, rows, D, C, "tensor map (q)")) != cudaSuccess) return err;
  if ((err = tile_map(&mk, k, rows, D, C, "tensor map (k)")) != cudaSuccess) return err;
  if ((err = tile_map(&mv, v, rows, E, C, "tensor map (v)")) != cudaSuccess) return err;
  if ((err = tile_map(&mp, prefix, (uint64_t)m.b * m.h * m.nc * D, E, D, "tensor map (prefix states)")) != cudaSuccess) return err;
  CUtensorMap mo;
  if ((err = tile_map(&mo, o, rows, E, C, "tensor map (o)")) != cudaSuccess) return err;
  const size_t smem = (size_t)(C * D + D * E + 2 * C * C + 3 * C * E) * 2 + 1024;
  const int tiles = m.nc * m.b * m.h;
  const int ctas = tiles < sm_count() ? tiles : sm_count();
  if (chained) {
    if ((err = opt_in_smem(k_tc_fwd_output<D, E, true>, smem)) != cudaSuccess) return err;
    if ((err = launch(k_tc_fwd_output<D, E, true>, dim3(ctas), dim3(320), smem, st, true, mq, mk, mv, mp, mo, s, m.h, m.n,
                      m.nc, tiles)) != cudaSuccess) {
      g_failed_step = "launch of the forward output kernel";
      return err;
    }
    return launched("launch of the forward output kernel");
  }
  if ((err = opt_in_smem(k_tc_fwd_output<D, E, false>, smem)) != cudaSuccess) return err;
  k_tc_fwd_output<D, E, false><<<ctas, 320, smem, st>>>(mq, mk, mv, mp, mo, s, m.h, m.n, m.nc, tiles);
  return launched("launch of the forward output kernel");
}

template <int D, int E>
cudaError_t launch_bwd_grads(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                             const float* s, const __nv_bfloat16* prefix, const __nv_bfloat16* suffix, void* dq,
                             void* dk, void* dv, bool chained, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mdo, mp, mdn;
  const uint64_t rows = (uint64_t)m.b * m.h * m.n;
  const uint64_t srows = (uint64_t)m.b * m.h * m.nc * D;
  cudaError_t err;
  if ((err = tile_map(&mq, q, rows, D, C, "tensor map (q)")) != cudaSuccess) return err;
  if ((err = tile_map(&mk, k, rows, D, C, "tensor map (k)")) != cudaSuccess) return err;
  if ((err = tile_map(&mv, v, rows, E, C, "tensor map (v)")) != cudaSuccess) return err;
  if ((err = tile_map(&mdo, d_o, rows, E, C, "tensor map (do)")) != cudaSuccess) return err;
  if ((err = tile_map(&mp, prefix, srows, E, D, "tensor map (prefix states)")) != cudaSuccess) return err;
  if ((err = tile_map(&mdn, suffix, srows, E, D, "tensor map (suffix states)")) != cudaSuccess) return err;
  CUtensorMap mdq, mdk, mdv;
  if ((err = tile_map(&mdq, dq, rows, D, C, "tensor map (dq)")) != cudaSuccess) return err;
  if ((err = tile_map(&mdk, dk, rows, D, C, "tensor map (dk)")) != cudaSuccess) return err;
  if ((err = tile_map(&mdv, dv, rows, E, C, "tensor map (dv)")) != cudaSuccess) return err;
  // Q, K, V, dO, Dn, dS_m, and the larger of P / S_m
  const size_t last = (size_t)(D * E > C * C ? D * E : C * C) * 2;
  const size_t smem = (size_t)(2 * C * D + 2 * C * E + D * E + C * C) * 2 + last + 1024;
  const int tiles = m.nc * m.b * m.h;
  const int ctas = tiles < sm_count() ? tiles : sm_count();
  if (chained) {
    if ((err = opt_in_smem(k_tc_bwd_grads<D, E, true>, smem)) != cudaSuccess) return err;
    if ((err = launch(k_tc_bwd_grads<D, E, true>, dim3(ctas), dim3(320), smem, st, true, mq, mk, mv, mdo, mp, mdn, mdq,
                      mdk, mdv, s, m.h, m.n, m.nc, tiles)) != cudaSuccess) {
      g_failed_step = "launch of the backward gradient kernel";
      return err;
    }
    return launched("launch of the backward gradient kernel");
  }
  if ((err = opt_in_smem(k_tc_bwd_grads<D, E, false>, smem)) != cudaSuccess) return err;
  k_tc_bwd_grads<D, E, false><<<ctas, 320, smem, st>>>(mq, mk, mv, mdo, mp, mdn, mdq, mdk, mdv, s, m.h, m.n, m.nc, tiles);
  return launched("launch of the backward gradient kernel");
}

}  // namespace

// the per-tile kernels of this file: full tiles only
bool tensor_tile_path_supported(const Dims& m) {
  const bool dims_ok = (m.d == 64 || m.d == 128) && (m.e == 64 || m.e == 128);
  return m.dtype == LASP_BF16 && dims_ok && m.n % C == 0 && (long long)m.b * m.h * m.n < (1LL << 31);
}

#define LASP_DISPATCH_DE(m, CALL)                                        \
  do {                                                                    \
    if ((m).d == 128 && (m).e == 128) return CALL(128, 128);              \
    if ((m).d == 128 && (m).e == 64) return CALL(128, 64);                \
    if ((m).d == 64 && (m).e == 128) return CALL(64, 128);                \
    if ((m).d == 64 && (m).e == 64) return CALL(64, 64);                  \
    return cudaErrorInvalidValue;                                         \
  } while (0)

cudaError_t tensor_chunk_states(const Dims& m, const void* a, const void* bten, const float* s,
                                __nv_bfloat16* states, bool backward, bool chained, cudaStream_t st) {
#define LASP_CALL(DD, EE) launch_chunk_states<DD, EE>(m, a, bten, s, states, backward, chained, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

cudaError_t tensor_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                              const __nv_bfloat16* prefix, void* o, bool chained, cudaStream_t st) {
#define LASP_CALL(DD, EE) launch_fwd_output<DD, EE>(m, q, k, v, s, prefix, o, chained, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

cudaError_t tensor_bwd_grads(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                             const float* s, const __nv_bfloat16* prefix, const __nv_bfloat16* suffix, void* dq,
                             void* dk, void* dv, bool chained, cudaStream_t st) {
#define LASP_CALL(DD, EE) launch_bwd_grads<DD, EE>(m, q, k, v, d_o, s, prefix, suffix, dq, dk, dv, chained, st)
  LASP_DISPATCH_DE(m, LASP_CALL);
#undef LASP_CALL
}

}  // namespace lasp
