// Tensor-core path: tcgen05 MMAs with accumulators in tensor memory, operands
// staged in shared memory by TMA.  bf16 inputs, fp32 accumulation, one rounding
// on store.  One CTA owns one 128-token chunk of one (batch, head).
//
// Every tile in shared memory is in the swizzled slab format of sm100.cuh, so a
// tile loaded once serves both as a K-major operand (rows = M/N) and as an
// MN-major operand (rows = K).  The decay mask is applied between MMAs on the
// way from tensor memory back to shared memory (S -> S_m as bf16).
//
// All waits are bounded; a wait that runs out sets a bit in g_fault_word and the
// CTA skips its remaining waits, frees its tensor memory and exits.
#include <stdio.h>

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

namespace {

using namespace sm100;

constexpr int C = kTensorChunk;  // 128 tokens per tile

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

// tab[i] = exp(-s i), i = 0..C
__device__ __forceinline__ void fill_decay_table(float* tab, float s) {
  for (int i = threadIdx.x; i <= C; i += blockDim.x) tab[i] = expf(-s * (float)i);
}

// Tensor-memory accumulator (32 columns at `taddr` for this thread's lane) ->
// decay-masked bf16 in a K-major swizzled tile: out[row][col0+j] = [row >= col] tab[row-col] acc.
__device__ __forceinline__ void masked_store32(uint32_t taddr, uint8_t* tile, int row, int col0, const float* tab) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint32_t pk[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int c0 = col0 + j + 2 * t, c1 = c0 + 1;
      const float a = (row >= c0) ? __uint_as_float(r[j + 2 * t]) * tab[row - c0] : 0.f;
      const float b = (row >= c1) ? __uint_as_float(r[j + 2 * t + 1]) * tab[row - c1] : 0.f;
      pk[t] = pack_bf16(a, b);
    }
    *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + j, C)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
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

// ---------------------------------------------------------------------------
// chunk states: out[i][j] = sum_c w_c A[c][i] B[c][j]   (A = K or Q, B = V or dO)
// ---------------------------------------------------------------------------
template <int D, int E>
__global__ void __launch_bounds__(128) k_tc_chunk_states(const __grid_constant__ CUtensorMap map_a,
                                                         const __grid_constant__ CUtensorMap map_b,
                                                         const float* __restrict__ s, float* __restrict__ states,
                                                         int h, int n, int nc, int backward) {
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
    float* out = states + ((size_t)bh * nc + chunk) * D * E + (size_t)tid * E;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll
    for (int c0 = 0; c0 < E; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<uint4*>(out + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// ---------------------------------------------------------------------------
// forward output: O = S_m V + diag(lambda^r) Q P
// ---------------------------------------------------------------------------
template <int D, int E>
__global__ void __launch_bounds__(256) k_tc_fwd_output(const __grid_constant__ CUtensorMap map_q,
                                                       const __grid_constant__ CUtensorMap map_k,
                                                       const __grid_constant__ CUtensorMap map_v,
                                                       const __grid_constant__ CUtensorMap map_p,
                                                       const float* __restrict__ s, __nv_bfloat16* __restrict__ O,
                                                       int h, int n, int nc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sq = smem;                  // C x D
  uint8_t* sv = sq + C * D * 2;        // C x E
  uint8_t* sp = sv + C * E * 2;        // D x E
  uint8_t* sk = sp + D * E * 2;        // C x D, then S_m (C x C) - kept last and sized for the larger
  __shared__ uint64_t bar_qk, bar_vp, bar_s, bar_o;
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  __shared__ float tab[C + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const float sh = s[bh % h];
  if (tid == 0) {
    dead = 0;
    mbar_init(&bar_qk, 1);
    mbar_init(&bar_vp, 1);
    mbar_init(&bar_s, 1);
    mbar_init(&bar_o, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  fill_decay_table(tab, sh);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t t_s = tmem, t_o2 = tmem + 128, t_o1 = tmem + 256;
  const int row0 = bh * n + chunk * C;
  if (tid == 0) {
    mbar_expect_tx(&bar_qk, 2 * C * D * 2);
    tma_load_3d(sq, &map_q, &bar_qk, 0, row0, 0);
    tma_load_3d(sk, &map_k, &bar_qk, 0, row0, 0);
    mbar_expect_tx(&bar_vp, (C * E + D * E) * 2);
    tma_load_3d(sv, &map_v, &bar_vp, 0, row0, 0);
    tma_load_3d(sp, &map_p, &bar_vp, 0, (bh * nc + chunk) * D, 0);
    wait_or_fault(&bar_qk, 0, &dead, kFaultTmaWait);
    if (!dead) {
      tc_fence_after_sync();
      umma_gemm(t_s, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sk), C, false}, C, D / 16, false);
      umma_commit(&bar_s);
    }
    wait_or_fault(&bar_vp, 0, &dead, kFaultTmaWait);
    if (!dead) {
      tc_fence_after_sync();
      umma_gemm(t_o2, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sp), D, true}, E, D / 16, false);
    }
  }
  __syncwarp();
  wait_or_fault(&bar_s, 0, &dead, kFaultMmaWait);
  tc_fence_after_sync();
  const int row = (warp & 3) * 32 + lane;
  const int half = warp >> 2;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  // S -> S_m (bf16) over the K tile
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int col0 = half * 64 + cc * 32;
    masked_store32(t_s + lane_base + col0, sk, row, col0, tab);
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && !dead) {
    tc_fence_after_sync();
    umma_gemm(t_o1, Operand{smem_u32(sk), C, false}, Operand{smem_u32(sv), C, true}, E, C / 16, false);
    umma_commit(&bar_o);
  }
  __syncwarp();
  wait_or_fault(&bar_o, 0, &dead, kFaultMmaWait);
  tc_fence_after_sync();
  {
    __nv_bfloat16* out_row = O + (size_t)(row0 + row) * E;
    const float qd = tab[row];
#pragma unroll
    for (int cc = 0; cc < E / 64; ++cc) {
      const int col0 = half * (E / 2) + cc * 32;
      store_row32(t_o1 + lane_base + col0, t_o2 + lane_base + col0, qd, out_row, col0);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// backward: dQ = dS_m K + diag(lambda^r) dO P^T
//           dK = dS_m^T Q + diag(lambda^(C-c)) V Dn^T
//           dV = S_m^T dO + diag(lambda^(C-c)) K Dn
// ---------------------------------------------------------------------------
template <int D, int E>
__global__ void __launch_bounds__(256) k_tc_bwd_grads(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
    const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_dn,
    const float* __restrict__ s, __nv_bfloat16* __restrict__ DQ, __nv_bfloat16* __restrict__ DK,
    __nv_bfloat16* __restrict__ DV, int h, int n, int nc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sq = smem;                   // C x D
  uint8_t* sk = sq + C * D * 2;         // C x D
  uint8_t* sv = sk + C * D * 2;         // C x E
  uint8_t* sdo = sv + C * E * 2;        // C x E
  uint8_t* sdn = sdo + C * E * 2;       // D x E  suffix state
  uint8_t* sds = sdn + D * E * 2;       // C x C  dS_m
  uint8_t* sp = sds + C * C * 2;        // D x E  prefix state, then S_m (C x C)
  __shared__ uint64_t bar_in, bar_st, bar_a, bar_b;
  __shared__ uint32_t tmem_slot;
  __shared__ int dead;
  __shared__ float tab[C + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const float sh = s[bh % h];
  if (tid == 0) {
    dead = 0;
    mbar_init(&bar_in, 1);
    mbar_init(&bar_st, 1);
    mbar_init(&bar_a, 1);
    mbar_init(&bar_b, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  fill_decay_table(tab, sh);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t t0 = tmem, t1 = tmem + 128, t2 = tmem + 256, t3 = tmem + 384;
  const int row0 = bh * n + chunk * C;
  if (tid == 0) {
    mbar_expect_tx(&bar_in, 2 * C * (D + E) * 2);
    tma_load_3d(sq, &map_q, &bar_in, 0, row0, 0);
    tma_load_3d(sk, &map_k, &bar_in, 0, row0, 0);
    tma_load_3d(sv, &map_v, &bar_in, 0, row0, 0);
    tma_load_3d(sdo, &map_do, &bar_in, 0, row0, 0);
    mbar_expect_tx(&bar_st, 2 * D * E * 2);
    tma_load_3d(sp, &map_p, &bar_st, 0, (bh * nc + chunk) * D, 0);
    tma_load_3d(sdn, &map_dn, &bar_st, 0, (bh * nc + chunk) * D, 0);
    wait_or_fault(&bar_in, 0, &dead, kFaultTmaWait);
    if (!dead) {
      tc_fence_after_sync();
      // S = Q K^T, dS = dO V^T
      umma_gemm(t0, Operand{smem_u32(sq), C, false}, Operand{smem_u32(sk), C, false}, C, D / 16, false);
      umma_gemm(t1, Operand{smem_u32(sdo), C, false}, Operand{smem_u32(sv), C, false}, C, E / 16, false);
    }
    wait_or_fault(&bar_st, 0, &dead, kFaultTmaWait);
    if (!dead) {
      tc_fence_after_sync();
      // dQ2 = dO P^T, dK2 = V Dn^T   (state tiles as K-major B operands: rows = d, K = e)
      umma_gemm(t2, Operand{smem_u32(sdo), C, false}, Operand{smem_u32(sp), D, false}, D, E / 16, false);
      umma_gemm(t3, Operand{smem_u32(sv), C, false}, Operand{smem_u32(sdn), D, false}, D, E / 16, false);
      umma_commit(&bar_a);
    }
  }
  __syncwarp();
  wait_or_fault(&bar_a, 0, &dead, kFaultMmaWait);
  tc_fence_after_sync();
  const int row = (warp & 3) * 32 + lane;
  const int half = warp >> 2;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int col0 = half * 64 + cc * 32;
    masked_store32(t0 + lane_base + col0, sp, row, col0, tab);    // S_m over the prefix-state tile
    masked_store32(t1 + lane_base + col0, sds, row, col0, tab);   // dS_m
  }
  {
    const float qd = tab[row], kd = tab[C - row];
#pragma unroll
    for (int cc = 0; cc < D / 64; ++cc) {
      const int col0 = half * (D / 2) + cc * 32;
      scale_tmem32(t2 + lane_base + col0, qd);
      scale_tmem32(t3 + lane_base + col0, kd);
    }
    tmem_st_wait();
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && !dead) {
    tc_fence_after_sync();
    // dQ += dS_m K ; dK += dS_m^T Q ; dV1 = S_m^T dO ; dV2 = K Dn
    umma_gemm(t2, Operand{smem_u32(sds), C, false}, Operand{smem_u32(sk), C, true}, D, C / 16, true);
    umma_gemm(t3, Operand{smem_u32(sds), C, true}, Operand{smem_u32(sq), C, true}, D, C / 16, true);
    umma_gemm(t0, Operand{smem_u32(sp), C, true}, Operand{smem_u32(sdo), C, true}, E, C / 16, false);
    umma_gemm(t1, Operand{smem_u32(sk), C, false}, Operand{smem_u32(sdn), D, true}, E, D / 16, false);
    umma_commit(&bar_b);
  }
  __syncwarp();
  wait_or_fault(&bar_b, 0, &dead, kFaultMmaWait);
  tc_fence_after_sync();
  {
    const float kd = tab[C - row];
    __nv_bfloat16* dq_row = DQ + (size_t)(row0 + row) * D;
    __nv_bfloat16* dk_row = DK + (size_t)(row0 + row) * D;
    __nv_bfloat16* dv_row = DV + (size_t)(row0 + row) * E;
#pragma unroll
    for (int cc = 0; cc < D / 64; ++cc) {
      const int col0 = half * (D / 2) + cc * 32;
      store_row32(t2 + lane_base + col0, 0xFFFFFFFFu, 0.f, dq_row, col0);
      store_row32(t3 + lane_base + col0, 0xFFFFFFFFu, 0.f, dk_row, col0);
    }
#pragma unroll
    for (int cc = 0; cc < E / 64; ++cc) {
      const int col0 = half * (E / 2) + cc * 32;
      store_row32(t0 + lane_base + col0, t1 + lane_base + col0, kd, dv_row, col0);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
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
cudaError_t launch_chunk_states(const Dims& m, const void* a, const void* bten, const float* s, float* states,
                                bool backward, cudaStream_t st) {
  CUtensorMap ma, mb;
  const uint64_t rows = (uint64_t)m.b * m.h * m.n;
  cudaError_t err = tile_map(&ma, a, rows, D, C, "tensor map (chunk-state A)");
  if (err != cudaSuccess) return err;
  if ((err = tile_map(&mb, bten, rows, E, C, "tensor map (chunk-state B)")) != cudaSuccess) return err;
  const size_t smem = (size_t)C * (D + E) * 2 + 1024;
  if ((err = opt_in_smem(k_tc_chunk_states<D, E>, smem)) != cudaSuccess) return err;
  dim3 grid(m.nc, m.b * m.h);
  k_tc_chunk_states<D, E><<<grid, 128, smem, st>>>(ma, mb, s, states, m.h, m.n, m.nc, backward ? 1 : 0);
  return cudaGetLastError();
}

template <int D, int E>
cudaError_t launch_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                              const __nv_bfloat16* prefix, void* o, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mp;
  const uint64_t rows = (uint64_t)m.b * m.h * m.n;
  cudaError_t err;
  if ((err = tile_map(&mq, q, rows, D, C, "tensor map (q)")) != cudaSuccess) return err;
  if ((err = tile_map(&mk, k, rows, D, C, "tensor map (k)")) != cudaSuccess) return err;
  if ((err = tile_map(&mv, v, rows, E, C, "tensor map (v)")) != cudaSuccess) return err;
  if ((err = tile_map(&mp, prefix, (uint64_t)m.b * m.h * m.nc * D, E, D, "tensor map (prefix states)")) != cudaSuccess) return err;
  const size_t smem = (size_t)(C * D + C * E + D * E + C * C) * 2 + 1024;
  if ((err = opt_in_smem(k_tc_fwd_output<D, E>, smem)) != cudaSuccess) return err;
  dim3 grid(m.nc, m.b * m.h);
  k_tc_fwd_output<D, E><<<grid, 256, smem, st>>>(mq, mk, mv, mp, s, (__nv_bfloat16*)o, m.h, m.n, m.nc);
  return launched("launch of the forward output kernel");
}

template <int D, int E>
cudaError_t launch_bwd_grads(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                             const float* s, const __nv_bfloat16* prefix, const __nv_bfloat16* suffix, void* dq,
                             void* dk, void* dv, cudaStream_t st) {
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
  // Q, K, V, dO, Dn, dS_m, and the larger of P / S_m
  const size_t last = (size_t)(D * E > C * C ? D * E : C * C) * 2;
  const size_t smem = (size_t)(2 * C * D + 2 * C * E + D * E + C * C) * 2 + last + 1024;
  if ((err = opt_in_smem(k_tc_bwd_grads<D, E>, smem)) != cudaSuccess) return err;
  dim3 grid(m.nc, m.b * m.h);
  k_tc_bwd_grads<D, E><<<grid, 256, smem, st>>>(mq, mk, mv, mdo, mp, mdn, s, (__nv_bfloat16*)dq, (__nv_bfloat16*)dk,
                                                (__nv_bfloat16*)dv, m.h, m.n, m.nc);
  return launched("launch of the backward gradient kernel");
}

}  // namespace

bool tensor_path_supported(const Dims& m) {
  return m.dtype == LASP_BF16 && m.d == 128 && m.e == 128 && m.n % C == 0 &&
         (long long)m.b * m.h * m.n < (1LL << 31);
}

cudaError_t tensor_chunk_states(const Dims& m, const void* a, const void* bten, const float* s, float* states,
                                bool backward, cudaStream_t st) {
  return launch_chunk_states<128, 128>(m, a, bten, s, states, backward, st);
}

cudaError_t tensor_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                              const __nv_bfloat16* prefix, void* o, cudaStream_t st) {
  return launch_fwd_output<128, 128>(m, q, k, v, s, prefix, o, st);
}

cudaError_t tensor_bwd_grads(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                             const float* s, const __nv_bfloat16* prefix, const __nv_bfloat16* suffix, void* dq,
                             void* dk, void* dv, cudaStream_t st) {
  return launch_bwd_grads<128, 128>(m, q, k, v, d_o, s, prefix, suffix, dq, dk, dv, st);
}

}  // namespace lasp
