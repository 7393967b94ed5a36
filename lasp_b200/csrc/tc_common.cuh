// Device helpers shared by the tensor-core kernels: bounded waits that report
// through the fault word, accumulator <-> shared-memory moves with the decay
// mask, and the enumeration of the tiles a persistent CTA walks over.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace lasp {
namespace tc {

using namespace sm100;

constexpr int C = kTensorTile;  // 128 tokens per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kNoAcc = 0xFFFFFFFFu;

// bounded wait that records a fault once and makes later waits of the CTA no-ops
__device__ __forceinline__ void wait_or_fault(uint64_t* bar, uint32_t parity, volatile int* dead, int32_t* fault,
                                              int32_t code) {
  if (*dead) return;
  if (!mbar_wait(bar, parity)) {
    *dead = 1;
    atomicOr(fault, code);
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

__device__ __forceinline__ float decay_pow(float sl2, int k) { return exp2f(-sl2 * (float)k); }

// acc (32 columns) *= f, in tensor memory
__device__ __forceinline__ void scale_tmem32(uint32_t taddr, float f) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
  tmem_st32(taddr, r);
}

// tile[row][col0 .. col0+31] = bf16(acc1 + f * acc2) into a swizzled staging tile of C rows
// (acc2 skipped when taddr2 == kNoAcc); a TMA store then moves the tile out
__device__ __forceinline__ void stage_row32(uint32_t taddr1, uint32_t taddr2, float f, uint8_t* tile, int row,
                                            int col0) {
  uint32_t a[32];
  tmem_ld32(taddr1, a);
  if (taddr2 != kNoAcc) {
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

// Tensor-memory accumulator (32 columns at `taddr`, this thread's lane = row) ->
// decay-masked bf16 in a K-major swizzled tile:
//   out[row][col] = [row >= col] lambda^(row-col) acc[col].
// Per group of eight columns the factor is built from the group's right-most unmasked column
// leftwards by repeated multiplication with lambda (short independent chains), so it can only
// underflow towards the far columns.  The 32 rows of a warp are `row0 .. row0+31`: groups wholly
// below the diagonal for every row of the warp need no comparisons, groups wholly above it are zero.
// `pre` multiplies every element (the folded q,k scale).
__device__ __forceinline__ void masked_store32(uint32_t taddr, uint8_t* tile, int row, int col0, float sl2,
                                               float lam, float pre = 1.f) {
  const int row0 = row & ~31;
  if (col0 > row0 + 31) {   // the whole block is above the diagonal (same for every lane of the warp)
#pragma unroll
    for (int g = 0; g < 4; ++g)
      *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + 8 * g, C)) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  uint32_t r[32];
  tmem_ld32(taddr, r);
  float f[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) f[g] = pre * decay_pow(sl2, row - min(row, col0 + 8 * g + 7));
  tmem_ld_wait();
  if (col0 + 31 <= row0) {  // the whole block is below the diagonal
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float m[8];
#pragma unroll
      for (int j = 7; j >= 0; --j) {
        m[j] = __uint_as_float(r[8 * g + j]) * f[g];
        f[g] *= lam;
      }
      *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + 8 * g, C)) =
          make_uint4(pack_bf16(m[0], m[1]), pack_bf16(m[2], m[3]), pack_bf16(m[4], m[5]), pack_bf16(m[6], m[7]));
    }
    return;
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float m[8];
#pragma unroll
    for (int j = 7; j >= 0; --j) {
      const bool live = (col0 + 8 * g + j) <= row;
      m[j] = live ? __uint_as_float(r[8 * g + j]) * f[g] : 0.f;
      f[g] = live ? f[g] * lam : f[g];
    }
    *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + 8 * g, C)) =
        make_uint4(pack_bf16(m[0], m[1]), pack_bf16(m[2], m[3]), pack_bf16(m[4], m[5]), pack_bf16(m[6], m[7]));
  }
}

// The same mask, but the result stays in tensor memory as the A operand of the next MMA: 32 fp32
// columns at `src` (columns col0 .. col0+31 of the score tile) become 16 columns of bf16 pairs at `dst`.
// TRANSPOSED = false: lane = query row r, column = key c:  [r >= c] lambda^(r-c)
// TRANSPOSED = true : lane = key c, column = query row r:  [r >= c] lambda^(r-c)   (the tile is S^T)
template <bool TRANSPOSED>
__device__ __forceinline__ void masked_pack32(uint32_t src, int row, int col0, float sl2, float lam,
                                              uint32_t (&out)[16], float pre = 1.f) {
  const int row0 = row & ~31;
  const bool none = TRANSPOSED ? (col0 + 31 < row0) : (col0 > row0 + 31);   // same for every lane of the warp
  if (none) {
#pragma unroll
    for (int j = 0; j < 16; ++j) out[j] = 0u;
    return;
  }
  uint32_t r[32];
  tmem_ld32(src, r);
  float f[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    // the chain of a group of eight columns starts at its live column nearest the diagonal
    const int start = TRANSPOSED ? max(row, col0 + 8 * g) : min(row, col0 + 8 * g + 7);
    f[g] = pre * decay_pow(sl2, TRANSPOSED ? start - row : row - start);
  }
  tmem_ld_wait();
  const bool all = TRANSPOSED ? (col0 >= row0 + 31) : (col0 + 31 <= row0);
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float m[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int j = TRANSPOSED ? jj : 7 - jj;           // away from the diagonal
      const int col = col0 + 8 * g + j;
      const bool live = all || (TRANSPOSED ? col >= row : col <= row);
      m[j] = live ? __uint_as_float(r[8 * g + j]) * f[g] : 0.f;
      f[g] = live ? f[g] * lam : f[g];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) out[4 * g + j] = pack_bf16(m[2 * j], m[2 * j + 1]);
  }
}

// exp of a pair of bf16 values: the argument is scaled in fp32, the exponential itself is ONE special-function
// operation for the pair (the map passes are bound by that unit)
__device__ __forceinline__ __nv_bfloat162 exp_bf16x2(uint32_t u) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
  const uint32_t t = pack_bf16(f.x * kLog2e, f.y * kLog2e);
  uint32_t r;
  asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(r) : "r"(t));
  return *reinterpret_cast<__nv_bfloat162*>(&r);
}
// elu(x) + 1 on a pair of bf16 values (the feature map of the no-decay linear-transformer configuration):
// x + 1 for x > 0, exp(x) otherwise = max(x, 0) + min(exp(x), 1), without a branch
__device__ __forceinline__ uint32_t elu1_bf16x2(uint32_t u) {
  const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&u);
  const __nv_bfloat162 r = __hadd2(__hmax2(x, __float2bfloat162_rn(0.f)), __hmin2(exp_bf16x2(u), __float2bfloat162_rn(1.f)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
// its derivative: 1 for x > 0, exp(x) otherwise = min(exp(x), 1)
__device__ __forceinline__ float2 elu1_slope_bf16x2(uint32_t u) {
  return __bfloat1622float2(__hmin2(exp_bf16x2(u), __float2bfloat162_rn(1.f)));
}

// Multiplies CHUNKS 16-byte pieces of row `row` of a swizzled tile of C rows by w, in place, starting
// at piece `first` (pieces are counted slab by slab; a row keeps its pieces under the swizzle, so the
// physical position inside the row does not matter).  `lane` rotates the order to spread the banks.
// MAP: each element goes through elu(x) + 1 first.
template <int CHUNKS, bool MAP = false>
__device__ __forceinline__ void scale_row_pieces(uint8_t* tile, int row, int first, float w, int lane) {
  static_assert((CHUNKS & (CHUNKS - 1)) == 0, "a power of two");
  uint4 v[CHUNKS];
  uint4* p[CHUNKS];
#pragma unroll
  for (int q = 0; q < CHUNKS; ++q) {   // all loads first: their latencies overlap
    const int piece = first + ((q + lane) & (CHUNKS - 1));
    p[q] = reinterpret_cast<uint4*>(tile + (piece >> 3) * C * 128 + row * 128 + (piece & 7) * 16);
    v[q] = *p[q];
  }
#pragma unroll
  for (int q = 0; q < CHUNKS; ++q) {
    uint32_t* u = reinterpret_cast<uint32_t*>(&v[q]);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (MAP) u[t] = elu1_bf16x2(u[t]);
      if (!MAP || w != 1.f) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u[t]));
        u[t] = pack_bf16(f.x * w, f.y * w);
      }
    }
    *p[q] = v[q];
  }
}

// stage_row32 with the chain rule of the folded q,k preprocessing x' = c * map(x): the 32 accumulator values
// (a gradient with respect to x') are multiplied by c * map'(x) on their way to the staging tile, x read from
// the raw tensor (`raw` points at column 0 of this thread's row).
__device__ __forceinline__ void stage_row32_chain(uint32_t taddr, uint8_t* tile, int row, int col0,
                                                  const __nv_bfloat16* raw, float c, bool elu) {
  uint4 x[4];
  if (elu) {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = __ldg(reinterpret_cast<const uint4*>(raw + col0) + j);
  }
  uint32_t a[32];
  tmem_ld32(taddr, a);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float m[8];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float sx = c, sy = c;
      if (elu) {
        const float2 sl = elu1_slope_bf16x2(reinterpret_cast<const uint32_t*>(&x[j])[t]);
        sx *= sl.x, sy *= sl.y;
      }
      m[2 * t] = __uint_as_float(a[8 * j + 2 * t]) * sx;
      m[2 * t + 1] = __uint_as_float(a[8 * j + 2 * t + 1]) * sy;
    }
    *reinterpret_cast<uint4*>(tile + tile_offset(row, col0 + 8 * j, C)) =
        make_uint4(pack_bf16(m[0], m[1]), pack_bf16(m[2], m[3]), pack_bf16(m[4], m[5]), pack_bf16(m[6], m[7]));
  }
}

// The work of a persistent CTA: items blockIdx.x, blockIdx.x + gridDim.x, ...; an item is one span of
// consecutive tiles of one (batch, head) sequence, walked first to last tile or last to first.
// Spans: `span` tiles each, the last one of a sequence whatever is left (even = false), or - for a
// kernel whose CTAs wait for one another - the tiles shared out evenly, spans differing by one tile at
// most, with the longer spans where the walk starts: there nobody has to wait for anybody's total, and the
// spans with the longest look-back get the fewest tiles (even = true).
struct TileWalk {
  int items, nspans, span, tiles, stride;
  bool backwards;
  bool even;
  int it, bh, t, t0, t1;  // current item, its sequence, current tile, the item's tile range [t0, t1)

  // first tile of span sp (sp = nspans: one past the last tile)
  __device__ __forceinline__ int span_t0(int sp) const {
    if (!even) return min(sp * span, tiles);
    const int base = tiles / nspans, extra = tiles - base * nspans;   // `extra` spans have base + 1 tiles
    return backwards ? sp * base + max(0, sp - (nspans - extra)) : sp * base + min(sp, extra);
  }
  __device__ __forceinline__ bool load() {
    if (it >= items) return false;
    bh = it / nspans;
    const int sp = it - bh * nspans;
    t0 = span_t0(sp);
    t1 = span_t0(sp + 1);
    t = backwards ? t1 - 1 : t0;
    return true;
  }
  __device__ __forceinline__ bool start(int first_item, int item_stride) {
    it = first_item;
    stride = item_stride;
    return load();
  }
  __device__ __forceinline__ bool next() {
    if (backwards ? (--t >= t0) : (++t < t1)) return true;
    it += stride;
    return load();
  }
  __device__ __forceinline__ bool first_of_item() const { return backwards ? t == t1 - 1 : t == t0; }
  __device__ __forceinline__ bool last_of_item() const { return backwards ? t == t0 : t == t1 - 1; }
};

}  // namespace tc
}  // namespace lasp
