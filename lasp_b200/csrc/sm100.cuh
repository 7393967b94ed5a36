// Blackwell (sm_100a) primitives used by the tensor-core kernels: mbarriers with
// bounded waits, TMA tile loads, tensor-memory allocation, tcgen05 MMA issue,
// commit and tensor-memory loads/stores, plus the host-side tensor-map builder.
// Everything is inline PTX; nothing here loads with a cluster-wide broadcast.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lasp {
namespace sm100 {

// ---------------------------------------------------------------------------
// shared-memory tile format
// ---------------------------------------------------------------------------
// A bf16 tile of R rows x W columns (W = 64 or 128) is held as W/64 slabs; a
// slab is R rows of 128 bytes (64 elements) with the 128-byte swizzle: the
// 16-byte chunk j of row r sits at chunk (j ^ (r & 7)).  Slabs start on 1024 B.
// This is what one 3-D TMA box {64, R, W/64} writes, and it is a canonical
// tcgen05 operand layout in two ways:
//   * "K-major"  : rows are the M (or N) index, columns the K index;
//   * "MN-major" : rows are the K index, columns the M (or N) index.
constexpr uint32_t kSlabRowBytes = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of element (row, col) inside a swizzled tile of R rows
__device__ __forceinline__ uint32_t tile_offset(uint32_t row, uint32_t col, uint32_t rows) {
  const uint32_t slab = col >> 6, chunk = (col & 63) >> 3, within = (col & 7) * 2;
  return slab * rows * kSlabRowBytes + row * kSlabRowBytes + (((chunk ^ (row & 7)) << 4) | within);
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// non-blocking probe of a phase (try_wait may suspend the thread for a while; this never does)
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~1e9 clocks (about half a second) and returns
// false, so a lost arrival becomes a reported fault instead of a hung GPU.
constexpr long long kWaitClocks = 1000000000LL;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitClocks) return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// TMA: 3-D tiled load global -> shared, completion counted on an mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// 3-D tiled store shared -> global (bulk async group of the issuing thread)
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// 4-D forms: coordinates {element, token, 64-column slab, sequence}.  Rows past the end of a sequence read
// as zero and are not written, so a ragged last tile needs no special case.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest `pending` store groups of this thread have finished READING shared memory
template <int pending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(pending) : "memory");
}
// ... have completed entirely (writes visible)
template <int pending>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(pending) : "memory");
}
// named barrier over `count` threads (count a multiple of 32); id 1..15
__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------
// warp-collective; ncols a power of two in [32, 512]; the address lands in *slot (shared memory)
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// tcgen05.mma (bf16 x bf16 -> fp32, M = 128, one CTA)
// ---------------------------------------------------------------------------
// shared-memory matrix descriptor, 128-byte swizzle.  lbo/sbo in bytes:
//   K-major : sbo = stride between 8-row groups (1024); lbo unused (16)
//   MN-major: lbo = stride between 64-element column slabs; sbo = stride between 8-row (K) groups (1024)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  d |= (uint64_t)2 << 61;  // 128-byte swizzle
  return d;
}
// instruction descriptor: fp32 accumulate, bf16 A and B, dense
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}
// one MMA of shape M x N x 16; accumulate = 0 overwrites the accumulator
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory: lane = row of A, and each 32-bit column holds two
// consecutive K elements (bf16), so one instruction (16 K elements) reads 8 columns from a_tmem on.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Operand views of a swizzled tile (see the tile format above).
struct Operand {
  uint32_t addr;   // shared address of the tile
  uint32_t rows;   // rows of the tile (slab stride = rows * 128 bytes)
  bool mn_major;   // false: rows = M/N index, cols = K;  true: rows = K index, cols = M/N
};
// descriptor for k-step `ks` (16 K elements each)
__device__ __forceinline__ uint64_t operand_desc(const Operand& op, uint32_t ks) {
  if (!op.mn_major) {
    // K runs along columns: 4 k-steps per slab, 32 bytes each inside the swizzle atom
    const uint32_t a = op.addr + (ks >> 2) * op.rows * kSlabRowBytes + (ks & 3) * 32;
    return umma_desc(a, 16, 1024);
  }
  // K runs along rows: 16 rows = 2048 bytes per k-step
  return umma_desc(op.addr + ks * 16 * kSlabRowBytes, op.rows * kSlabRowBytes, 1024);
}
// D[128 x n] (+)= A x B over `ksteps` k-steps; issued by ONE thread
__device__ __forceinline__ void umma_gemm(uint32_t d_tmem, const Operand& a, const Operand& b, uint32_t n,
                                          uint32_t ksteps, bool accumulate) {
  const uint32_t idesc = umma_idesc(128, n, a.mn_major, b.mn_major);
  for (uint32_t ks = 0; ks < ksteps; ++ks)
    umma(d_tmem, operand_desc(a, ks), operand_desc(b, ks), idesc, (accumulate || ks > 0) ? 1u : 0u);
}

// D[128 x n] (+)= A x B over 8 k-steps with A = a 128 x 128 bf16 matrix in tensor memory.  `split`:
// K elements 0..63 sit in columns [0, 32) and 64..127 in columns [64, 96) of the region at a_tmem (what
// packing an fp32 accumulator in place, half by half, leaves); otherwise in columns [0, 64).
__device__ __forceinline__ void umma_gemm_ts(uint32_t d_tmem, uint32_t a_tmem, bool split, const Operand& b,
                                             uint32_t n, bool accumulate) {
  const uint32_t idesc = umma_idesc(128, n, false, b.mn_major);
  for (uint32_t ks = 0; ks < 8; ++ks) {
    const uint32_t col = split ? (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8) : ks * 8;
    umma_ts(d_tmem, a_tmem + col, operand_desc(b, ks), idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// ---------------------------------------------------------------------------
// host: tensor map of a row-major bf16 matrix [rows x width], box = {64, box_rows, width/64}
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// CUresult of the last failed encode on this thread (diagnostics)
inline int& last_encode_result() {
  static thread_local int r = 0;
  return r;
}

inline cudaError_t make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t width,
                                 uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return cudaErrorNotSupported;
  if (width % 64 || box_rows > 256 || rows == 0) return cudaErrorInvalidValue;
  const cuuint64_t dims[3] = {64, rows, width / 64};
  const cuuint64_t strides[2] = {(cuuint64_t)width * 2, 128};  // bytes, for dims 1 and 2
  const cuuint32_t box[3] = {64, box_rows, width / 64};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) last_encode_result() = (int)r;
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// tensor map of `seqs` row-major bf16 matrices [n x width] lying one after the other,
// box = {64, box_rows, width/64, 1}: a tile never crosses from one sequence into the next
// `pitch`: elements from one token's row to the next (= width for a tensor of its own; larger for a slice of the
// head dimension of a wider tensor, which is then read and written in place)
inline cudaError_t make_seq_tile_map(CUtensorMap* map, const void* base, uint64_t seqs, uint64_t n, uint32_t width,
                                     uint32_t box_rows, uint32_t pitch) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return cudaErrorNotSupported;
  if (width % 64 || box_rows > 256 || n == 0 || seqs == 0 || pitch < width || pitch % 8) return cudaErrorInvalidValue;
  const cuuint64_t dims[4] = {64, n, width / 64, seqs};
  const cuuint64_t strides[3] = {(cuuint64_t)pitch * 2, 128, (cuuint64_t)n * pitch * 2};  // bytes, dims 1..3
  const cuuint32_t box[4] = {64, box_rows, width / 64, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) last_encode_result() = (int)r;
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace sm100
}  // namespace lasp
