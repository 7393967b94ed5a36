// fp32 FFMA kernels: the precision path (fp32 I/O parity mode) and the path
// for shapes the tensor-core kernels do not take (ragged n, d/e not in
// {64,128}, fp16).  Operands are converted to fp32 on load, every product is
// accumulated in fp32, results are rounded once on store.
//
// One CTA of 256 threads (16x16) owns one 64-token chunk of one (batch, head).
// Shared-memory tiles carry one float of row padding so that column walks are
// bank-conflict free.
#include "common.cuh"

namespace lasp {
namespace {

constexpr int C = kSimtChunk;  // 64 tokens
constexpr int NT = 256;
constexpr int MAXD16 = 8;      // d, e <= 128

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// rows [0,len) of a (len x w) global tile -> smem (C x (w+1)) fp32, zero fill beyond len
template <typename T>
__device__ __forceinline__ void load_tile(float* sm, const T* g, int len, int w) {
  const int ld = w + 1;
  for (int idx = threadIdx.x; idx < C * w; idx += NT) {
    int r = idx / w, c = idx - r * w;
    sm[r * ld + c] = (r < len) ? to_f<T>(g[(size_t)r * w + c]) : 0.f;
  }
}

// ---------------------------------------------------------------------------
// chunk states: out[i][j] = sum_c w_c A[c][i] B[c][j]
//   forward : A = K, B = V,  w_c = lambda^(len-c)
//   backward: A = Q, B = dO, w_c = lambda^c
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) k_chunk_states(const T* __restrict__ A, const T* __restrict__ B,
                                                     const float* __restrict__ s, float* __restrict__ states,
                                                     int h, int n, int d, int e, int nc, int backward) {
  extern __shared__ float sm[];
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int len = min(C, n - chunk * C);
  const float sh = s[bh % h];
  float* sa = sm;                 // C x (d+1)
  float* sb = sm + C * (d + 1);   // C x (e+1)
  load_tile<T>(sa, A + ((size_t)bh * n + (size_t)chunk * C) * d, len, d);
  load_tile<T>(sb, B + ((size_t)bh * n + (size_t)chunk * C) * e, len, e);
  __syncthreads();
  // fold the weight into A
  for (int idx = threadIdx.x; idx < C * d; idx += NT) {
    int r = idx / d, c = idx - r * d;
    float w = backward ? expf(-sh * (float)r) : expf(-sh * (float)max(len - r, 0));
    sa[r * (d + 1) + c] *= w;
  }
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int d16 = d >> 4, e16 = e >> 4;
  float acc[MAXD16][MAXD16];
#pragma unroll
  for (int i = 0; i < MAXD16; ++i)
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) acc[i][j] = 0.f;
  for (int c = 0; c < C; ++c) {
    float a[MAXD16], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < MAXD16; ++i) a[i] = (i < d16) ? sa[c * (d + 1) + ty + 16 * i] : 0.f;
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < e16) ? sb[c * (e + 1) + tx + 16 * j] : 0.f;
#pragma unroll
    for (int i = 0; i < MAXD16; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
  }
  float* out = states + ((size_t)bh * nc + chunk) * d * e;
#pragma unroll
  for (int i = 0; i < MAXD16; ++i)
#pragma unroll
    for (int j = 0; j < MAXD16; ++j)
      if (i < d16 && j < e16) out[(size_t)(ty + 16 * i) * e + tx + 16 * j] = acc[i][j];
}

// ---------------------------------------------------------------------------
// scan over chunks, elementwise in (d,e).  forward: exclusive prefix seeded
// with x_in; reverse: exclusive suffix.  k_scan reads the fp32 local states
// and writes the prefix states to a second array.  Loads of a batch of chunks are issued before the
// dependent recurrence so that their latencies overlap.
// ---------------------------------------------------------------------------
constexpr int kScanBatch = 8;

__global__ void __launch_bounds__(256) k_scan(const float* __restrict__ s, const float* __restrict__ local,
                                              float* __restrict__ prefix, const float* __restrict__ x_in,
                                              float* __restrict__ x_out, int h,
                                              int n, int de, int nc, int chunk, int reverse, int lane_rows,
                                              int cols) {
  const int bh = blockIdx.y;
  const int el = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (el >= de) return;
  // where this float4 lives in the caller's row-major rank states
  const int ext = lane_rows > 0 ? lane_order_to_row_major(el / 4, lane_rows, cols) * 4 : el;
  const float sh = s[bh % h];
  const float full = expf(-sh * (float)chunk);
  const int last_len = n - (nc - 1) * chunk;
  const float tail = expf(-sh * (float)last_len);
  float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
  if (x_in) p = *reinterpret_cast<const float4*>(x_in + (size_t)bh * de + ext);
  const float* base = local + (size_t)bh * nc * de + el;
  float* out = prefix + (size_t)bh * nc * de + el;
  for (int i0 = 0; i0 < nc; i0 += kScanBatch) {
    float4 loc[kScanBatch];
#pragma unroll
    for (int u = 0; u < kScanBatch; ++u) {
      const int i = i0 + u;
      if (i < nc) loc[u] = *reinterpret_cast<const float4*>(base + (size_t)(reverse ? nc - 1 - i : i) * de);
    }
#pragma unroll
    for (int u = 0; u < kScanBatch; ++u) {
      const int i = i0 + u;
      if (i < nc) {
        const int c = reverse ? nc - 1 - i : i;
        const float dec = (c == nc - 1) ? tail : full;
        *reinterpret_cast<float4*>(out + (size_t)c * de) = p;
        p.x = fmaf(dec, p.x, loc[u].x);
        p.y = fmaf(dec, p.y, loc[u].y);
        p.z = fmaf(dec, p.z, loc[u].z);
        p.w = fmaf(dec, p.w, loc[u].w);
      }
    }
  }
  if (x_out) *reinterpret_cast<float4*>(x_out + (size_t)bh * de + ext) = p;
}

__global__ void __launch_bounds__(256) k_state_combine(const float* __restrict__ s, const float* __restrict__ x_in,
                                                       const float* __restrict__ x_local, float* __restrict__ x_out,
                                                       int h, int de, int n) {
  const int bh = blockIdx.y;
  const int el = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (el >= de) return;
  const float dec = expf(-s[bh % h] * (float)n);
  float4 loc = *reinterpret_cast<const float4*>(x_local + (size_t)bh * de + el);
  if (x_in) {
    float4 p = *reinterpret_cast<const float4*>(x_in + (size_t)bh * de + el);
    loc.x = fmaf(dec, p.x, loc.x);
    loc.y = fmaf(dec, p.y, loc.y);
    loc.z = fmaf(dec, p.z, loc.z);
    loc.w = fmaf(dec, p.w, loc.w);
  }
  *reinterpret_cast<float4*>(x_out + (size_t)bh * de + el) = loc;
}

// masked 64x64 product: out[r][c] = [r>=c] lambda^(r-c) sum_i X[r][i] Y[c][i]
__device__ __forceinline__ void masked_gram(float* out, const float* X, const float* Y, int w, float sh) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int ld = w + 1;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k = 0; k < w; ++k) {
    float x[4], y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = X[(ty + 16 * i) * ld + k];
#pragma unroll
    for (int j = 0; j < 4; ++j) y[j] = Y[(tx + 16 * j) * ld + k];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(x[i], y[j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = ty + 16 * i, c = tx + 16 * j;
      out[r * (C + 1) + c] = (r >= c) ? acc[i][j] * expf(-sh * (float)(r - c)) : 0.f;
    }
}

// ---------------------------------------------------------------------------
// forward output: O = S_m V + diag(lambda^r) Q P,  S_m = (Q K^T) * M
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) k_fwd_output(const T* __restrict__ Q, const T* __restrict__ K,
                                                   const T* __restrict__ V, const float* __restrict__ s,
                                                   const float* __restrict__ prefix, T* __restrict__ O, int h, int n,
                                                   int d, int e, int nc) {
  extern __shared__ float sm[];
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int len = min(C, n - chunk * C);
  const float sh = s[bh % h];
  float* sq = sm;
  float* sk = sq + C * (d + 1);
  float* sv = sk + C * (d + 1);
  float* ss = sv + C * (e + 1);  // C x (C+1)
  const size_t tok0 = (size_t)bh * n + (size_t)chunk * C;
  load_tile<T>(sq, Q + tok0 * d, len, d);
  load_tile<T>(sk, K + tok0 * d, len, d);
  load_tile<T>(sv, V + tok0 * e, len, e);
  __syncthreads();
  masked_gram(ss, sq, sk, d, sh);
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int e16 = e >> 4;
  float intra[4][MAXD16], inter[4][MAXD16];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) intra[i][j] = inter[i][j] = 0.f;
  for (int c = 0; c < C; ++c) {
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = ss[(ty + 16 * i) * (C + 1) + c];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < e16) ? sv[c * (e + 1) + tx + 16 * j] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) intra[i][j] = fmaf(a[i], bb[j], intra[i][j]);
  }
  const float* P = prefix + ((size_t)bh * nc + chunk) * d * e;
  for (int k = 0; k < d; ++k) {
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sq[(ty + 16 * i) * (d + 1) + k];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < e16) ? __ldg(P + (size_t)k * e + tx + 16 * j) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) inter[i][j] = fmaf(a[i], bb[j], inter[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty + 16 * i;
    if (r < len) {
      const float qd = expf(-sh * (float)r);
#pragma unroll
      for (int j = 0; j < MAXD16; ++j)
        if (j < e16) O[(tok0 + r) * e + tx + 16 * j] = from_f<T>(fmaf(qd, inter[i][j], intra[i][j]));
    }
  }
}

// ---------------------------------------------------------------------------
// backward: dQ = dS_m K + diag(lambda^r) dO P^T
//           dK = dS_m^T Q + diag(lambda^(len-c)) V D^T
//           dV = S_m^T dO + diag(lambda^(len-c)) K D
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) k_bwd_grads(const T* __restrict__ Q, const T* __restrict__ K,
                                                  const T* __restrict__ V, const T* __restrict__ DO,
                                                  const float* __restrict__ s, const float* __restrict__ prefix,
                                                  const float* __restrict__ suffix, T* __restrict__ DQ,
                                                  T* __restrict__ DK, T* __restrict__ DV, int h, int n, int d, int e,
                                                  int nc) {
  extern __shared__ float sm[];
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int len = min(C, n - chunk * C);
  const float sh = s[bh % h];
  float* sq = sm;
  float* sk = sq + C * (d + 1);
  float* sv = sk + C * (d + 1);
  float* sdo = sv + C * (e + 1);
  float* ss = sdo + C * (e + 1);   // S_m
  float* sds = ss + C * (C + 1);   // dS_m
  const size_t tok0 = (size_t)bh * n + (size_t)chunk * C;
  load_tile<T>(sq, Q + tok0 * d, len, d);
  load_tile<T>(sk, K + tok0 * d, len, d);
  load_tile<T>(sv, V + tok0 * e, len, e);
  load_tile<T>(sdo, DO + tok0 * e, len, e);
  __syncthreads();
  masked_gram(ss, sq, sk, d, sh);
  masked_gram(sds, sdo, sv, e, sh);
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int d16 = d >> 4, e16 = e >> 4;
  const float* P = prefix + ((size_t)bh * nc + chunk) * d * e;
  const float* D = suffix + ((size_t)bh * nc + chunk) * d * e;
  float a1[4][MAXD16], a2[4][MAXD16];

  // ---- dQ[r][i]
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) a1[i][j] = a2[i][j] = 0.f;
  for (int c = 0; c < C; ++c) {
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sds[(ty + 16 * i) * (C + 1) + c];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < d16) ? sk[c * (d + 1) + tx + 16 * j] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) a1[i][j] = fmaf(a[i], bb[j], a1[i][j]);
  }
  for (int k = 0; k < e; ++k) {  // sum_j dO[r][j] P[i][j]
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sdo[(ty + 16 * i) * (e + 1) + k];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < d16) ? __ldg(P + (size_t)(tx + 16 * j) * e + k) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) a2[i][j] = fmaf(a[i], bb[j], a2[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty + 16 * i;
    if (r < len) {
      const float qd = expf(-sh * (float)r);
#pragma unroll
      for (int j = 0; j < MAXD16; ++j)
        if (j < d16) DQ[(tok0 + r) * d + tx + 16 * j] = from_f<T>(fmaf(qd, a2[i][j], a1[i][j]));
    }
  }

  // ---- dK[c][i]
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) a1[i][j] = a2[i][j] = 0.f;
  for (int r = 0; r < C; ++r) {
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sds[r * (C + 1) + ty + 16 * i];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < d16) ? sq[r * (d + 1) + tx + 16 * j] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) a1[i][j] = fmaf(a[i], bb[j], a1[i][j]);
  }
  for (int k = 0; k < e; ++k) {  // sum_j V[c][j] D[i][j]
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sv[(ty + 16 * i) * (e + 1) + k];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < d16) ? __ldg(D + (size_t)(tx + 16 * j) * e + k) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) a2[i][j] = fmaf(a[i], bb[j], a2[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = ty + 16 * i;
    if (c < len) {
      const float kd = expf(-sh * (float)(len - c));
#pragma unroll
      for (int j = 0; j < MAXD16; ++j)
        if (j < d16) DK[(tok0 + c) * d + tx + 16 * j] = from_f<T>(fmaf(kd, a2[i][j], a1[i][j]));
    }
  }

  // ---- dV[c][j]
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) a1[i][j] = a2[i][j] = 0.f;
  for (int r = 0; r < C; ++r) {
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = ss[r * (C + 1) + ty + 16 * i];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < e16) ? sdo[r * (e + 1) + tx + 16 * j] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) a1[i][j] = fmaf(a[i], bb[j], a1[i][j]);
  }
  for (int k = 0; k < d; ++k) {  // sum_i K[c][i] D[i][j]
    float a[4], bb[MAXD16];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sk[(ty + 16 * i) * (d + 1) + k];
#pragma unroll
    for (int j = 0; j < MAXD16; ++j) bb[j] = (j < e16) ? __ldg(D + (size_t)k * e + tx + 16 * j) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < MAXD16; ++j) a2[i][j] = fmaf(a[i], bb[j], a2[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = ty + 16 * i;
    if (c < len) {
      const float kd = expf(-sh * (float)(len - c));
#pragma unroll
      for (int j = 0; j < MAXD16; ++j)
        if (j < e16) DV[(tok0 + c) * e + tx + 16 * j] = from_f<T>(fmaf(kd, a2[i][j], a1[i][j]));
    }
  }
}

template <typename F>
cudaError_t set_smem(F* fn, size_t bytes) {
  return cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

#define LASP_DISPATCH_DTYPE(dt, ...)                                   \
  switch (dt) {                                                         \
    case LASP_F32: { using T = float; __VA_ARGS__; break; }             \
    case LASP_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }    \
    case LASP_F16: { using T = __half; __VA_ARGS__; break; }            \
    default: return cudaErrorInvalidValue;                              \
  }

cudaError_t simt_chunk_states(const Dims& m, const void* a, const void* bten, const float* s, float* states,
                              bool backward, cudaStream_t st) {
  const size_t smem = (size_t)C * (m.d + 1 + m.e + 1) * sizeof(float);
  dim3 grid(m.nc, m.b * m.h);
  LASP_DISPATCH_DTYPE(m.dtype, {
    cudaError_t err = set_smem(k_chunk_states<T>, smem);
    if (err != cudaSuccess) return err;
    k_chunk_states<T><<<grid, NT, smem, st>>>((const T*)a, (const T*)bten, s, states, m.h, m.n, m.d, m.e, m.nc,
                                              backward ? 1 : 0);
  });
  return cudaGetLastError();
}

cudaError_t scan_states(const Dims& m, const float* s, const float* local, float* prefix, const float* x_in,
                        float* x_out, bool reverse, cudaStream_t st) {
  const int de = m.d * m.e;
  dim3 grid((de / 4 + 255) / 256, m.b * m.h);
  k_scan<<<grid, 256, 0, st>>>(s, local, prefix, x_in, x_out, m.h, m.n, de, m.nc, m.chunk, reverse ? 1 : 0, m.walk ? m.d : 0,
                               m.e);
  return cudaGetLastError();
}


cudaError_t state_combine(int b, int h, int d, int e, int n, const float* s, const float* x_in,
                          const float* x_local, float* x_out, cudaStream_t st) {
  const int de = d * e;
  dim3 grid((de / 4 + 255) / 256, b * h);
  k_state_combine<<<grid, 256, 0, st>>>(s, x_in, x_local, x_out, h, de, n);
  return cudaGetLastError();
}

cudaError_t simt_fwd_output(const Dims& m, const void* q, const void* k, const void* v, const float* s,
                            const float* prefix, void* o, cudaStream_t st) {
  const size_t smem = (size_t)C * (2 * (m.d + 1) + (m.e + 1) + (C + 1)) * sizeof(float);
  dim3 grid(m.nc, m.b * m.h);
  LASP_DISPATCH_DTYPE(m.dtype, {
    cudaError_t err = set_smem(k_fwd_output<T>, smem);
    if (err != cudaSuccess) return err;
    k_fwd_output<T><<<grid, NT, smem, st>>>((const T*)q, (const T*)k, (const T*)v, s, prefix, (T*)o, m.h, m.n, m.d,
                                            m.e, m.nc);
  });
  return cudaGetLastError();
}

cudaError_t simt_bwd_grads(const Dims& m, const void* q, const void* k, const void* v, const void* d_o,
                           const float* s, const float* prefix, const float* suffix, void* dq, void* dk,
                           void* dv, cudaStream_t st) {
  const size_t smem = (size_t)C * (2 * (m.d + 1) + 2 * (m.e + 1) + 2 * (C + 1)) * sizeof(float);
  dim3 grid(m.nc, m.b * m.h);
  LASP_DISPATCH_DTYPE(m.dtype, {
    cudaError_t err = set_smem(k_bwd_grads<T>, smem);
    if (err != cudaSuccess) return err;
    k_bwd_grads<T><<<grid, NT, smem, st>>>((const T*)q, (const T*)k, (const T*)v, (const T*)d_o, s, prefix, suffix,
                                           (T*)dq, (T*)dk, (T*)dv, m.h, m.n, m.d, m.e, m.nc);
  });
  return cudaGetLastError();
}

}  // namespace lasp
