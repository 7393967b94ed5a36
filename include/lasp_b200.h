/*
 * lasp_b200 - C ABI of the B200 (sm_100a) linear-attention library.
 *
 * The reference (OpenNLPLab/LASP) has no FFI layer: its Python autograd
 * functions launch Triton kernels directly.  This header is the boundary the
 * Python operator surface of this repository binds with ctypes; every entry
 * point names the reference launcher / kernel whose work it takes over
 * (paths relative to the reference checkout).
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless
 *     its name ends in _host;
 *   - the caller owns all memory; nothing here allocates device memory;
 *   - every call is asynchronous on the given stream (a cudaStream_t passed
 *     as void*; NULL = the legacy default stream);
 *   - return value: LASP_OK or a negative lasp_status; invalid arguments are
 *     rejected BEFORE anything is launched;
 *   - tensors are contiguous: q,k (b,h,n,d); v,o,do (b,h,n,e); s h floats;
 *     rank states kv_in/kv_out/dkv_in/dkv_out (b,h,d,e) fp32.
 *
 * Math (per batch, head; lambda = exp(-s_h)):
 *   O  = ((Q K^T) * M) V + diag(lambda^pos) Q KV_in,   M_ij = lambda^(i-j) [i>=j]
 *   KV_out  = lambda^n KV_in  + sum_j lambda^(n-j) k_j v_j^T
 *   DKV_out = lambda^n DKV_in + sum_i lambda^i     q_i do_i^T
 * The sequence is cut into chunks; each phase below is one kernel launch:
 *   chunk states (independent of the incoming rank state) -> scan over chunks
 *   (consumes KV_in, yields KV_out) -> outputs.  The split lets a
 *   sequence-parallel caller overlap the first phase with the state transfer.
 */
#ifndef LASP_B200_H
#define LASP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LASP_B200_ABI_VERSION 3

/* the library is built with hidden visibility; only the entry points below are exported */
#if defined(__GNUC__)
#define LASP_B200_API __attribute__((visibility("default")))
#else
#define LASP_B200_API
#endif

typedef enum {
  LASP_OK = 0,
  LASP_ERR_NULL = -1,       /* a required pointer is NULL */
  LASP_ERR_SHAPE = -2,      /* unsupported b,h,n,d,e */
  LASP_ERR_DTYPE = -3,      /* unknown dtype */
  LASP_ERR_ALIGN = -4,      /* a pointer is not 16-byte aligned */
  LASP_ERR_WORKSPACE = -5,  /* workspace too small */
  LASP_ERR_CUDA = -6,       /* a CUDA runtime call failed (see lasp_b200_last_cuda_error) */
  LASP_ERR_PATH = -7,       /* requested kernel path cannot run this problem */
  LASP_ERR_DEVICE = -8,     /* a kernel reported a fault (see lasp_b200_read_status) */
  LASP_ERR_TOO_LARGE = -9   /* problem exceeds a fixed capacity of the entry point */
} lasp_status;

typedef enum { LASP_F32 = 0, LASP_BF16 = 1, LASP_F16 = 2 } lasp_dtype;

/* which kernels run: AUTO picks TENSOR when the problem qualifies */
typedef enum {
  LASP_PATH_AUTO = 0,
  LASP_PATH_SIMT = 1,   /* fp32 FFMA kernels: any dtype, d,e multiples of 16 up to 128, any n */
  LASP_PATH_TENSOR = 2  /* tcgen05/TMEM/TMA kernels: bf16, d,e in {64,128}, n >= 128 (a ragged tail is fine) */
} lasp_path;

/* Preprocessing of q and k folded into the kernels' load path: the operator is evaluated on
 * qk_scale * map(q) and qk_scale * map(k), and dq, dk are the gradients with respect to the RAW q and k
 * (chain rule applied in the epilogues).  Replaces the caller-side passes `q, k = elu(q) + 1, elu(k) + 1`
 * and `q, k *= d ** -0.5` in front of lightning_attn / lasp_* (lasp/lightning_attention.py:510); each of
 * them would read and write q and k once more in an operator bound by memory traffic.  Only the fused
 * tensor-core launches (forward, backward, the linked forms, bwd_dq, bwd_dkv) take it; every other entry
 * point returns LASP_ERR_PATH when it is requested. */
typedef enum { LASP_QK_IDENTITY = 0, LASP_QK_ELU1 = 1 /* elu(x) + 1 */ } lasp_qk_map;

typedef struct {
  int32_t b, h, n, d, e;
  int32_t dtype;   /* lasp_dtype of q,k,v,o,do,dq,dk,dv */
  int32_t path;    /* lasp_path */
  int32_t qk_map;  /* lasp_qk_map */
  float qk_scale;  /* 0 is read as 1 */
  /* Elements from one token's row to the next in q,k,dq,dk (pitch_d) and in v,o,do,dv (pitch_e); 0 = d / e, i.e.
   * tensors of their own.  Larger values let a call work in place on a 128-wide slice of the head dimension of
   * wider tensors (the slicing of lasp/lightning_attention.py:510-531 without a copy per slice): pass the address
   * of the slice's first column.  Multiples of 8; tensor-core path only (LASP_ERR_PATH otherwise). */
  int32_t pitch_d, pitch_e;
} lasp_problem;

/* Forward arguments.  ws = workspace of lasp_b200_fwd_workspace_bytes(); after
 * the scan phase it holds the per-chunk prefix states, which the backward
 * reads (the "intermediate state caching" of lasp/lasp_fuse_parallel.py:876,
 * 1103) - keep it alive until backward has run. */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const float* s;
  const float* kv_in; /* NULL = zero state (first rank / single device) */
  float* kv_out;      /* NULL = not wanted */
  void* o;
  void* ws;
  size_t ws_bytes;
} lasp_fwd_args;

/* Backward arguments.  fwd_ws = the forward's workspace (read only);
 * ws = scratch of lasp_b200_bwd_workspace_bytes(). */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const void* d_o;
  const float* s;
  const float* dkv_in; /* NULL = zero state (last rank / single device) */
  float* dkv_out;      /* NULL = not wanted */
  void* dq;
  void* dk;
  void* dv;
  const void* fwd_ws;
  size_t fwd_ws_bytes;
  void* ws;
  size_t ws_bytes;
} lasp_bwd_args;

LASP_B200_API int lasp_b200_abi_version(void);
LASP_B200_API const char* lasp_b200_strerror(int status);
/* text of the last CUDA runtime error seen by this thread inside the library */
LASP_B200_API const char* lasp_b200_last_cuda_error(void);

/* Resolves LASP_PATH_AUTO; returns LASP_PATH_SIMT / LASP_PATH_TENSOR or a
 * negative status when the problem is invalid (lasp_forward's shape asserts,
 * lasp/lasp_fuse_parallel.py:1080-1085, made explicit). */
LASP_B200_API int lasp_b200_resolve_path(const lasp_problem* p);
/* tokens per chunk state for the resolved path */
LASP_B200_API int lasp_b200_chunk_tokens(const lasp_problem* p);
LASP_B200_API size_t lasp_b200_fwd_workspace_bytes(const lasp_problem* p);
LASP_B200_API size_t lasp_b200_bwd_workspace_bytes(const lasp_problem* p);

/* ---- forward phases -------------------------------------------------- */
/* per-chunk local states sum_c lambda^(len-c) k_c v_c^T.
 * Replaces _fwd_kv_parallel, lasp/lasp_fuse_parallel.py:117-200. */
LASP_B200_API int lasp_b200_fwd_chunk_states(const lasp_problem* p, const lasp_fwd_args* a, void* stream);
/* exclusive decayed scan of the chunk states seeded with kv_in; writes kv_out.
 * Replaces _fwd_kv_reduce, lasp/lasp_fuse_parallel.py:203-257, and the host
 * update KV = block_decay*KV + kv, lasp/lasp_fuse_parallel.py:941-942. */
LASP_B200_API int lasp_b200_fwd_scan(const lasp_problem* p, const lasp_fwd_args* a, void* stream);
/* O = intra-chunk masked product + decayed Q x prefix state.
 * Replaces _fwd_diag_kernel + _fwd_none_diag_kernel,
 * lasp/lasp_fuse_parallel.py:15-114,261-336 (== _fwd_kernel of
 * lasp/lightning_attention.py:6-83 and lasp/lasp_fuse.py:15-127). */
LASP_B200_API int lasp_b200_fwd_output(const lasp_problem* p, const lasp_fwd_args* a, void* stream);
/* the whole forward: lasp_forward, lasp/lasp_fuse.py:356-406.  On the tensor-core path ONE launch (span
 * totals, the states at the span borders from them and kv_in, the walk; kv_out on the way) whenever the
 * spans fit one per SM; otherwise, and on the fp32 path, the three phases back to back. */
LASP_B200_API int lasp_b200_forward(const lasp_problem* p, const lasp_fwd_args* a, void* stream);

/* ---- backward phases ------------------------------------------------- */
/* per-chunk local dKV states sum_r lambda^r q_r do_r^T.
 * Replaces _bwd_dkv_parallel, lasp/lasp_fuse_parallel.py:522-604. */
LASP_B200_API int lasp_b200_bwd_chunk_states(const lasp_problem* p, const lasp_bwd_args* a, void* stream);
/* reverse exclusive decayed scan seeded with dkv_in; writes dkv_out.
 * Replaces _bwd_dkv_reduce, lasp/lasp_fuse_parallel.py:607-662, and the host
 * update DKV = block_decay*DKV + dkv, lasp/lasp_fuse_parallel.py:1067-1068. */
LASP_B200_API int lasp_b200_bwd_scan(const lasp_problem* p, const lasp_bwd_args* a, void* stream);
/* dQ, dK, dV from the cached prefix states and the suffix dKV states.
 * Replaces _bwd_diag_kernel + _bwd_none_diag_kernel,
 * lasp/lasp_fuse_parallel.py:339-519,665-830 (== _bwd_intra_kernel +
 * _bwd_inter_kernel, lasp/lightning_attention.py:86-393). */
LASP_B200_API int lasp_b200_bwd_grads(const lasp_problem* p, const lasp_bwd_args* a, void* stream);
/* the whole backward: lasp_backward, lasp/lasp_fuse.py:409-475.  On the tensor-core path two launches:
 * dQ (a forward walk over the states the forward pass kept in fwd_ws) and dK,dV (one fused launch: span
 * totals of q,do, the suffix states from them and dkv_in, the reverse walk; dkv_out on the way). */
LASP_B200_API int lasp_b200_backward(const lasp_problem* p, const lasp_bwd_args* a, void* stream);
/* those two launches on their own (each independent of the other's results); on the fp32 path the
 * first does nothing and the second is the whole backward.  Replace _bwd_inter_kernel's forward sweep
 * and reverse sweep, lasp/lightning_attention.py:238-278 and :333-393, with their intra-block parts. */
LASP_B200_API int lasp_b200_bwd_dq(const lasp_problem* p, const lasp_bwd_args* a, void* stream);
LASP_B200_API int lasp_b200_bwd_dkv(const lasp_problem* p, const lasp_bwd_args* a, void* stream);
/* dK, dV alone from the suffix states that lasp_b200_bwd_scan (or lasp_b200_exchange_scan) left in ws:
 * lasp_b200_bwd_grads without its dQ launch (on the fp32 path: all of lasp_b200_bwd_grads). */
LASP_B200_API int lasp_b200_bwd_dkv_walk(const lasp_problem* p, const lasp_bwd_args* a, void* stream);

/* x_out = exp(-s_h n) x_in + x_local on (b,h,d,e) fp32 states; x_in may be NULL.
 * Replaces the torch glue KV = block_decay*KV + kv, lasp/lasp_naive.py:565,614. */
LASP_B200_API int lasp_b200_state_combine(int b, int h, int d, int e, int n, const float* s, const float* x_in,
                            const float* x_local, float* x_out, void* stream);

/* ---- state hand-over over NVLink peer memory --------------------------- */
/* The state hand-over of a sequence-parallel group, one launch per rank and
 * direction, over peer-mapped buffers.  Rank-to-rank passing,
 *     x_in(r+1) = exp(-s n) x_in(r) + total(r),
 * has the closed form x_in(r) = sum_{q<r} exp(-s n)^(r-1-q) total(q).  Called
 * between the chunk-state phase and the output / gradient phase IN PLACE OF the
 * scan phase, the kernel
 *   - reduces this rank's chunk states (in `ws`) to its total and stores it
 *     into the receive slots of the ranks after it in the chain order (plain
 *     peer stores over NVLink);
 *   - waits for what the ranks before it stored here, sums it with the decay
 *     powers (= the incoming rank state) and runs the scan with it, leaving
 *     `ws` exactly as lasp_b200_fwd_scan / lasp_b200_bwd_scan would.
 * A contribution whose decay power exp(-s n (r-1-q)) is below 1e-12 is neither
 * sent nor awaited.  Replaces dist.recv / KV update / dist.send of
 * lasp/lasp_fuse_parallel.py:1095-1106 (forward) and :1129-1135 (backward: the
 * caller reverses the chain order and sets `reverse`) - one NVLink latency
 * instead of ranks-1 - together with _fwd_kv_reduce / _bwd_dkv_reduce
 * (lasp/lasp_fuse_parallel.py:203-257, 607-662).
 * `position` is this rank's place in the chain order (0 sends only, ranks-1
 * receives only); peer_* arrays are indexed by position.  All pointers are
 * device pointers; peer_* point into other GPUs' memory mapped into this
 * process (a symmetric allocation, zeroed once).  Per rank and direction:
 *   slots   : 2 x ranks x (b*h*d*e) 8-byte words {value, step}
 *             [step parity][source][element]; a word is valid for the current
 *             step when its second half equals the step number, so no flag or
 *             fence is needed on the path
 *   acks    : ranks x 8 words, 128 bytes apart  [destination][slice], written by destinations
 *   counters: 16 words, zeroed once; the kernel keeps the step number there, so
 *             a replayed CUDA graph needs no new arguments.
 * Waits give up after wait_clocks GPU clocks (0 = about ten seconds), set bit 4
 * of the fault word (lasp_b200_read_status) and make the states they could not
 * complete NaN, so that a late peer cannot pass for a delivered state. */
/* The two halves can also go out as two launches of the same step - LASP_EXCHANGE_PUSH as soon as the
 * chunk states exist, LASP_EXCHANGE_GATHER (which completes the step) later - so that work that does not
 * need the incoming state (dQ in the backward pass) runs between them while the states are in flight. */
typedef enum { LASP_EXCHANGE_BOTH = 0, LASP_EXCHANGE_PUSH = 1, LASP_EXCHANGE_GATHER = 2 } lasp_exchange_phase;
typedef struct {
  int32_t ranks;             /* group size, 2..8 */
  int32_t position;          /* this rank's place in the chain order */
  int32_t reverse;           /* 0: forward (KV, prefix scan); 1: backward (dKV, suffix scan) */
  int32_t phase;             /* lasp_exchange_phase */
  const float* s;            /* h decay rates */
  void* ws;                  /* the forward / backward workspace after its chunk-state phase */
  size_t ws_bytes;
  const void* my_slots;      /* local receive slots */
  const uint32_t* my_acks;   /* local acknowledgement words */
  uint32_t* counters;        /* local */
  void* peer_slots[8];       /* receive slots of each position (entries > position are written) */
  uint32_t* peer_acks[8];    /* acknowledgement words of each position (entries < position are written) */
  int64_t wait_clocks;
} lasp_exchange_args;
LASP_B200_API int lasp_b200_exchange_scan(const lasp_problem* p, const lasp_exchange_args* a, void* stream);

/* Compute and hand-over in ONE launch per direction: the fused forward kernel (lasp_b200_forward) and
 * the fused dK,dV kernel (lasp_b200_bwd_dkv) with the group's peer-mapped buffers (x: ranks, position,
 * my_slots, my_acks, counters, peer_slots, peer_acks, wait_clocks; for the backward call the chain order
 * reversed; the other fields are ignored).  The CTA that owns the end of a sequence stores the
 * sequence's total into the slots of the ranks after this one as soon as the span totals exist; every
 * CTA adds what the ranks before stored here to the state at its span's border, and walks.  kv_in /
 * kv_out (dkv_in / dkv_out) of the arguments are not used.  Replaces, for a sequence-parallel rank,
 * LaspFuseParallel.forward / .backward of lasp/lasp_fuse_parallel.py:1075-1137 in one launch each
 * (plus lasp_b200_bwd_dq).  Needs every span on an SM of its own: lasp_b200_linked_ok returns 1 when
 * the problem qualifies (0: use the chunk-state phase, lasp_b200_exchange_scan and the output phase),
 * and the calls return LASP_ERR_PATH when it does not. */
LASP_B200_API int lasp_b200_linked_ok(const lasp_problem* p);
LASP_B200_API int lasp_b200_forward_linked(const lasp_problem* p, const lasp_fwd_args* a, const lasp_exchange_args* x,
                                           void* stream);
LASP_B200_API int lasp_b200_bwd_dkv_linked(const lasp_problem* p, const lasp_bwd_args* a, const lasp_exchange_args* x,
                                           void* stream);

/* Copies this device's sticky kernel-fault word to *status_host (synchronises
 * the stream) and clears it when clear != 0.  0 = no kernel reported a fault;
 * the tensor-core kernels set bits when one of their bounded waits (TMA
 * arrival, tcgen05 completion) runs out instead of spinning for ever. */
LASP_B200_API int lasp_b200_read_status(int32_t* status_host, int clear, void* stream);
/* The same word copied to PINNED host memory by an asynchronous copy on `stream`, without
 * synchronising: the caller looks at *status_host_pinned once an event recorded behind this call
 * has completed (how the operators notice a fault one step later without stalling the stream). */
LASP_B200_API int lasp_b200_copy_status_async(int32_t* status_host_pinned, void* stream);

/* Forward pass that allocates nothing and needs no workspace from the caller.
 * (No counterpart in the reference, whose launchers allocate with torch.)
 *
 * For hosts that cannot allocate device memory when they call the operator:
 * a server that gave the whole GPU to its own pool at start-up, or a serving
 * loop in which cudaMalloc / cudaFree (they may synchronise the device) are
 * off limits.  The chunk-state workspace is a fixed array inside the library,
 * LASP_B200_STATIC_SCRATCH_BYTES on every GPU that loads the library, held
 * until the process exits.  a->ws and a->ws_bytes are ignored; inputs, outputs
 * and the optional rank states are the caller's, as in lasp_b200_forward, and
 * the result is the same.
 *   - Problems whose forward workspace (lasp_b200_fwd_workspace_bytes) is
 *     larger than the array are refused with LASP_ERR_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (with
 *     that device current); make that first call before any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents;
 *     each call overwrites everything it later reads, so no clearing is needed,
 *     but two calls whose kernels overlap on the GPU (different streams,
 *     different threads) race - serialise them.
 *   - The prefix states are not kept for a backward pass: this is a
 *     forward-only (inference / prefill) entry point. */
#define LASP_B200_STATIC_SCRATCH_BYTES (64u << 20)
LASP_B200_API int lasp_b200_forward_static(const lasp_problem* p, const lasp_fwd_args* a, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LASP_B200_H */
