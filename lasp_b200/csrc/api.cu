// extern "C" entry points of liblasp_b200.so: argument validation, workspace
// layout and the choice between the tensor-core and the fp32 kernels.
#include <stdio.h>
#include <string.h>

#include <stdlib.h>

#include "common.cuh"

namespace lasp {
thread_local const char* g_failed_step = "";

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int v = 0;
    cached[dev] = (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) ? v : 148;
  }
  return cached[dev];
}

// The tensor-core path takes bf16 with head widths 64 or 128 and at least one full tile per sequence;
// a ragged last tile is handled by the TMA bounds of the walk kernels.
bool tensor_path_supported(const Dims& m) {
  const bool dims_ok = (m.d == 64 || m.d == 128) && (m.e == 64 || m.e == 128);
  return m.dtype == LASP_BF16 && dims_ok && m.n >= kTensorTile;
}
}

namespace {

thread_local char g_cuda_error[256] = "";

int cuda_fail(cudaError_t err) {
  if (err == cudaSuccess) return LASP_OK;
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s%s%s", cudaGetErrorString(err),
           lasp::g_failed_step[0] ? " in " : "", lasp::g_failed_step);
  lasp::g_failed_step = "";
  return LASP_ERR_CUDA;
}

// A thread that has made no CUDA runtime call yet (PyTorch's autograd worker for
// device 0 is one) has no driver context bound, and the driver-API tensor-map
// encoder then fails.  The first entry on each thread binds the context of the
// thread's current device.
void bind_context_once() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// LASP_B200_UNFUSED=1 runs a composite call as its separate phases; LASP_B200_SPAN_TILES=k fixes the span
// length (experiments).  Read once.
bool unfused_requested() {
  static const bool on = [] {
    const char* v = getenv("LASP_B200_UNFUSED");
    return v && v[0] == '1';
  }();
  return on;
}
int span_tiles_requested() {
  static const int k = [] {
    const char* v = getenv("LASP_B200_SPAN_TILES");
    return v ? atoi(v) : 0;
  }();
  return k;
}

// validates the problem and fills Dims; returns LASP_OK or a negative status
int make_dims(const lasp_problem* p, lasp::Dims* m) {
  if (!p) return LASP_ERR_NULL;
  bind_context_once();
  if (p->dtype != LASP_F32 && p->dtype != LASP_BF16 && p->dtype != LASP_F16) return LASP_ERR_DTYPE;
  if (p->b <= 0 || p->h <= 0 || p->n <= 0 || p->d <= 0 || p->e <= 0) return LASP_ERR_SHAPE;
  if (p->d % 16 || p->e % 16 || p->d > 128 || p->e > 128) return LASP_ERR_SHAPE;
  if ((long long)p->b * p->h > 65535) return LASP_ERR_SHAPE;
  m->b = p->b; m->h = p->h; m->n = p->n; m->d = p->d; m->e = p->e;
  m->dtype = p->dtype;
  if (p->qk_map != LASP_QK_IDENTITY && p->qk_map != LASP_QK_ELU1) return LASP_ERR_SHAPE;
  if (p->pitch_d < 0 || p->pitch_e < 0 || (p->pitch_d && p->pitch_d < p->d) || (p->pitch_e && p->pitch_e < p->e) ||
      p->pitch_d % 8 || p->pitch_e % 8)
    return LASP_ERR_SHAPE;
  m->pitch_d = p->pitch_d ? p->pitch_d : p->d;
  m->pitch_e = p->pitch_e ? p->pitch_e : p->e;
  m->qk_map = p->qk_map;
  m->qk_scale = p->qk_scale == 0.f ? 1.f : p->qk_scale;
  m->walk = 0;
  m->tiles = (p->n + lasp::kTensorTile - 1) / lasp::kTensorTile;
  m->span = 1;
  const bool tensor_ok = lasp::tensor_path_supported(*m);
  int path = p->path;
  if (path == LASP_PATH_AUTO) path = tensor_ok ? LASP_PATH_TENSOR : LASP_PATH_SIMT;
  if (path == LASP_PATH_TENSOR && !tensor_ok) return LASP_ERR_PATH;
  if (path != LASP_PATH_TENSOR && path != LASP_PATH_SIMT) return LASP_ERR_PATH;
  m->path = path;
  if (path == LASP_PATH_SIMT) {
    if (lasp::has_qk_preprocessing(*m)) return LASP_ERR_PATH;   // folded into the tensor-core kernels only
    if (m->pitch_d != m->d || m->pitch_e != m->e) return LASP_ERR_PATH;   // slices in place: TMA tensor maps only
    m->chunk = lasp::kSimtChunk;
    m->nc = (p->n + m->chunk - 1) / m->chunk;
    return LASP_OK;
  }
  // Spans: as few tiles per span as keeps the number of spans (= work items of the persistent kernels,
  // b*h per span index) within one CTA per SM; a sequence-rich problem gets one span per sequence.
  m->walk = 1;
  int span = span_tiles_requested();
  if (span <= 0) {
    const int per_seq = lasp::sm_count() / (p->b * p->h);
    span = per_seq >= 1 ? (m->tiles + per_seq - 1) / per_seq : m->tiles;
  }
  if (span > m->tiles) span = m->tiles;
  m->span = span;
  m->chunk = span * lasp::kTensorTile;
  m->nc = (m->tiles + span - 1) / span;
  // the q,k preprocessing lives in the fused launches (and the dQ walk): not in the phase-by-phase schedule
  if (lasp::has_qk_preprocessing(*m) &&
      (unfused_requested() || (m->nc > 1 && p->b * p->h * m->nc > lasp::sm_count())))
    return LASP_ERR_PATH;
  return LASP_OK;
}

size_t workspace_bytes(const lasp::Dims& m) {
  size_t s = lasp::state_elems(m);
  size_t bytes = 2 * s * 4;  // local + prefix states
  if (m.walk) bytes += lasp::kWalkSyncBytes;
  return (bytes + 255) & ~(size_t)255;
}

// one launch per direction when the CTAs of a launch can all be resident (or do not depend on each other)
bool fusable(const lasp::Dims& m) {
  return m.walk && !unfused_requested() && (m.nc == 1 || m.b * m.h * m.nc <= lasp::sm_count());
}

int check_fwd(const lasp_problem* p, const lasp_fwd_args* a, lasp::Dims* m, bool need_qo) {
  int st = make_dims(p, m);
  if (st != LASP_OK) return st;
  if (!a || !a->k || !a->v || !a->s || !a->ws) return LASP_ERR_NULL;
  if (need_qo && (!a->q || !a->o)) return LASP_ERR_NULL;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o) || !aligned16(a->kv_in) ||
      !aligned16(a->kv_out) || !aligned16(a->ws))
    return LASP_ERR_ALIGN;
  if (a->ws_bytes < workspace_bytes(*m)) return LASP_ERR_WORKSPACE;
  return LASP_OK;
}

int check_bwd(const lasp_problem* p, const lasp_bwd_args* a, lasp::Dims* m, bool need_all) {
  int st = make_dims(p, m);
  if (st != LASP_OK) return st;
  if (!a || !a->q || !a->d_o || !a->s || !a->ws) return LASP_ERR_NULL;
  if (need_all && (!a->k || !a->v || !a->dq || !a->dk || !a->dv || !a->fwd_ws)) return LASP_ERR_NULL;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->d_o) || !aligned16(a->dq) ||
      !aligned16(a->dk) || !aligned16(a->dv) || !aligned16(a->dkv_in) || !aligned16(a->dkv_out) ||
      !aligned16(a->ws) || !aligned16(a->fwd_ws))
    return LASP_ERR_ALIGN;
  if (a->ws_bytes < workspace_bytes(*m)) return LASP_ERR_WORKSPACE;
  if (need_all && a->fwd_ws_bytes < workspace_bytes(*m)) return LASP_ERR_WORKSPACE;
  return LASP_OK;
}

}  // namespace

extern "C" {

int lasp_b200_abi_version(void) { return LASP_B200_ABI_VERSION; }

const char* lasp_b200_strerror(int status) {
  switch (status) {
    case LASP_OK: return "ok";
    case LASP_ERR_NULL: return "a required pointer is NULL";
    case LASP_ERR_SHAPE: return "unsupported shape (need b,h,n > 0; d,e multiples of 16 up to 128; b*h <= 65535)";
    case LASP_ERR_DTYPE: return "unknown dtype";
    case LASP_ERR_ALIGN: return "pointer not 16-byte aligned";
    case LASP_ERR_WORKSPACE: return "workspace too small";
    case LASP_ERR_CUDA: return "CUDA runtime error";
    case LASP_ERR_PATH: return "requested kernel path cannot run this problem";
    case LASP_ERR_DEVICE: return "a kernel reported a fault";
    case LASP_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
    default: return "unknown status";
  }
}

const char* lasp_b200_last_cuda_error(void) { return g_cuda_error; }

int lasp_b200_resolve_path(const lasp_problem* p) {
  lasp::Dims m;
  int st = make_dims(p, &m);
  return st != LASP_OK ? st : m.path;
}

int lasp_b200_chunk_tokens(const lasp_problem* p) {
  lasp::Dims m;
  int st = make_dims(p, &m);
  return st != LASP_OK ? st : m.chunk;
}

size_t lasp_b200_fwd_workspace_bytes(const lasp_problem* p) {
  lasp::Dims m;
  return make_dims(p, &m) == LASP_OK ? workspace_bytes(m) : 0;
}

size_t lasp_b200_bwd_workspace_bytes(const lasp_problem* p) { return lasp_b200_fwd_workspace_bytes(p); }

}  // extern "C"

namespace {

int fwd_chunk_states(const lasp::Dims& m, const lasp_fwd_args* a, cudaStream_t cs) {
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  if (m.walk) return cuda_fail(lasp::walk_span_totals(m, a->k, a->v, a->s, lasp::ws_local(a->ws, m), false, cs));
  return cuda_fail(lasp::simt_chunk_states(m, a->k, a->v, a->s, lasp::ws_local(a->ws, m), false, cs));
}

int fwd_scan(const lasp::Dims& m, const lasp_fwd_args* a, cudaStream_t cs) {
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  return cuda_fail(lasp::scan_states(m, a->s, lasp::ws_local(a->ws, m), lasp::ws_prefix(a->ws, m), a->kv_in, a->kv_out,
                                     false, cs));
}

int fwd_output(const lasp::Dims& m, const lasp_fwd_args* a, cudaStream_t cs) {
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  if (m.walk)
    return cuda_fail(lasp::walk_fwd_output(m, a->q, a->k, a->v, a->s, lasp::ws_walk_border(a->ws, m),
                                           lasp::ws_walk_sync(a->ws), a->o, cs));
  return cuda_fail(lasp::simt_fwd_output(m, a->q, a->k, a->v, a->s, lasp::ws_prefix(a->ws, m), a->o, cs));
}

int bwd_chunk_states(const lasp::Dims& m, const lasp_bwd_args* a, cudaStream_t cs) {
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  if (m.walk) return cuda_fail(lasp::walk_span_totals(m, a->q, a->d_o, a->s, lasp::ws_local(a->ws, m), true, cs));
  return cuda_fail(lasp::simt_chunk_states(m, a->q, a->d_o, a->s, lasp::ws_local(a->ws, m), true, cs));
}

int bwd_scan(const lasp::Dims& m, const lasp_bwd_args* a, cudaStream_t cs) {
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  return cuda_fail(lasp::scan_states(m, a->s, lasp::ws_local(a->ws, m), lasp::ws_prefix(a->ws, m), a->dkv_in,
                                     a->dkv_out, true, cs));
}

int bwd_grads(const lasp::Dims& m, const lasp_bwd_args* a, cudaStream_t cs) {
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  if (m.walk) {
    // dQ walks forward over the border states the forward pass left in its workspace; dK, dV walk backward
    int st = cuda_fail(lasp::walk_bwd_dq(m, a->q, a->k, a->v, a->d_o, a->s, lasp::ws_walk_border(a->fwd_ws, m),
                                          lasp::ws_walk_sync(a->fwd_ws), a->dq, cs));
    if (st != LASP_OK) return st;
    return cuda_fail(lasp::walk_bwd_dkv(m, a->q, a->k, a->v, a->d_o, a->s, lasp::ws_walk_border(a->ws, m), a->dk,
                                        a->dv, cs));
  }
  return cuda_fail(lasp::simt_bwd_grads(m, a->q, a->k, a->v, a->d_o, a->s, lasp::ws_prefix(a->fwd_ws, m),
                                        lasp::ws_prefix(a->ws, m), a->dq, a->dk, a->dv, cs));
}

}  // namespace

extern "C" {

// ---- forward --------------------------------------------------------------
int lasp_b200_fwd_chunk_states(const lasp_problem* p, const lasp_fwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_fwd(p, a, &m, false);
  return st != LASP_OK ? st : fwd_chunk_states(m, a, static_cast<cudaStream_t>(stream));
}

int lasp_b200_fwd_scan(const lasp_problem* p, const lasp_fwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_fwd(p, a, &m, false);
  return st != LASP_OK ? st : fwd_scan(m, a, static_cast<cudaStream_t>(stream));
}

int lasp_b200_fwd_output(const lasp_problem* p, const lasp_fwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_fwd(p, a, &m, true);
  return st != LASP_OK ? st : fwd_output(m, a, static_cast<cudaStream_t>(stream));
}

int lasp_b200_forward(const lasp_problem* p, const lasp_fwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_fwd(p, a, &m, true);
  if (st != LASP_OK) return st;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (fusable(m))
    return cuda_fail(lasp::walk_fwd_fused(m, a->q, a->k, a->v, a->s, a->kv_in, a->kv_out, lasp::ws_walk_sync(a->ws),
                                          lasp::ws_walk_totals(a->ws), lasp::ws_walk_border(a->ws, m), a->o, nullptr,
                                          cs));
  if ((st = fwd_chunk_states(m, a, cs)) != LASP_OK) return st;
  if ((st = fwd_scan(m, a, cs)) != LASP_OK) return st;
  return fwd_output(m, a, cs);
}

// ---- backward -------------------------------------------------------------
int lasp_b200_bwd_chunk_states(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, false);
  return st != LASP_OK ? st : bwd_chunk_states(m, a, static_cast<cudaStream_t>(stream));
}

int lasp_b200_bwd_scan(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, false);
  return st != LASP_OK ? st : bwd_scan(m, a, static_cast<cudaStream_t>(stream));
}

int lasp_b200_bwd_grads(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, true);
  return st != LASP_OK ? st : bwd_grads(m, a, static_cast<cudaStream_t>(stream));
}

// The two launches of the tensor-core backward, separately (the fp32 path has one gradient kernel: there
// lasp_b200_bwd_dq does nothing and lasp_b200_bwd_dkv is the whole backward).
int lasp_b200_bwd_dq(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, true);
  if (st != LASP_OK || !m.walk) return st;
  return cuda_fail(lasp::walk_bwd_dq(m, a->q, a->k, a->v, a->d_o, a->s, lasp::ws_walk_border(a->fwd_ws, m),
                                          lasp::ws_walk_sync(a->fwd_ws), a->dq,
                                     static_cast<cudaStream_t>(stream)));
}

int lasp_b200_bwd_dkv_walk(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, true);
  if (st != LASP_OK) return st;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (!m.walk) return bwd_grads(m, a, cs);
  if (lasp::has_qk_preprocessing(m)) return LASP_ERR_PATH;
  return cuda_fail(lasp::walk_bwd_dkv(m, a->q, a->k, a->v, a->d_o, a->s, lasp::ws_walk_border(a->ws, m), a->dk, a->dv,
                                      cs));
}

int lasp_b200_bwd_dkv(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, true);
  if (st != LASP_OK) return st;
  if (!fusable(m)) return lasp_b200_backward(p, a, stream);
  return cuda_fail(lasp::walk_bwd_dkv_fused(m, a->q, a->k, a->v, a->d_o, a->s, a->dkv_in, a->dkv_out,
                                            lasp::ws_walk_sync(a->ws), lasp::ws_walk_totals(a->ws), a->dk, a->dv,
                                            nullptr, static_cast<cudaStream_t>(stream)));
}

int lasp_b200_backward(const lasp_problem* p, const lasp_bwd_args* a, void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, true);
  if (st != LASP_OK) return st;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (fusable(m)) {
    // dQ walks forward over the border states the forward pass kept; dK, dV walk backward in one fused launch
    if ((st = cuda_fail(lasp::walk_bwd_dq(m, a->q, a->k, a->v, a->d_o, a->s, lasp::ws_walk_border(a->fwd_ws, m),
                                          lasp::ws_walk_sync(a->fwd_ws), a->dq,
                                          cs))) != LASP_OK)
      return st;
    return cuda_fail(lasp::walk_bwd_dkv_fused(m, a->q, a->k, a->v, a->d_o, a->s, a->dkv_in, a->dkv_out,
                                              lasp::ws_walk_sync(a->ws), lasp::ws_walk_totals(a->ws), a->dk, a->dv,
                                              nullptr, cs));
  }
  if ((st = bwd_chunk_states(m, a, cs)) != LASP_OK) return st;
  if ((st = bwd_scan(m, a, cs)) != LASP_OK) return st;
  return bwd_grads(m, a, cs);
}

int lasp_b200_state_combine(int b, int h, int d, int e, int n, const float* s, const float* x_in,
                            const float* x_local, float* x_out, void* stream) {
  if (!s || !x_local || !x_out) return LASP_ERR_NULL;
  if (b <= 0 || h <= 0 || d <= 0 || e <= 0 || n < 0 || (d * e) % 4 || (long long)b * h > 65535) return LASP_ERR_SHAPE;
  if (!aligned16(x_in) || !aligned16(x_local) || !aligned16(x_out)) return LASP_ERR_ALIGN;
  return cuda_fail(lasp::state_combine(b, h, d, e, n, s, x_in, x_local, x_out, static_cast<cudaStream_t>(stream)));
}

// checks of the peer-mapped buffers shared by the hand-over entry points
static int check_link(const lasp_exchange_args* a) {
  if (!a || !a->counters) return LASP_ERR_NULL;
  if (a->ranks < 2 || a->ranks > 8 || a->position < 0 || a->position >= a->ranks) return LASP_ERR_SHAPE;
  if (a->position > 0 && !a->my_slots) return LASP_ERR_NULL;
  if (a->position < a->ranks - 1 && !a->my_acks) return LASP_ERR_NULL;
  for (int q = 0; q < a->ranks; ++q) {
    if (q < a->position && !a->peer_acks[q]) return LASP_ERR_NULL;
    if (q > a->position && !a->peer_slots[q]) return LASP_ERR_NULL;
  }
  if (!aligned16(a->my_slots)) return LASP_ERR_ALIGN;
  return LASP_OK;
}

int lasp_b200_linked_ok(const lasp_problem* p) {
  lasp::Dims m;
  int st = make_dims(p, &m);
  if (st != LASP_OK) return st;
  return (m.walk && !unfused_requested() && m.b * m.h * m.nc <= lasp::sm_count()) ? 1 : 0;
}

int lasp_b200_forward_linked(const lasp_problem* p, const lasp_fwd_args* a, const lasp_exchange_args* x,
                             void* stream) {
  lasp::Dims m;
  int st = check_fwd(p, a, &m, true);
  if (st != LASP_OK) return st;
  if ((st = check_link(x)) != LASP_OK) return st;
  if (lasp_b200_linked_ok(p) != 1) return LASP_ERR_PATH;
  return cuda_fail(lasp::walk_fwd_fused(m, a->q, a->k, a->v, a->s, nullptr, nullptr, lasp::ws_walk_sync(a->ws),
                                        lasp::ws_walk_totals(a->ws), lasp::ws_walk_border(a->ws, m), a->o, x,
                                        static_cast<cudaStream_t>(stream)));
}

int lasp_b200_bwd_dkv_linked(const lasp_problem* p, const lasp_bwd_args* a, const lasp_exchange_args* x,
                             void* stream) {
  lasp::Dims m;
  int st = check_bwd(p, a, &m, true);
  if (st != LASP_OK) return st;
  if ((st = check_link(x)) != LASP_OK) return st;
  if (lasp_b200_linked_ok(p) != 1) return LASP_ERR_PATH;
  return cuda_fail(lasp::walk_bwd_dkv_fused(m, a->q, a->k, a->v, a->d_o, a->s, nullptr, nullptr,
                                            lasp::ws_walk_sync(a->ws), lasp::ws_walk_totals(a->ws), a->dk, a->dv, x,
                                            static_cast<cudaStream_t>(stream)));
}

int lasp_b200_exchange_scan(const lasp_problem* p, const lasp_exchange_args* a, void* stream) {
  lasp::Dims m;
  int st = make_dims(p, &m);
  if (st != LASP_OK) return st;
  if (!a || !a->s || !a->ws || !a->counters) return LASP_ERR_NULL;
  if (a->ranks < 2 || a->ranks > 8 || a->position < 0 || a->position >= a->ranks) return LASP_ERR_SHAPE;
  if (a->phase < LASP_EXCHANGE_BOTH || a->phase > LASP_EXCHANGE_GATHER) return LASP_ERR_SHAPE;
  if ((m.d * m.e) % 4) return LASP_ERR_SHAPE;
  if (a->position > 0 && !a->my_slots) return LASP_ERR_NULL;
  if (a->position < a->ranks - 1 && !a->my_acks) return LASP_ERR_NULL;
  for (int q = 0; q < a->ranks; ++q) {
    if (q < a->position && !a->peer_acks[q]) return LASP_ERR_NULL;
    if (q > a->position && !a->peer_slots[q]) return LASP_ERR_NULL;
  }
  if (!aligned16(a->ws) || !aligned16(a->my_slots)) return LASP_ERR_ALIGN;
  if (a->ws_bytes < workspace_bytes(m)) return LASP_ERR_WORKSPACE;
  return cuda_fail(lasp::exchange_scan(m, *a, lasp::ws_local(a->ws, m), lasp::ws_prefix(a->ws, m),
                                       static_cast<cudaStream_t>(stream)));
}

int lasp_b200_copy_status_async(int32_t* status_host_pinned, void* stream) {
  if (!status_host_pinned) return LASP_ERR_NULL;
  bind_context_once();
  int32_t* word = nullptr;
  cudaError_t err = lasp::fault_word_address(&word);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(status_host_pinned, word, sizeof(int32_t), cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(stream));
  return cuda_fail(err);
}

int lasp_b200_read_status(int32_t* status_host, int clear, void* stream) {
  if (!status_host) return LASP_ERR_NULL;
  return cuda_fail(lasp::read_fault_word(status_host, clear != 0, static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
