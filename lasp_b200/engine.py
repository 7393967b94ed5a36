"""Torch-facing launcher of the C-ABI kernels.

Takes contiguous CUDA tensors, fills the ``lasp_problem`` / ``lasp_fwd_args`` /
``lasp_bwd_args`` structures of include/lasp_b200.h and calls the library on
torch's current stream.  PyTorch is used for device memory and streams only.

This module is what the five operators call; it plays the role of the
reference's launchers ``lasp_forward`` / ``lasp_backward``
(lasp/lasp_fuse_parallel.py:833-944, 947-1070).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch

from . import _cabi
from ._cabi import LaspLibraryError, LaspStatusError  # noqa: F401  (what the calls below raise)

_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}
_PATHS = {"auto": _cabi.PATH_AUTO, "simt": _cabi.PATH_SIMT, "tensor": _cabi.PATH_TENSOR}


def default_path() -> str:
    """Kernel path used when an operator is not told one: env LASP_B200_PATH or 'auto'."""
    return os.environ.get("LASP_B200_PATH", "auto")


@dataclass
class Plan:
    """A validated problem: shape, dtype, resolved kernel path, workspace size."""
    problem: _cabi.Problem
    b: int
    h: int
    n: int
    d: int
    e: int
    path: int           # _cabi.PATH_SIMT or _cabi.PATH_TENSOR
    chunk: int          # tokens per chunk state
    ws_bytes: int

    @property
    def path_name(self) -> str:
        return "tensor" if self.path == _cabi.PATH_TENSOR else "simt"


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _check_layout(plan, **tensors):
    """Every (b,h,n,width) tensor of a call must have the row pitch the plan was made for (the kernels address it
    by that pitch alone): raises instead of letting a kernel write past a buffer."""
    for name, t in tensors.items():
        if t is None:
            continue
        wide = name in ("v", "o", "do", "dv")
        width = plan.e if wide else plan.d
        pitch = (plan.problem.pitch_e if wide else plan.problem.pitch_d) or width
        want = (plan.h * plan.n * pitch, plan.n * pitch, pitch, 1)
        # (the stride of a dimension of extent 1 is never used and may be anything)
        strides_ok = all(st == w or ext == 1 for st, w, ext in zip(t.stride(), want, t.shape))
        if tuple(t.shape) != (plan.b, plan.h, plan.n, width) or not strides_ok:
            raise ValueError(f"{name}: shape {tuple(t.shape)} strides {tuple(t.stride())}; this plan needs shape "
                             f"{(plan.b, plan.h, plan.n, width)} with strides {want}")


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _on_device:
    """Make ``device`` current for the duration of a library call.  Backward
    runs on autograd's worker threads, whose current device need not be the
    tensors' device; the library launches on the calling thread's device."""

    def __init__(self, device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        self.prev = torch.cuda._exchange_device(self.idx)

    def __exit__(self, *exc):
        torch.cuda._maybe_exchange_device(self.prev)
        return False


_NVTX = os.environ.get("LASP_B200_NVTX", "0") == "1"


class _traced:
    """NVTX range around a library call (LASP_B200_NVTX=1), for timeline tools."""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        return False


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lasp_b200 runs on CUDA tensors only (there is no CPU fallback); "
                               f"got a tensor on {t.device}")


def make_plan(b: int, h: int, n: int, d: int, e: int, dtype: torch.dtype, path: str | None = None,
              qk_scale: float = 1.0, feature_map: str | None = None, pitch_d: int = 0, pitch_e: int = 0) -> Plan:
    """``qk_scale`` / ``feature_map`` ("elu1"): the operator is evaluated on qk_scale * map(q), qk_scale * map(k)
    inside the kernels (lasp_problem.qk_map, .qk_scale); raises LaspStatusError when the problem's kernels
    cannot do that.  ``pitch_d`` / ``pitch_e``: row pitch in elements of q,k,dq,dk / v,o,do,dv when they are slices
    of the head dimension of wider tensors (0: tensors of their own); tensor-core path only."""
    if dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {dtype}; use float32, bfloat16 or float16")
    name = path or default_path()
    if name not in _PATHS:
        raise ValueError(f"unknown kernel path {name!r}; use auto, simt or tensor")
    if feature_map not in _cabi.QK_MAPS:
        raise ValueError(f"unknown feature map {feature_map!r}; use None or 'elu1'")
    prob = _cabi.Problem(b, h, n, d, e, _DTYPES[dtype], _PATHS[name], _cabi.QK_MAPS[feature_map], float(qk_scale),
                         int(pitch_d), int(pitch_e))
    resolved = _cabi.call("lasp_b200_resolve_path", C.byref(prob))
    prob.path = resolved
    chunk = _cabi.call("lasp_b200_chunk_tokens", C.byref(prob))
    ws = _cabi.load().lasp_b200_fwd_workspace_bytes(C.byref(prob))
    return Plan(prob, b, h, n, d, e, resolved, chunk, ws)


SYNC_BYTES = 4096


def new_workspace(plan: Plan, device) -> torch.Tensor:
    """Workspace of a forward or backward call.  Its first 4 KB hold the words through which the CTAs of
    the fused kernels synchronise: they must be zero before the workspace is first used (the library keeps
    them consistent afterwards)."""
    ws = torch.empty(plan.ws_bytes, dtype=torch.uint8, device=device)
    ws[:SYNC_BYTES].zero_()
    return ws


def _slopes(s: torch.Tensor, h: int, device) -> torch.Tensor:
    s = s.reshape(-1)
    if s.numel() != h:
        raise ValueError(f"decay tensor has {s.numel()} entries for {h} heads")
    return s.to(device=device, dtype=torch.float32).contiguous()


class Forward:
    """One forward call split in its three phases (see include/lasp_b200.h)."""

    def __init__(self, plan: Plan, q, k, v, s, kv_in=None, kv_out=None, o=None, ws=None):
        _require_cuda(q, k, v, kv_in, kv_out)
        self.plan = plan
        self.q, self.k, self.v = q, k, v
        self.s = _slopes(s, plan.h, q.device)
        self.kv_in, self.kv_out = kv_in, kv_out
        self.o = o if o is not None else torch.empty(plan.b, plan.h, plan.n, plan.e, dtype=q.dtype, device=q.device)
        _check_layout(plan, q=q, k=k, v=v, o=self.o)
        self.ws = ws if ws is not None else new_workspace(plan, q.device)
        self._args = _cabi.FwdArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(self.s), _ptr(kv_in), _ptr(kv_out),
                                   _ptr(self.o), _ptr(self.ws), self.ws.numel())

    def _call(self, fn):
        with _on_device(self.q.device), _traced(fn):
            _cabi.call(fn, C.byref(self.plan.problem), C.byref(self._args), _stream())

    def chunk_states(self):
        self._call("lasp_b200_fwd_chunk_states")

    def scan(self):
        self._call("lasp_b200_fwd_scan")

    def output(self):
        self._call("lasp_b200_fwd_output")

    def run(self):
        self._call("lasp_b200_forward")
        return self.o

    def run_linked(self, link_args):
        """The whole forward of a sequence-parallel rank in one launch (lasp_b200_forward_linked)."""
        with _on_device(self.q.device), _traced("lasp_b200_forward_linked"):
            _cabi.call("lasp_b200_forward_linked", C.byref(self.plan.problem), C.byref(self._args),
                       C.byref(link_args), _stream())
        return self.o


class Backward:
    """One backward call split in its three phases."""

    def __init__(self, plan: Plan, q, k, v, do, s, fwd_ws, dkv_in=None, dkv_out=None, ws=None, dq=None, dk=None,
                 dv=None):
        _require_cuda(q, k, v, do, fwd_ws, dkv_in, dkv_out)
        self.plan = plan
        self.s = _slopes(s, plan.h, q.device)
        self.keep = (q, k, v, do, fwd_ws, dkv_in, dkv_out)
        self.dq = dq if dq is not None else torch.empty_like(q)
        self.dk = dk if dk is not None else torch.empty_like(k)
        self.dv = dv if dv is not None else torch.empty_like(v)
        _check_layout(plan, q=q, k=k, v=v, do=do, dq=self.dq, dk=self.dk, dv=self.dv)
        self.ws = ws if ws is not None else new_workspace(plan, q.device)
        self._args = _cabi.BwdArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(do), _ptr(self.s), _ptr(dkv_in), _ptr(dkv_out),
                                   _ptr(self.dq), _ptr(self.dk), _ptr(self.dv), _ptr(fwd_ws), fwd_ws.numel(),
                                   _ptr(self.ws), self.ws.numel())

    def _call(self, fn):
        with _on_device(self.keep[0].device), _traced(fn):
            _cabi.call(fn, C.byref(self.plan.problem), C.byref(self._args), _stream())

    def chunk_states(self):
        self._call("lasp_b200_bwd_chunk_states")

    def scan(self):
        self._call("lasp_b200_bwd_scan")

    def grads(self):
        self._call("lasp_b200_bwd_grads")

    def dq_only(self):
        self._call("lasp_b200_bwd_dq")

    def dkv_only(self):
        self._call("lasp_b200_bwd_dkv")

    def dkv_after_scan(self):
        self._call("lasp_b200_bwd_dkv_walk")

    def dkv_linked(self, link_args):
        """dK, dV of a sequence-parallel rank with the hand-over inside the launch."""
        with _on_device(self.keep[0].device), _traced("lasp_b200_bwd_dkv_linked"):
            _cabi.call("lasp_b200_bwd_dkv_linked", C.byref(self.plan.problem), C.byref(self._args),
                       C.byref(link_args), _stream())

    def run(self):
        self._call("lasp_b200_backward")
        return self.dq, self.dk, self.dv


def state_combine(s, x_in, x_local, n: int, out=None):
    """out = exp(-s n) x_in + x_local on (b,h,d,e) fp32 states."""
    _require_cuda(x_local, x_in)
    b, h, d, e = x_local.shape
    out = out if out is not None else torch.empty_like(x_local)
    with _on_device(x_local.device):
        _cabi.call("lasp_b200_state_combine", b, h, d, e, n, _ptr(_slopes(s, h, x_local.device)), _ptr(x_in),
                   _ptr(x_local), _ptr(out), _stream())
    return out


def linked_ok(plan: Plan) -> bool:
    """True when the fused kernels can do the hand-over themselves for this problem (one span per SM)."""
    return _cabi.call("lasp_b200_linked_ok", C.byref(plan.problem)) == 1


def exchange_scan(plan: Plan, args: "_cabi.ExchangeArgs", device) -> None:
    """The state hand-over of one direction (see lasp_b200_exchange_scan in include/lasp_b200.h)."""
    with _on_device(device), _traced("lasp_b200_exchange_scan"):
        _cabi.call("lasp_b200_exchange_scan", C.byref(plan.problem), C.byref(args), _stream())


def read_status(clear: bool = True) -> int:
    """Sticky kernel-fault word of the current device (synchronises)."""
    word = C.c_int32(0)
    _cabi.call("lasp_b200_read_status", C.byref(word), 1 if clear else 0, _stream())
    return word.value


class KernelFault(_cabi.LaspStatusError):
    """A kernel of the library gave up on a bounded wait (a peer that never delivered its state, a
    copy or tensor-core operation that never completed): the results of that call are not valid."""

    def __init__(self, word: int):
        names = [n for bit, n in ((1, "TMA wait"), (2, "tensor-core wait"), (4, "peer state wait"),
                                  (8, "span-total wait")) if word & bit]
        RuntimeError.__init__(self, f"lasp_b200: a kernel reported a fault ({', '.join(names) or word}); "
                                    "the outputs of that call are invalid")
        self.status = -8
        self.word = word


def check_faults(clear: bool = True) -> None:
    """Synchronise the current stream and raise KernelFault if any kernel of this device has reported
    a fault since the word was last cleared."""
    word = read_status(clear=clear)
    if word:
        raise KernelFault(word)


class _FaultWatch:
    """Notices a fault without stalling the stream: `arm()` enqueues a copy of the fault word to pinned
    memory behind the work just launched; `poll()` (called at the start of the next operator call)
    looks at it once that copy has completed, and raises."""

    def __init__(self):
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = None

    def arm(self, device) -> None:
        with _on_device(device):
            _cabi.call("lasp_b200_copy_status_async", C.c_void_p(self.host.data_ptr()), _stream())
            self.event = torch.cuda.Event()
            self.event.record()

    def poll(self) -> None:
        if self.event is not None and self.event.query():
            self.event = None
            word = int(self.host.item())
            if word:
                self.host.zero_()
                raise KernelFault(word)


_watches = {}


def fault_watch(device) -> _FaultWatch:
    key = torch.device(device).index
    if key not in _watches:
        _watches[key] = _FaultWatch()
    return _watches[key]
