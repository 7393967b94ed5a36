"""ctypes binding of liblasp_b200.so (declared in include/lasp_b200.h).

The library is the product: there is no CPU or torch fallback.  Importing this
module never fails, but the first call that needs the library raises
``LaspLibraryError`` when it has not been built (``python -m lasp_b200.build``).
"""
from __future__ import annotations

import ctypes as C
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "liblasp_b200.so")
ABI_VERSION = 3

# lasp_dtype / lasp_path / lasp_status of include/lasp_b200.h
F32, BF16, F16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2
EXCHANGE_BOTH, EXCHANGE_PUSH, EXCHANGE_GATHER = 0, 1, 2
OK = 0


class LaspLibraryError(RuntimeError):
    """liblasp_b200.so is missing, stale or failed to load."""


class LaspStatusError(RuntimeError):
    """A C-ABI call returned a negative lasp_status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed: {text} (status {status})")
        self.status = status


class Problem(C.Structure):   # lasp_problem
    _fields_ = ([(n, C.c_int32) for n in ("b", "h", "n", "d", "e", "dtype", "path", "qk_map")] + [("qk_scale", C.c_float)]
                + [(n, C.c_int32) for n in ("pitch_d", "pitch_e")])


QK_MAPS = {None: 0, "identity": 0, "elu1": 1}   # lasp_qk_map


class FwdArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("s", C.c_void_p),
                ("kv_in", C.c_void_p), ("kv_out", C.c_void_p), ("o", C.c_void_p),
                ("ws", C.c_void_p), ("ws_bytes", C.c_size_t)]


class BwdArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("d_o", C.c_void_p),
                ("s", C.c_void_p), ("dkv_in", C.c_void_p), ("dkv_out", C.c_void_p),
                ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
                ("fwd_ws", C.c_void_p), ("fwd_ws_bytes", C.c_size_t),
                ("ws", C.c_void_p), ("ws_bytes", C.c_size_t)]


class ExchangeArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("ranks", "position", "reverse", "phase")] + \
               [("s", C.c_void_p), ("ws", C.c_void_p), ("ws_bytes", C.c_size_t)] + \
               [(n, C.c_void_p) for n in ("my_slots", "my_acks", "counters")] + \
               [("peer_slots", C.c_void_p * 8), ("peer_acks", C.c_void_p * 8), ("wait_clocks", C.c_int64)]


_PP, _FP, _BP = C.POINTER(Problem), C.POINTER(FwdArgs), C.POINTER(BwdArgs)

# symbol -> (restype, argtypes); every entry point include/lasp_b200.h declares
SIGNATURES = {
    "lasp_b200_abi_version": (C.c_int, []),
    "lasp_b200_strerror": (C.c_char_p, [C.c_int]),
    "lasp_b200_last_cuda_error": (C.c_char_p, []),
    "lasp_b200_resolve_path": (C.c_int, [_PP]),
    "lasp_b200_chunk_tokens": (C.c_int, [_PP]),
    "lasp_b200_fwd_workspace_bytes": (C.c_size_t, [_PP]),
    "lasp_b200_bwd_workspace_bytes": (C.c_size_t, [_PP]),
    "lasp_b200_fwd_chunk_states": (C.c_int, [_PP, _FP, C.c_void_p]),
    "lasp_b200_fwd_scan": (C.c_int, [_PP, _FP, C.c_void_p]),
    "lasp_b200_fwd_output": (C.c_int, [_PP, _FP, C.c_void_p]),
    "lasp_b200_forward": (C.c_int, [_PP, _FP, C.c_void_p]),
    "lasp_b200_bwd_chunk_states": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_bwd_scan": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_bwd_grads": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_backward": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_bwd_dq": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_bwd_dkv": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_bwd_dkv_walk": (C.c_int, [_PP, _BP, C.c_void_p]),
    "lasp_b200_state_combine": (C.c_int, [C.c_int] * 5 + [C.c_void_p] * 5),
    "lasp_b200_read_status": (C.c_int, [C.POINTER(C.c_int32), C.c_int, C.c_void_p]),
    "lasp_b200_copy_status_async": (C.c_int, [C.c_void_p, C.c_void_p]),
    "lasp_b200_forward_static": (C.c_int, [_PP, _FP, C.c_void_p]),
    "lasp_b200_exchange_scan": (C.c_int, [_PP, C.POINTER(ExchangeArgs), C.c_void_p]),
    "lasp_b200_linked_ok": (C.c_int, [_PP]),
    "lasp_b200_forward_linked": (C.c_int, [_PP, _FP, C.POINTER(ExchangeArgs), C.c_void_p]),
    "lasp_b200_bwd_dkv_linked": (C.c_int, [_PP, _BP, C.POINTER(ExchangeArgs), C.c_void_p]),
}
STATIC_SCRATCH_BYTES = 64 << 20  # LASP_B200_STATIC_SCRATCH_BYTES

_lib = None


def load() -> C.CDLL:
    """Load the library once and type every symbol; raises LaspLibraryError."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LaspLibraryError(f"{LIB_PATH} not found: build it with `python -m lasp_b200.build` "
                               "(there is no CPU fallback)")
    try:
        lib = C.CDLL(LIB_PATH)
    except OSError as exc:
        raise LaspLibraryError(f"cannot load {LIB_PATH}: {exc}") from exc
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise LaspLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from exc
        fn.restype, fn.argtypes = res, args
    if lib.lasp_b200_abi_version() != ABI_VERSION:
        raise LaspLibraryError(f"{LIB_PATH} has ABI {lib.lasp_b200_abi_version()}, expected {ABI_VERSION}; rebuild")
    _lib = lib
    return lib


def check(fn: str, status: int) -> None:
    if status >= 0:
        return
    lib = load()
    text = lib.lasp_b200_strerror(status).decode()
    if status == -6:
        text += ": " + lib.lasp_b200_last_cuda_error().decode()
    raise LaspStatusError(fn, status, text)


def call(fn: str, *args) -> int:
    """Call an int-returning entry point; negative status -> LaspStatusError."""
    status = getattr(load(), fn)(*args)
    check(fn, status)
    return status
