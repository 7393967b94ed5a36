"""The C-ABI library loads on a machine without a GPU, exports every symbol the
header declares, and rejects bad arguments before launching anything."""
import ctypes as C
import os
import re

import pytest

from lasp_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_cabi.LIB_PATH):
        from lasp_b200.build import build
        build()
    return _cabi.load()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "lasp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lasp_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = header_symbols()
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), name
        assert name in _cabi.SIGNATURES, f"{name} declared in the header but not bound in _cabi.SIGNATURES"
    assert sorted(_cabi.SIGNATURES) == names


def test_abi_version_and_strerror(lib):
    assert lib.lasp_b200_abi_version() == _cabi.ABI_VERSION
    assert lib.lasp_b200_strerror(0) == b"ok"
    for code in range(-9, 0):
        assert lib.lasp_b200_strerror(code) != b"unknown status"


def _problem(**kw):
    base = dict(b=2, h=3, n=256, d=64, e=64, dtype=_cabi.F32, path=_cabi.PATH_AUTO, qk_map=0, qk_scale=0.0)
    base.update(kw)
    return _cabi.Problem(**base)


def test_problem_validation(lib):
    assert lib.lasp_b200_resolve_path(C.byref(_problem())) == _cabi.PATH_SIMT
    assert lib.lasp_b200_chunk_tokens(C.byref(_problem())) == 64
    assert lib.lasp_b200_resolve_path(C.byref(_problem(d=24))) == -2       # not a multiple of 16
    assert lib.lasp_b200_resolve_path(C.byref(_problem(e=256))) == -2      # wider than one slice
    assert lib.lasp_b200_resolve_path(C.byref(_problem(n=0))) == -2
    assert lib.lasp_b200_resolve_path(C.byref(_problem(dtype=7))) == -3
    assert lib.lasp_b200_resolve_path(C.byref(_problem(path=9))) == -7
    # fp32 cannot run on the tensor-core path
    assert lib.lasp_b200_resolve_path(C.byref(_problem(path=_cabi.PATH_TENSOR))) == -7
    assert lib.lasp_b200_resolve_path(None) == -1


def test_workspace_size(lib):
    p = _problem(n=200)  # 4 chunks of 64
    # local + prefix states
    assert lib.lasp_b200_fwd_workspace_bytes(C.byref(p)) == 2 * 2 * 3 * 4 * 64 * 64 * 4
    assert lib.lasp_b200_bwd_workspace_bytes(C.byref(p)) == 2 * 2 * 3 * 4 * 64 * 64 * 4
    assert lib.lasp_b200_fwd_workspace_bytes(C.byref(_problem(d=20))) == 0


def test_argument_checks_come_before_any_launch(lib):
    p = _problem()
    args = _cabi.FwdArgs()
    assert lib.lasp_b200_forward(C.byref(p), C.byref(args), None) == -1          # NULL pointers
    args = _cabi.FwdArgs(q=4096, k=4096, v=4096, s=4096, o=4096, ws=4104, ws_bytes=1 << 40)
    assert lib.lasp_b200_forward(C.byref(p), C.byref(args), None) == -4          # ws misaligned
    args = _cabi.FwdArgs(q=4096, k=4096, v=4096, s=4096, o=4096, ws=4096, ws_bytes=16)
    assert lib.lasp_b200_forward(C.byref(p), C.byref(args), None) == -5          # ws too small
    bargs = _cabi.BwdArgs()
    assert lib.lasp_b200_backward(C.byref(p), C.byref(bargs), None) == -1
    assert lib.lasp_b200_state_combine(1, 1, 16, 16, 4, None, None, None, None, None) == -1
    with pytest.raises(_cabi.LaspStatusError):
        _cabi.call("lasp_b200_forward", C.byref(p), C.byref(_cabi.FwdArgs()), None)


def test_operators_refuse_cpu_tensors():
    import torch
    from lasp_b200 import lightning_attn
    q = torch.randn(1, 1, 64, 16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        lightning_attn(q, q, q, torch.zeros(1, 1, 1))


def test_exchange_argument_checks(lib):
    p = _problem()
    a = _cabi.ExchangeArgs()
    assert lib.lasp_b200_exchange_scan(C.byref(p), C.byref(a), None) == -1               # NULL pointers
    assert lib.lasp_b200_exchange_scan(None, C.byref(a), None) == -1
    a.s, a.ws, a.counters, a.ws_bytes = 4096, 4096, 4096, 1 << 40
    a.ranks, a.position = 9, 0
    assert lib.lasp_b200_exchange_scan(C.byref(p), C.byref(a), None) == -2               # more than 8 ranks
    a.ranks, a.position = 4, 4
    assert lib.lasp_b200_exchange_scan(C.byref(p), C.byref(a), None) == -2               # position outside the group
    a.ranks, a.position = 4, 1
    assert lib.lasp_b200_exchange_scan(C.byref(p), C.byref(a), None) == -1               # position > 0 needs its slots
    a.my_slots = 4096
    assert lib.lasp_b200_exchange_scan(C.byref(p), C.byref(a), None) == -1               # missing ack / peer pointers
    a.my_acks = 4096
    for q in range(4):
        a.peer_acks[q], a.peer_slots[q] = 4096, 4096
    a.ws_bytes = 16
    assert lib.lasp_b200_exchange_scan(C.byref(p), C.byref(a), None) == -5               # workspace too small
    assert lib.lasp_b200_copy_status_async(None, None) == -1
