"""The forward entry point that allocates nothing (lasp_b200_forward_static).

A host that has given all GPU memory to its own pool, or that may not call
cudaMalloc where it invokes the operator, has no workspace to pass.  This
entry point keeps the chunk-state workspace in a fixed array inside the
library.  The test calls it through the C ABI twice in a row (the array is
shared and keeps the previous call's contents, so the second call must not be
disturbed by the first) and compares with the ordinary forward; it also checks
that an oversized problem is refused.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from lasp_b200 import _cabi, engine
from oracle import lasp_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _forward_static(plan, q, k, v, s, kv_in, kv_out):
    o = torch.empty(plan.b, plan.h, plan.n, plan.e, dtype=q.dtype, device=q.device)
    args = _cabi.FwdArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), s.data_ptr(),
                         kv_in.data_ptr() if kv_in is not None else None,
                         kv_out.data_ptr() if kv_out is not None else None, o.data_ptr(), None, 0)
    _cabi.call("lasp_b200_forward_static", C.byref(plan.problem), C.byref(args),
               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return o


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 2e-2)])
def test_static_scratch_forward_matches_ordinary_forward_twice(dtype, tol):
    s_host = O.baseline_slopes(4)
    s = s_host.reshape(-1).to(DEV)
    shapes = [(2, 4, 333, 64, 48), (1, 4, 512, 128, 128)]   # two different problems share the array
    for rep in range(2):
        for i, (b, h, n, d, e) in enumerate(shapes):
            q, k, v, _ = O.make_inputs(50 + 10 * rep + i, b, h, n, d, e)
            q, k, v = (t.to(DEV, dtype) for t in (q, k, v))
            kv_in = torch.randn(b, h, d, e, device=DEV)
            plan = engine.make_plan(b, h, n, d, e, dtype)
            kv_ref = torch.empty_like(kv_in)
            o_ref = engine.Forward(plan, q, k, v, s, kv_in=kv_in, kv_out=kv_ref).run()
            kv_got = torch.empty_like(kv_in)
            o_got = _forward_static(plan, q, k, v, s, kv_in, kv_got)
            torch.cuda.synchronize()
            assert O.max_rel_err(o_got, o_ref) < tol, (rep, i)
            assert O.max_rel_err(kv_got, kv_ref) < tol, (rep, i)
            # and against the CPU oracle, so both entry points cannot be wrong together
            o_cpu, kv_cpu = O.blocked_forward(q.float().cpu(), k.float().cpu(), v.float().cpu(), s_host, kv_in.cpu())
            assert O.max_rel_err(o_got, o_cpu) < tol
            assert O.max_rel_err(kv_got, kv_cpu) < tol


def test_static_scratch_refuses_oversized_problem():
    b, h, n, d, e = 8, 16, 4096, 128, 128            # workspace far beyond the fixed array
    plan = engine.make_plan(b, h, n, d, e, torch.float32)
    assert plan.ws_bytes > _cabi.STATIC_SCRATCH_BYTES
    t = torch.empty(16, device=DEV)
    args = _cabi.FwdArgs(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, None, t.data_ptr(), None, 0)
    rc = _cabi.load().lasp_b200_forward_static(C.byref(plan.problem), C.byref(args), None)
    assert rc == -9                                   # LASP_ERR_TOO_LARGE, nothing launched
    assert b"capacity" in _cabi.load().lasp_b200_strerror(rc)
