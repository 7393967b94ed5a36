"""Stand-in for lasp_b200.engine used ONLY by the CPU host-logic tests.

It has the launcher's interface (make_plan, Forward, Backward with the same
phase methods) and computes with the oracle, so that the gloo ranks exercise
the operators' group lookup, buffer handling and message order without a GPU.
It is never importable from the package.
"""
import types

import torch

from oracle import lasp_oracle as O


def make_plan(b, h, n, d, e, dtype, path=None):
    if d % 16 or e % 16 or d > 128 or e > 128:
        raise ValueError("unsupported shape")
    return types.SimpleNamespace(b=b, h=h, n=n, d=d, e=e, dtype=dtype)


class Forward:
    def __init__(self, plan, q, k, v, s, kv_in=None, kv_out=None, o=None, ws=None):
        self.plan, self.q, self.k, self.v, self.s = plan, q, k, v, s
        self.kv_in, self.kv_out = kv_in, kv_out
        self.o = torch.empty(plan.b, plan.h, plan.n, plan.e, dtype=q.dtype)
        self.ws = {}
        self.calls = []

    def chunk_states(self):
        self.calls.append("chunk_states")
        _, self.ws["local"] = O.blocked_forward(self.q, self.k, self.v, self.s)

    def scan(self):
        assert self.calls == ["chunk_states"]
        self.calls.append("scan")
        self.ws["kv_in"] = None if self.kv_in is None else self.kv_in.clone()
        if self.kv_out is not None:
            dec = torch.exp(-self.s.reshape(1, -1, 1, 1).float() * self.plan.n)
            prev = 0 if self.kv_in is None else dec * self.kv_in
            self.kv_out.copy_(prev + self.ws["local"])

    def output(self):
        assert self.calls == ["chunk_states", "scan"]
        self.calls.append("output")
        o, _ = O.blocked_forward(self.q, self.k, self.v, self.s, self.ws["kv_in"])
        self.o.copy_(o.to(self.o.dtype))

    def run(self):
        self.chunk_states(), self.scan(), self.output()
        return self.o


class Backward:
    def __init__(self, plan, q, k, v, do, s, fwd_ws, dkv_in=None, dkv_out=None, ws=None):
        self.plan, self.q, self.k, self.v, self.do, self.s = plan, q, k, v, do, s
        self.fwd_ws, self.dkv_in, self.dkv_out = fwd_ws, dkv_in, dkv_out
        self.dq, self.dk, self.dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        self.calls = []

    def chunk_states(self):
        self.calls.append("chunk_states")
        *_, self.local = O.blocked_backward(self.q, self.k, self.v, self.s, self.do)

    def scan(self):
        assert self.calls == ["chunk_states"]
        self.calls.append("scan")
        self.saved_in = None if self.dkv_in is None else self.dkv_in.clone()
        if self.dkv_out is not None:
            dec = torch.exp(-self.s.reshape(1, -1, 1, 1).float() * self.plan.n)
            prev = 0 if self.dkv_in is None else dec * self.dkv_in
            self.dkv_out.copy_(prev + self.local)

    def grads(self):
        assert self.calls == ["chunk_states", "scan"]
        dq, dk, dv, _ = O.blocked_backward(self.q, self.k, self.v, self.s, self.do, self.fwd_ws["kv_in"],
                                           self.saved_in)
        self.dq.copy_(dq.to(self.dq.dtype)), self.dk.copy_(dk.to(self.dk.dtype)), self.dv.copy_(dv.to(self.dv.dtype))

    def run(self):
        self.chunk_states(), self.scan(), self.grads()
        return self.dq, self.dk, self.dv
