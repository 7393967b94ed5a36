"""A pre-planned forward + backward of the operator on fixed buffers.

``FixedStep`` binds one set of input/output tensors to the C-ABI launches of a
forward and a backward pass - six kernels on a single device, plus the two
state totals and the two state exchanges when the rank is part of a
sequence-parallel group.  Nothing is allocated by ``run()``, and no NCCL call
is made, so the whole step can be captured in a CUDA graph and replayed.
It issues exactly the launches the autograd functions of ``_core`` issue.
"""
from __future__ import annotations

import torch

from . import comm, engine


class FixedStep:
    def __init__(self, q, k, v, do, s, group=None):
        b, h, n, d = q.shape
        e = v.shape[-1]
        self.n, self.s = n, s
        self.plan = engine.make_plan(b, h, n, d, e, q.dtype)
        self.relay = None
        self.rank, self.last = 0, 0
        if group is not None and torch.distributed.get_world_size(group) > 1:
            self.rank = torch.distributed.get_rank(group)
            self.last = torch.distributed.get_world_size(group) - 1
            self.relay = comm.relay_for(group, b * h * d * e, q.device)
            if self.relay is None:
                raise RuntimeError("FixedStep needs the peer-mapped relay transport (LASP_B200_TRANSPORT=nvlink)")
        state = lambda: torch.empty(b, h, d, e, dtype=torch.float32, device=q.device)  # noqa: E731
        self.kv_in = state() if self.rank > 0 else None
        self.dkv_in = state() if self.rank < self.last else None
        self.total_f, self.total_b = (state(), state()) if self.relay is not None else (None, None)
        self.fw = engine.Forward(self.plan, q, k, v, s, kv_in=self.kv_in)
        self.bw = engine.Backward(self.plan, q, k, v, do, s, self.fw.ws, dkv_in=self.dkv_in)

    @property
    def launches(self) -> int:
        return 6 if self.relay is None else 10

    @property
    def outputs(self):
        return self.fw.o, self.bw.dq, self.bw.dk, self.bw.dv

    def run(self) -> None:
        fw, bw = self.fw, self.bw
        if self.relay is None:
            fw.run()
            bw.run()
            return
        fw.chunk_states()
        engine.state_total(self.plan, fw.ws, self.s, reverse=False, out=self.total_f)
        self.relay.exchange(self.total_f, self.kv_in, self.s, self.n, backward=False)
        fw.scan()
        fw.output()
        bw.chunk_states()
        engine.state_total(self.plan, bw.ws, self.s, reverse=True, out=self.total_b)
        self.relay.exchange(self.total_b, self.dkv_in, self.s, self.n, backward=True)
        bw.scan()
        bw.grads()
