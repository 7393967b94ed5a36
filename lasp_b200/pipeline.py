"""A pre-planned forward + backward of the operator on fixed buffers.

``FixedStep`` binds one set of input/output tensors to the C-ABI launches of a
forward and a backward pass: on a single device three kernels on the tensor-core
path (fused forward, dQ walk, fused dK/dV walk; six on the fp32 path).  As a rank
of a sequence-parallel group the same three, the two fused ones handing the rank
state over inside the launch; when the spans do not fit one per SM, eight (span
totals, hand-over in two halves around dQ, scan, walks).  Nothing is allocated by ``run()``, and no NCCL call
is made, so the whole step can be captured in a CUDA graph and replayed.
It issues exactly the launches the autograd functions of ``_core`` issue.
"""
from __future__ import annotations

import torch

from . import comm, engine


class FixedStep:
    def __init__(self, q, k, v, do, s, group=None, qk_scale=1.0, feature_map=None):
        """``qk_scale`` / ``feature_map``: the operator on qk_scale * map(q), qk_scale * map(k), folded into the
        kernels (engine.make_plan)."""
        b, h, n, d = q.shape
        e = v.shape[-1]
        self.n, self.s = n, s
        self.plan = engine.make_plan(b, h, n, d, e, q.dtype, qk_scale=qk_scale, feature_map=feature_map)
        self.relay = None
        self.rank, self.last = 0, 0
        if group is not None and torch.distributed.get_world_size(group) > 1:
            self.rank = torch.distributed.get_rank(group)
            self.last = torch.distributed.get_world_size(group) - 1
            self.relay = comm.relay_for(group, b * h * d * e, q.device)
            if self.relay is None:
                raise RuntimeError("FixedStep needs the peer-mapped relay transport (LASP_B200_TRANSPORT=nvlink)")
        self.fw = engine.Forward(self.plan, q, k, v, s)
        self.bw = engine.Backward(self.plan, q, k, v, do, s, self.fw.ws)
        self.linked = self.relay is not None and engine.linked_ok(self.plan)
        if self.linked:
            self.link_f, self.link_b = self.relay.link_args(backward=False), self.relay.link_args(backward=True)

    @property
    def launches(self) -> int:
        tensor = self.plan.path_name == "tensor"
        if self.relay is None or self.linked:
            return 3 if tensor else 6
        return 8 if tensor else 7

    @property
    def outputs(self):
        return self.fw.o, self.bw.dq, self.bw.dk, self.bw.dv

    def run(self) -> None:
        fw, bw = self.fw, self.bw
        if self.relay is None:
            fw.run()
            bw.run()
            return
        if self.linked:
            fw.run_linked(self.link_f)
            if self.rank == self.last:        # nobody to wait for in the backward pass: send first
                bw.dkv_linked(self.link_b)
                bw.dq_only()
            else:
                bw.dq_only()
                bw.dkv_linked(self.link_b)
            return
        fw.chunk_states()
        self.relay.exchange_scan(self.plan, fw.ws, self.s, backward=False)
        fw.output()
        bw.chunk_states()
        self.relay.exchange_scan(self.plan, bw.ws, self.s, backward=True, phase="push")
        bw.dq_only()                       # needs no incoming state: overlaps the states' flight
        self.relay.exchange_scan(self.plan, bw.ws, self.s, backward=True, phase="gather")
        bw.dkv_after_scan()
