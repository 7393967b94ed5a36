"""Rank-to-rank transfer of the (b,h,d,e) fp32 KV / dKV state.

The reference moves the state with blocking ``dist.recv`` before any local
compute and ``dist.send`` after all of it (lasp/lasp_fuse_parallel.py:1094-1106,
1129-1135), so the ranks of a sequence-parallel group run one after another.
``StateLink`` posts the receive on a side stream before the state-independent
kernels are launched and the send as soon as the scan has produced the
outgoing state; the main stream only waits where the data is consumed.

On CPU tensors (gloo; used by the host-logic tests) there are no streams: the
same calls degrade to isend/irecv plus ``wait()``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_side_streams = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


class _Pending:
    def __init__(self, work, tensor, side):
        self.work, self.tensor, self.side = work, tensor, side


class StateLink:
    """Asynchronous neighbour exchange inside one sequence-parallel group."""

    def __init__(self, group):
        self.group = group

    def post_recv(self, buf: torch.Tensor, src: int) -> _Pending:
        """Start receiving into ``buf``; earlier work on the current stream that
        touches ``buf`` is ordered before the receive."""
        if not buf.is_cuda:
            return _Pending(dist.irecv(buf, src=src, group=self.group), buf, None)
        main = torch.cuda.current_stream(buf.device)
        side = _side_stream(buf.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            work = dist.irecv(buf, src=src, group=self.group)
        return _Pending(work, buf, side)

    def post_send(self, buf: torch.Tensor, dst: int) -> _Pending:
        """Start sending ``buf`` once the current stream has produced it."""
        if not buf.is_cuda:
            return _Pending(dist.isend(buf, dst=dst, group=self.group), buf, None)
        main = torch.cuda.current_stream(buf.device)
        side = _side_stream(buf.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            work = dist.isend(buf, dst=dst, group=self.group)
        return _Pending(work, buf, side)

    def wait(self, pending: _Pending) -> None:
        """Order the transfer before whatever the current stream runs next
        (blocks the host only on CPU tensors)."""
        if pending is None:
            return
        if pending.side is None:
            pending.work.wait()
            return
        with torch.cuda.stream(pending.side):
            pending.work.wait()
        torch.cuda.current_stream(pending.tensor.device).wait_stream(pending.side)

    # blocking forms, as the reference uses them
    def recv(self, buf: torch.Tensor, src: int) -> None:
        dist.recv(buf, src=src, group=self.group)

    def send(self, buf: torch.Tensor, dst: int) -> None:
        dist.send(buf, dst=dst, group=self.group)
