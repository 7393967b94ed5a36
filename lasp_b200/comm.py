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

import os
import warnings

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


# ---------------------------------------------------------------------------
# NVLink exchange: the whole state exchange as one kernel over peer-mapped buffers
# ---------------------------------------------------------------------------
class NvlinkExchange:
    """Peer-mapped receive slots, flags and acknowledgement words of one
    sequence-parallel group for one state size, and the launcher of the
    hand-over kernel.

    The buffers come from torch's symmetric-memory allocator (a CUDA virtual
    memory allocation exported to the group's other ranks); the transfer itself
    is done by the library's own kernel (``lasp_b200_exchange_scan``) with plain
    peer stores - no NCCL call is on the path, so a whole forward or backward
    can be captured in a CUDA graph.  Each rank's buffer holds two regions (forward, backward), each:
        [0, 8K) acks [destination][slice]   [8K, 9K) counters
        [32K, ...) slots [parity][source][element] of 8-byte {value, step} words
    """
    MAX_RANKS = 8
    _HEADER = 32768

    def __init__(self, group, elems: int, device):
        import torch.distributed._symmetric_memory as symm
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        self.group, self.elems, self.device = group, elems, torch.device(device)
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        if self.size > self.MAX_RANKS:
            raise RuntimeError(f"the peer-mapped exchange handles groups of up to {self.MAX_RANKS} ranks")
        self.region = self._HEADER + 2 * self.size * elems * 8
        self.buf = symm.empty(2 * self.region // 4, dtype=torch.float32, device=self.device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)   # every rank has zeroed its flags before any peer writes one

    def link_args(self, backward: bool, wait_clocks: int | None = None):
        """The group's buffers of one direction as the ``lasp_exchange_args`` the linked calls take."""
        from . import _cabi
        pos = self.size - 1 - self.rank if backward else self.rank
        off = self.region if backward else 0
        a = _cabi.ExchangeArgs()
        a.ranks, a.position, a.reverse = self.size, pos, 1 if backward else 0
        me = self.ptrs[self.rank] + off
        a.my_acks, a.counters, a.my_slots = me, me + 8192, me + self._HEADER
        for q in range(self.size):
            base = self.ptrs[self.size - 1 - q if backward else q] + off   # buffer of the rank at position q
            a.peer_acks[q], a.peer_slots[q] = base, base + self._HEADER
        a.wait_clocks = wait_timeout_clocks() if wait_clocks is None else wait_clocks
        return a

    def exchange_scan(self, plan, ws, s, backward: bool, wait_clocks: int | None = None, phase: str = "both") -> None:
        """Launch the hand-over of one direction on the current stream, between the chunk-state phase and
        the output / gradient phase of the call that owns ``ws`` and in place of its scan phase.
        Forward: states flow towards higher ranks; backward: towards lower ranks.  ``phase``: "both", or
        "push" followed later by "gather" (two launches of one step; whatever runs between them overlaps
        the states' flight)."""
        from . import _cabi, engine
        assert plan.b * plan.h * plan.d * plan.e == self.elems
        pos = self.size - 1 - self.rank if backward else self.rank
        off = self.region if backward else 0
        sl = s.reshape(-1).to(device=ws.device, dtype=torch.float32).contiguous()
        a = _cabi.ExchangeArgs()
        a.ranks, a.position, a.reverse = self.size, pos, 1 if backward else 0
        a.phase = {"both": _cabi.EXCHANGE_BOTH, "push": _cabi.EXCHANGE_PUSH, "gather": _cabi.EXCHANGE_GATHER}[phase]
        a.s, a.ws, a.ws_bytes = sl.data_ptr(), ws.data_ptr(), ws.numel()
        me = self.ptrs[self.rank] + off
        a.my_acks, a.counters, a.my_slots = me, me + 8192, me + self._HEADER
        for q in range(self.size):
            base = self.ptrs[self.size - 1 - q if backward else q] + off   # buffer of the rank at position q
            a.peer_acks[q], a.peer_slots[q] = base, base + self._HEADER
        a.wait_clocks = wait_timeout_clocks() if wait_clocks is None else wait_clocks
        engine.exchange_scan(plan, a, ws.device)
        self._keep = (sl, ws)   # alive until the next launch is enqueued on the same stream


def wait_timeout_clocks() -> int:
    """How long the hand-over kernel waits for a peer before it reports a fault, in GPU clocks: env
    LASP_B200_EXCHANGE_TIMEOUT_MS (default 30 s, the order of a process-group timeout, not of a step)."""
    ms = float(os.environ.get("LASP_B200_EXCHANGE_TIMEOUT_MS", "30000"))
    return max(1, int(ms * 1.9e6))


_relays = {}
_relay_unavailable = False


def transport() -> str:
    """'nvlink' (the library's exchange kernel over peer memory) or 'nccl'
    (rank-to-rank isend/irecv); env LASP_B200_TRANSPORT, default 'auto' = nvlink
    when the group's buffers can be peer-mapped."""
    return os.environ.get("LASP_B200_TRANSPORT", "auto")


def _make_relay(group, elems: int, device):
    return NvlinkExchange(group, elems, device)


def relay_for(group, elems: int, device):
    """The group's NvlinkExchange for this state size, or None when peer mapping is not available.
    Collective: every rank of the group calls it alike, and the ranks AGREE on the outcome - if setting
    the buffers up fails on any rank, all of them use NCCL send/recv (a rank on the other transport
    would wait for words that never come)."""
    global _relay_unavailable
    if transport() == "nccl" or _relay_unavailable:
        return None
    key = (id(group), elems, torch.device(device).index)
    if key not in _relays:
        relay, failure = None, None
        try:
            relay = _make_relay(group, elems, device)
        except Exception as exc:  # noqa: BLE001
            failure = exc
        ok = torch.tensor([0 if relay is None else 1], dtype=torch.int32,
                          device=device if dist.get_backend(group) == "nccl" else "cpu")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if not int(ok.item()):
            if transport() == "nvlink":
                raise RuntimeError("lasp_b200: the peer-mapped state exchange could not be set up on every rank"
                                   ) from failure
            warnings.warn(f"lasp_b200: peer-mapped state exchange unavailable on some rank "
                          f"({failure or 'another rank failed'}); every rank uses NCCL send/recv")
            _relay_unavailable = True
            return None
        _relays[key] = relay
    return _relays[key]
