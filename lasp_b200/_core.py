"""Shared machinery of the five operators: head-dim slicing, the single-device
autograd function and the sequence-parallel autograd function.

The kernels are reached through ``ENGINE`` (module ``lasp_b200.engine``, the
ctypes launcher of the CUDA library).  The host-logic tests replace ``ENGINE``
with a stand-in to exercise group mapping and message order on gloo ranks; the
product has no other backend.
"""
from __future__ import annotations

import torch

from . import comm
from . import engine as ENGINE  # noqa: N812  (replaced as a whole by host-logic tests)
from .utils.seq_parallel_manager import (
    get_seq_parallel_receive_rank,
    get_seq_parallel_send_rank,
    get_sequence_parallel_group,
    get_sequence_parallel_rank,
    get_sequence_parallel_world_size,
)

MAX_HEAD_SLICE = 128  # widest q/k (d) or v (e) slice one kernel call takes


def _cuts(width: int):
    """[0, 128, 256, ..., width]: slice borders of a head dimension."""
    edges = list(range(0, width, MAX_HEAD_SLICE)) + [width]
    return list(zip(edges[:-1], edges[1:]))


def sliced_apply(fn, q, k, v, state_bufs=()):
    """Head-dim slicing of the reference wrappers (lasp/lightning_attention.py:510-531):
    the op is a sum over 128-wide q,k slices.  Wider v than 128 is handled the
    same way in the other direction (outputs of v slices are concatenated).
    ``state_bufs`` are (b,h,d,e) buffers sliced alongside.

    For the sequence-parallel operators (those with state buffers), when both
    widths are multiples of 128, the (q/k slice, v slice) pairs are stacked along
    the batch dimension and go through ONE call: one state hand-over per direction
    instead of one per slice (the reference runs a separate chain per slice,
    lasp/lasp_fuse.py:546-559).  On a single device there is nothing to hand over
    and the slices go one after the other, each with its spans spread over all SMs.
    """
    d, e = q.shape[-1], v.shape[-1]
    nd, ne = d // MAX_HEAD_SLICE, e // MAX_HEAD_SLICE
    if state_bufs and d % MAX_HEAD_SLICE == 0 and e % MAX_HEAD_SLICE == 0 and nd * ne > 1:
        b, h, n = q.shape[:3]
        w = MAX_HEAD_SLICE

        def stack(t, parts, over_e):
            # (b,h,n,parts*w) -> (ne*nd*b, h, n, w), batch index = (v slice, q/k slice, batch row)
            t = t.reshape(b, h, n, parts, w).permute(3, 0, 1, 2, 4)                 # (parts,b,h,n,w)
            t = t[:, None] if over_e else t[None]                                   # (ne|1, nd|1, ...)
            return t.expand(ne, nd, b, h, n, w).reshape(ne * nd * b, h, n, w).contiguous()

        bufs = [x.reshape(b, h, nd, w, ne, w).permute(4, 2, 0, 1, 3, 5).reshape(ne * nd * b, h, w, w).contiguous()
                for x in state_bufs]                                                # cut alongside
        o = fn(stack(q, nd, False), stack(k, nd, False), stack(v, ne, True), *bufs)
        o = o.reshape(ne, nd, b, h, n, w).sum(dim=1)                                # sum over q/k slices
        return o.permute(1, 2, 3, 0, 4).reshape(b, h, n, e)                        # v slices side by side
    outs = []
    for e0, e1 in _cuts(e):
        vs = v if (e0, e1) == (0, e) else v[..., e0:e1]
        acc = None
        for d0, d1 in _cuts(d):
            whole = (d0, d1) == (0, d)
            qs = q if whole else q[..., d0:d1]
            ks = k if whole else k[..., d0:d1]
            bufs = [x if (whole and (e0, e1) == (0, e)) else x[:, :, d0:d1, e0:e1].contiguous() for x in state_bufs]
            o = fn(qs, ks, vs, *bufs)
            acc = o if acc is None else acc + o
        outs.append(acc)
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)


def _plan_for(q, v, path=None, qk_scale=1.0, feature_map=None):
    b, h, n, d = q.shape
    if qk_scale == 1.0 and feature_map is None:
        return ENGINE.make_plan(b, h, n, d, v.shape[-1], q.dtype, path)
    return ENGINE.make_plan(b, h, n, d, v.shape[-1], q.dtype, path, qk_scale=qk_scale, feature_map=feature_map)


def preprocess_qk(x, qk_scale=1.0, feature_map=None):
    """qk_scale * map(x) with torch operations: what a caller of the reference writes in front of the operator,
    and what the ``*_fused`` operators do themselves when the kernels of a problem cannot take it over."""
    if feature_map == "elu1":
        x = torch.nn.functional.elu(x) + 1.0
    elif feature_map is not None:
        raise ValueError(f"unknown feature map {feature_map!r}; use None or 'elu1'")
    return x if qk_scale == 1.0 else x * qk_scale


def kernels_preprocess(q, v, qk_scale, feature_map) -> bool:
    """True when the kernels that will run this (slice of a) problem fold qk_scale * map(.) into their loads."""
    if not q.is_cuda:
        return False
    try:
        _plan_for(q, v, qk_scale=qk_scale, feature_map=feature_map)
    except ENGINE.LaspStatusError:
        return False
    return True


def _check_shapes(q, k, v, s):
    if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError(f"expected q,k (b,h,n,d) and v (b,h,n,e); got {tuple(q.shape)}, {tuple(k.shape)}, "
                         f"{tuple(v.shape)}")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one dtype")
    if s.numel() != q.shape[1]:
        raise ValueError(f"decay tensor has {s.numel()} entries for {q.shape[1]} heads")
    d, e = q.shape[-1], v.shape[-1]
    for name, width in (("q/k", d), ("v", e)):
        rest = width % MAX_HEAD_SLICE
        if width % 16 or (width > MAX_HEAD_SLICE and rest and rest % 16):
            raise ValueError(f"head dimension of {name} is {width}: it must be a multiple of 16 "
                             f"(wider than {MAX_HEAD_SLICE}: cut in {MAX_HEAD_SLICE}-wide slices)")
    if q.shape[0] * q.shape[1] > 65535:
        raise ValueError(f"batch x heads = {q.shape[0] * q.shape[1]} exceeds 65535")


class LightningAttention(torch.autograd.Function):
    """Single-device op: O = ((Q K^T) * M) V.  Interface of LightningAttention,
    lasp/lightning_attention.py:396-504; gradients for q, k, v only.

    Head dimensions wider than 128 are cut here, inside the function, the way the reference's wrapper cuts
    them (lasp/lightning_attention.py:510-531: a sum over 128-wide q,k slices; v slices side by side) - but
    the slices' results go straight into their place in o, dq, dk, dv.  Slicing outside, through autograd,
    builds a full-size zero tensor per slice and adds them up: at d = e = 256 that costs more memory traffic
    than the operator itself.
    """

    @staticmethod
    def forward(ctx, q, k, v, s, qk_scale=1.0, feature_map=None):
        _check_shapes(q, k, v, s)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        d, e = q.shape[-1], v.shape[-1]
        ctx.pre = (qk_scale, feature_map)
        ctx.save_for_backward(q, k, v, s)
        if d <= MAX_HEAD_SLICE and e <= MAX_HEAD_SLICE:
            plan = _plan_for(q, v, qk_scale=qk_scale, feature_map=feature_map)
            fw = ENGINE.Forward(plan, q, k, v, s)
            ctx.pairs = None
            ctx.plan, ctx.fwd_ws = plan, fw.ws
            return fw.run()
        o = torch.empty(*q.shape[:3], e, dtype=q.dtype, device=q.device)
        # Where the kernels take a row pitch (tensor-core path), a slice is read and written where it lies in the
        # wide tensors; otherwise it is copied out and back.
        in_place = _slices_in_place(q, v, qk_scale, feature_map)
        ctx.in_place = in_place
        ctx.pairs = []                                   # (q/k slice, v slice, plan, forward workspace)
        # in place, every tensor of a call has the wide tensors' row pitch: later contributions to a slice of o land
        # in a slice of a second wide tensor and are added from there
        more = torch.empty_like(o) if (in_place and len(_cuts(d)) > 1) else None
        for e0, e1 in _cuts(e):
            vs = v[..., e0:e1] if in_place else v[..., e0:e1].contiguous()
            for i, (d0, d1) in enumerate(_cuts(d)):
                qs, ks = (q[..., d0:d1], k[..., d0:d1]) if in_place else (q[..., d0:d1].contiguous(), k[..., d0:d1].contiguous())
                plan = _slice_plan(q, v, d1 - d0, e1 - e0, qk_scale, feature_map, in_place)
                first = i == 0
                fw = ENGINE.Forward(plan, qs, ks, vs, s,
                                    o=None if not in_place else (o if first else more)[..., e0:e1])
                part = fw.run()
                if not first:
                    o[..., e0:e1] += part
                elif not in_place:
                    o[..., e0:e1] = part
                ctx.pairs.append(((d0, d1), (e0, e1), plan, fw.ws))
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, s = ctx.saved_tensors
        do = do.contiguous()
        if ctx.pairs is None:
            bw = ENGINE.Backward(ctx.plan, q, k, v, do, s, ctx.fwd_ws)
            dq, dk, dv = bw.run()
            return dq, dk, dv, None, None, None
        in_place = ctx.in_place
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        # (as in forward: later contributions go through second wide tensors with the same row pitch)
        mq, mk, mv = (torch.empty_like(t) for t in (q, k, v)) if in_place else (None, None, None)
        seen_d, seen_e = set(), set()
        cut = (lambda t, lo, hi: t[..., lo:hi]) if in_place else (lambda t, lo, hi: t[..., lo:hi].contiguous())
        for (d0, d1), (e0, e1), plan, fwd_ws in ctx.pairs:
            new_d, new_e = d0 not in seen_d, e0 not in seen_e
            # a q/k slice collects from every v slice, a v slice from every q/k slice: the first contribution is
            # written in place (where the kernels can), the later ones are added
            bw = ENGINE.Backward(plan, cut(q, d0, d1), cut(k, d0, d1), cut(v, e0, e1), cut(do, e0, e1), s, fwd_ws,
                                 dq=None if not in_place else (dq if new_d else mq)[..., d0:d1],
                                 dk=None if not in_place else (dk if new_d else mk)[..., d0:d1],
                                 dv=None if not in_place else (dv if new_e else mv)[..., e0:e1])
            gq, gk, gv = bw.run()
            if not new_d:
                dq[..., d0:d1] += gq
                dk[..., d0:d1] += gk
            elif not in_place:
                dq[..., d0:d1] = gq
                dk[..., d0:d1] = gk
            if not new_e:
                dv[..., e0:e1] += gv
            elif not in_place:
                dv[..., e0:e1] = gv
            seen_d.add(d0), seen_e.add(e0)
        return dq, dk, dv, None, None, None


def _slice_plan(q, v, wd, we, qk_scale, feature_map, in_place):
    b, h, n = q.shape[:3]
    pitches = dict(pitch_d=q.shape[-1], pitch_e=v.shape[-1]) if in_place else {}
    if qk_scale == 1.0 and feature_map is None and not in_place:
        return ENGINE.make_plan(b, h, n, wd, we, q.dtype)
    return ENGINE.make_plan(b, h, n, wd, we, q.dtype, qk_scale=qk_scale, feature_map=feature_map, **pitches)


def _slices_in_place(q, v, qk_scale, feature_map) -> bool:
    """True when every (q/k slice, v slice) pair of these head dimensions can run on the wide tensors in place."""
    try:
        for d0, d1 in _cuts(q.shape[-1]):
            for e0, e1 in _cuts(v.shape[-1]):
                _slice_plan(q, v, d1 - d0, e1 - e0, qk_scale, feature_map, True)
    except (ENGINE.LaspStatusError, TypeError):
        return False
    return True


class SequenceParallelAttention(torch.autograd.Function):
    """Sequence-parallel op shared by lasp_naive / lasp_cache / lasp_fuse /
    lasp_fuse_parallel (LaspNaive ... LaspFuseParallel of the reference, e.g.
    lasp/lasp_fuse_parallel.py:1073-1137).

    Each rank holds one contiguous chunk of the sequence.  Forward: the KV
    state arrives from the ranks before, the outgoing state leaves for the
    ranks after; backward: dKV travels the other way.  Three schedules:

    * ``overlap=False`` (lasp_naive, lasp_cache): the reference's order -
      blocking receive, all three kernels, blocking send (NCCL / gloo).
    * ``overlap=True`` with the peer-mapped exchange (the default on GPUs of
      one node): chunk-state kernel -> ONE hand-over kernel that reduces this
      rank's states to its total, stores it into the later ranks' memory over
      NVLink, sums what earlier ranks stored here and runs the scan with it
      -> output kernel.  A peer that never delivers makes the results NaN and
      raises ``KernelFault`` at the start of the next call (or at
      ``lasp_b200.check_faults()``).
    * ``overlap=True`` over NCCL (LASP_B200_TRANSPORT=nccl, or CPU tensors):
      post the receive, run the state-independent chunk-state kernel, wait,
      scan, post the send, run the output kernel.
    """

    @staticmethod
    def forward(ctx, q, k, v, s, KV, DKV, overlap, qk_scale=1.0, feature_map=None):
        _check_shapes(q, k, v, s)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        b, h, n, d = q.shape
        e = v.shape[-1]
        for name, buf in (("KV", KV), ("DKV", DKV)):
            if tuple(buf.shape) != (b, h, d, e) or buf.dtype != torch.float32 or not buf.is_contiguous():
                raise ValueError(f"{name} must be a contiguous float32 tensor of shape {(b, h, d, e)}")
        group = get_sequence_parallel_group()
        rank = get_sequence_parallel_rank()
        last = get_sequence_parallel_world_size() - 1
        prev_rank, next_rank = get_seq_parallel_send_rank(), get_seq_parallel_receive_rank()
        link = comm.StateLink(group)
        plan = _plan_for(q, v, qk_scale=qk_scale, feature_map=feature_map)
        kv_in = KV if rank > 0 else None
        exchange = comm.relay_for(group, KV.numel(), q.device) if (overlap and last > 0 and q.is_cuda) else None

        if exchange is not None:
            ENGINE.fault_watch(q.device).poll()          # a fault of the previous step surfaces here
            fw = ENGINE.Forward(plan, q, k, v, s)
            if ENGINE.linked_ok(plan):
                fw.run_linked(exchange.link_args(backward=False))     # compute and hand-over in one launch
            else:
                fw.chunk_states()
                exchange.exchange_scan(plan, fw.ws, s, backward=False)
                fw.output()
        else:
            fw = ENGINE.Forward(plan, q, k, v, s, kv_in=kv_in, kv_out=KV if rank < last else None)
            if overlap:
                pending = link.post_recv(KV, prev_rank) if rank > 0 else None
                fw.chunk_states()
                link.wait(pending)
                fw.scan()
                sent = link.post_send(KV, next_rank) if rank < last else None
                fw.output()
                link.wait(sent)
            else:
                if rank > 0:
                    link.recv(KV, prev_rank)
                fw.run()
                if rank < last:
                    link.send(KV, next_rank)

        ctx.plan, ctx.fwd_ws, ctx.DKV, ctx.overlap = plan, fw.ws, DKV, overlap
        ctx.link, ctx.rank, ctx.last, ctx.exchange = link, rank, last, exchange
        ctx.prev_rank, ctx.next_rank = prev_rank, next_rank
        ctx.save_for_backward(q, k, v, s)
        return fw.o

    @staticmethod
    def backward(ctx, do):
        q, k, v, s = ctx.saved_tensors
        DKV, link, rank, last = ctx.DKV, ctx.link, ctx.rank, ctx.last
        dkv_in = DKV if rank < last else None
        if ctx.exchange is not None:
            bw = ENGINE.Backward(ctx.plan, q, k, v, do.contiguous(), s, ctx.fwd_ws)
            if ENGINE.linked_ok(ctx.plan):
                # dQ needs no incoming state.  The last rank has nobody to wait for and the others wait for
                # it: it sends first; the others do their dQ while the states travel.
                if rank == last:
                    bw.dkv_linked(ctx.exchange.link_args(backward=True))
                    bw.dq_only()
                else:
                    bw.dq_only()
                    bw.dkv_linked(ctx.exchange.link_args(backward=True))
            else:
                bw.chunk_states()
                # dQ needs no incoming state: it runs between the two halves of the hand-over
                ctx.exchange.exchange_scan(ctx.plan, bw.ws, s, backward=True, phase="push")
                bw.dq_only()
                ctx.exchange.exchange_scan(ctx.plan, bw.ws, s, backward=True, phase="gather")
                bw.dkv_after_scan()
            ENGINE.fault_watch(q.device).arm(q.device)   # looked at when the next call starts
            return bw.dq, bw.dk, bw.dv, None, None, None, None, None, None
        bw = ENGINE.Backward(ctx.plan, q, k, v, do.contiguous(), s, ctx.fwd_ws, dkv_in=dkv_in,
                             dkv_out=DKV if rank > 0 else None)
        if ctx.overlap:
            pending = link.post_recv(DKV, ctx.next_rank) if rank < last else None
            bw.chunk_states()
            link.wait(pending)
            bw.scan()
            sent = link.post_send(DKV, ctx.prev_rank) if rank > 0 else None
            bw.grads()
            link.wait(sent)
        else:
            if rank < last:
                link.recv(DKV, ctx.next_rank)
            bw.run()
            if rank > 0:
                link.send(DKV, ctx.prev_rank)
        return bw.dq, bw.dk, bw.dv, None, None, None, None, None, None


def sequence_parallel(q, k, v, s, KV, DKV, overlap: bool):
    return sliced_apply(lambda qs, ks, vs, kv, dkv: SequenceParallelAttention.apply(qs, ks, vs, s, kv, dkv, overlap),
                        q, k, v, (KV, DKV))


def _slice_like(q, v):
    """The widest slice `sliced_apply` will hand to the kernels for these head dimensions."""
    return q[..., :MAX_HEAD_SLICE], v[..., :MAX_HEAD_SLICE]


def lightning_attn_fused(q, k, v, s, qk_scale: float = 1.0, feature_map=None):
    """``lightning_attn(c * map(q), c * map(k), v, s)`` with the preprocessing of q and k folded into the
    kernels' load path (and its chain rule into their epilogues): q and k are read once, nothing is written in
    between.  ``feature_map``: None or "elu1" (elu(x) + 1); ``qk_scale``: c.  Problems whose kernels cannot
    do this (fp32 path, head dims other than 64 / 128 per slice, more spans than SMs) get the same result from
    torch operations in front of the operator."""
    if (qk_scale == 1.0 and feature_map is None) or not kernels_preprocess(*_slice_like(q, v), qk_scale, feature_map):
        return LightningAttention.apply(preprocess_qk(q, qk_scale, feature_map), preprocess_qk(k, qk_scale, feature_map), v, s)
    return LightningAttention.apply(q, k, v, s, qk_scale, feature_map)


def sequence_parallel_fused(q, k, v, s, KV, DKV, qk_scale: float = 1.0, feature_map=None):
    """``lasp_fuse_parallel`` on c * map(q), c * map(k) with the preprocessing inside the kernels where the
    rank's launches are the fused ones that hand the state over themselves; torch operations otherwise."""
    qs, vs = _slice_like(q, v)
    in_kernel = (qk_scale != 1.0 or feature_map is not None) and kernels_preprocess(qs, vs, qk_scale, feature_map)
    if in_kernel and get_sequence_parallel_world_size() > 1:
        b, h, n, d = qs.shape
        plan = _plan_for(qs, vs, qk_scale=qk_scale, feature_map=feature_map)
        relay = comm.relay_for(get_sequence_parallel_group(), b * h * d * vs.shape[-1], q.device)
        in_kernel = relay is not None and ENGINE.linked_ok(plan)
    if not in_kernel:
        return sequence_parallel(preprocess_qk(q, qk_scale, feature_map), preprocess_qk(k, qk_scale, feature_map), v, s,
                                 KV, DKV, True)
    return sliced_apply(lambda qs_, ks_, vs_, kv, dkv: SequenceParallelAttention.apply(qs_, ks_, vs_, s, kv, dkv, True,
                                                                                       qk_scale, feature_map),
                        q, k, v, (KV, DKV))
