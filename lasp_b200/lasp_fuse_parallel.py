"""``lasp_fuse_parallel``: block-parallel sequence-parallel linear attention.

Drop-in for ``lasp/lasp_fuse_parallel.py`` (:1073-1166).  Chunk states are
computed for all chunks at once, scanned, then applied; the receive of the
rank state is posted before the chunk-state kernel and the send right after
the scan, so neighbouring ranks overlap everything but the scan.  No
world-wide barrier is issued (the reference calls one per forward, :1094).
"""
from ._core import SequenceParallelAttention, sequence_parallel


def lasp_fuse_parallel_(q, k, v, s, KV, DKV):
    return SequenceParallelAttention.apply(q, k, v, s, KV, DKV, True)


def lasp_fuse_parallel(q, k, v, ed, KV, DKV):
    """KV, DKV: (b,h,d,e) float32 scratch, overwritten."""
    return sequence_parallel(q, k, v, ed, KV, DKV, overlap=True)
