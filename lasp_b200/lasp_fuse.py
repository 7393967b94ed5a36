"""``lasp_fuse``: sequence-parallel linear attention with the rank-state terms
fused into the kernels.

Drop-in for ``lasp/lasp_fuse.py`` (:478-561).  The incoming KV / dKV state is
folded into the per-chunk prefix states by the scan kernel, so the output and
gradient kernels apply it in the same pass as the local terms.
"""
from ._core import SequenceParallelAttention, sequence_parallel


def lasp_fuse_(q, k, v, s, KV, DKV):
    return SequenceParallelAttention.apply(q, k, v, s, KV, DKV, True)


def lasp_fuse(q, k, v, ed, KV, DKV):
    """KV, DKV: (b,h,d,e) float32 scratch, overwritten."""
    return sequence_parallel(q, k, v, ed, KV, DKV, overlap=True)
