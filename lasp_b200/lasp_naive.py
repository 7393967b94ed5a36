"""``lasp_naive``: sequence-parallel linear attention, reference order of work.

Drop-in for ``lasp/lasp_naive.py`` (:541-648): the rank state buffers are made
here, the KV state is received before the local kernels run and sent after.
"""
import torch

from ._core import SequenceParallelAttention, sequence_parallel


def lasp_naive_(q, k, v, s):
    b, h, _, d = q.shape
    e = v.shape[-1]
    KV = torch.empty(b, h, d, e, dtype=torch.float32, device=q.device)
    DKV = torch.empty(b, h, d, e, dtype=torch.float32, device=q.device)
    return SequenceParallelAttention.apply(q, k, v, s, KV, DKV, False)


def lasp_naive(q, k, v, ed):
    """q, k (b,h,n_local,d), v (b,h,n_local,e): this rank's chunk; ed (h,1,1)."""
    b, h, _, d = q.shape
    e = v.shape[-1]
    KV = torch.empty(b, h, d, e, dtype=torch.float32, device=q.device)
    DKV = torch.empty(b, h, d, e, dtype=torch.float32, device=q.device)
    return sequence_parallel(q, k, v, ed, KV, DKV, overlap=False)
