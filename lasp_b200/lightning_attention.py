"""Single-device decay-masked causal linear attention.

Drop-in for ``lasp/lightning_attention.py`` of the reference: ``lightning_attn``
(:510-531) and ``lightning_attn_`` (= the autograd function's ``apply``, :507).
"""
from ._core import LightningAttention

lightning_attn_ = LightningAttention.apply


def lightning_attn(q, k, v, ed):
    """o = ((q k^T) * M) v with M_ij = exp(-ed_h (i-j)) for i >= j, else 0.

    q, k: (b, h, n, d); v: (b, h, n, e); ed: (h, 1, 1) decay rates.  Returns
    (b, h, n, e) in q's dtype.  Any n; d and e multiples of 16 (wider than 128
    is sliced).  No scaling, no normaliser: exactly the reference's op.
    """
    return lightning_attn_(q, k, v, ed)
