"""Decay slopes and a peak-memory helper.

Mirrors lasp/utils/module_utils.py of the reference: ``build_slope_tensor``
(:6-31) returns the ALiBi-style per-head slopes as an (h,1,1) tensor and
``get_memory`` (:34-38) reads and resets the CUDA peak-allocation counter.
"""
from __future__ import annotations

import math

import torch


def _geometric(count: int):
    # count is a power of two: slopes r, r^2, ..., r^count with r = 2^(-8/count)
    ratio = 2.0 ** (-(2.0 ** -(math.log2(count) - 3)))
    return [ratio * ratio**i for i in range(count)]


def build_slope_tensor(n_attention_heads: int) -> torch.Tensor:
    """Per-head decay rates, shape (h, 1, 1).

    A power-of-two head count gets the geometric sequence 2^(-8 i/h), i = 1..h.
    Any other count takes the sequence of the largest power of two below it and
    fills the remaining heads with the odd-indexed terms of the sequence that
    is twice as long (the rule of lasp/utils/module_utils.py:15-24).
    """
    h = int(n_attention_heads)
    if h < 1:
        raise ValueError("need at least one head")
    values = []
    remaining = h
    width = 2 ** math.floor(math.log2(h))
    first = True
    while remaining > 0:
        seq = _geometric(width)
        if not first:
            seq = seq[0::2]
        take = seq[: remaining if not first else min(remaining, width)]
        values += take
        remaining -= len(take)
        width *= 2
        first = False
    return torch.tensor(values).reshape(h, 1, 1)


def get_memory(device) -> float:
    """Peak allocated MiB on ``device`` since the last call (resets the counter)."""
    peak = torch.cuda.max_memory_allocated(device) / 1024 / 1024
    torch.cuda.reset_peak_memory_stats(device)
    return peak
