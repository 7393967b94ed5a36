"""Shared helpers of the test-suite: golden-fixture access and tolerances."""
import json
import os

import numpy as np
import torch

from oracle import lasp_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
with open(os.path.join(GOLDEN, "cases.json")) as _f:
    CASES = json.load(_f)

# parity gates: max|x - ref| / max|ref|
TOL_FP32 = 1e-3
TOL_BF16 = 2e-2


def slopes_for(kind, h):
    if kind == "baseline":
        return O.baseline_slopes(h)
    if kind == "alibi":
        return O.build_slope_tensor_ref(h).to(torch.float32)
    return torch.zeros(h, 1, 1)


def case_inputs(p):
    q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"],
                                scale_qk=p.get("scale_qk", True), feature_map=p.get("feature_map"))
    return q, k, v, do, slopes_for(p["slopes"], p["h"])


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def golden_tensor(arr):
    """fixtures hold fp32 arrays, or bf16 bit patterns as uint16"""
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16).float()
    return torch.from_numpy(arr)


def input_checksum(*ts):
    return float(sum(t.double().abs().sum().item() for t in ts))


def split(x, dp, sp, dp_rank, sp_rank):
    """batch interleaved over dp, sequence contiguous over sp (tests/test.py:48-60 of the reference)"""
    b = x.shape[0]
    x = x.reshape(b // dp, dp, *x.shape[1:])[:, dp_rank]
    nl = x.shape[2] // sp
    return x[:, :, sp_rank * nl:(sp_rank + 1) * nl].clone()
