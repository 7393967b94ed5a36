"""CPU oracle for LASP's decay-masked causal linear attention (forward + backward).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module; it is the checker used by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline / reference legs of ``bench.py``.

It restates, in plain torch on the CPU, the arithmetic of the reference's
Triton kernels.  The reference holds no pure-torch implementation of the op,
so every function below cites the reference lines it follows:

* ``dense_closed_form``      - O = ((Q K^T) * M) V and its analytic gradients,
  the definition the kernels of ``lasp/lightning_attention.py:6-83,86-181``
  implement block-wise.
* ``blocked_forward``        - ``lasp/lightning_attention.py:45-83`` (block
  recurrence) with the incoming rank state of ``lasp/lasp_fuse.py:104-127``.
* ``blocked_backward``       - ``lasp/lightning_attention.py:154-160,238-278,
  333-393`` with the incoming states of ``lasp/lasp_fuse.py:237-260,316-353``.
* ``sp_chain``               - the rank-to-rank recurrence of
  ``lasp/lasp_naive.py:547-568,593-616`` emulated in one process.
* ``slice_wrapper``          - the head-dim slicing of
  ``lasp/lightning_attention.py:510-531``.
* ``build_slope_tensor_ref`` - ``lasp/utils/module_utils.py:6-31``.

Parity pin: the reference ships no golden vectors (its only test prints
unseeded mean differences), so the oracle is pinned against outputs of the
reference's own Triton kernels executed on the CPU through Triton's
interpreter; ``tests/golden/make_golden.py`` generated those fixtures and
``tests/test_oracle_golden.py`` checks every function here against them.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

BLOCK = 64  # the reference's block size (lasp/lightning_attention.py:407)


# ----------------------------------------------------------------------------
# inputs
# ----------------------------------------------------------------------------
def baseline_slopes(h: int) -> torch.Tensor:
    """Per-head decay s_i = 2^(-8(i+1)/h), shape (h,1,1) fp32 (bench configs)."""
    i = torch.arange(1, h + 1, dtype=torch.float64)
    return torch.pow(2.0, -8.0 * i / h).to(torch.float32).reshape(h, 1, 1)


def build_slope_tensor_ref(h: int) -> torch.Tensor:
    """ALiBi-style slopes as the reference builds them.

    Follows lasp/utils/module_utils.py:6-31: powers of two get the geometric
    sequence start=2^(-2^-(log2 n - 3)); other head counts take the closest
    lower power of two and interleave every other slope of the next one.
    """

    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * start**i for i in range(n)]

    def slopes(n):
        if math.log2(n).is_integer():
            return pow2(n)
        c = 2 ** math.floor(math.log2(n))
        return pow2(c) + slopes(2 * c)[0::2][: n - c]

    return torch.tensor(slopes(h)).reshape(h, 1, 1)


def make_inputs(seed: int, b: int, h: int, n: int, d: int, e: int,
                scale_qk: bool = True, feature_map: Optional[str] = None):
    """Seeded iid N(0,1) q,k,v,do in fp32 (numpy RandomState: frozen stream).

    q,k are scaled by d^-0.5 when ``scale_qk``; ``feature_map='elu1'`` applies
    elu(x)+1 to q and k (the LinearTransformer-style config).
    """
    rs = np.random.RandomState(seed)
    q = torch.from_numpy(rs.standard_normal((b, h, n, d)).astype(np.float32))
    k = torch.from_numpy(rs.standard_normal((b, h, n, d)).astype(np.float32))
    v = torch.from_numpy(rs.standard_normal((b, h, n, e)).astype(np.float32))
    do = torch.from_numpy(rs.standard_normal((b, h, n, e)).astype(np.float32))
    if feature_map == "elu1":
        q = torch.nn.functional.elu(q) + 1.0
        k = torch.nn.functional.elu(k) + 1.0
    if scale_qk:
        q = q * d ** -0.5
        k = k * d ** -0.5
    return q, k, v, do


def max_rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x-ref| / max|ref|: the parity metric (elementwise relative error is
    meaningless near zeros)."""
    x = x.detach().to(torch.float64).cpu()
    ref = ref.detach().to(torch.float64).cpu()
    den = ref.abs().max().item()
    num = (x - ref).abs().max().item()
    if not math.isfinite(num):
        return float("inf")
    return num / den if den > 0 else num


# ----------------------------------------------------------------------------
# dense closed form (ground truth, O(n^2))
# ----------------------------------------------------------------------------
def _decay_mask(s: torch.Tensor, n: int, dtype) -> torch.Tensor:
    # M_ij = exp(-s (i-j)) for i>=j else 0    (lasp/lightning_attention.py:49-52)
    idx = torch.arange(n, dtype=dtype)
    diff = idx[:, None] - idx[None, :]
    s = s.reshape(-1, 1, 1).to(dtype)
    m = torch.exp(-s * diff.clamp(min=0))
    return torch.where(diff >= 0, m, torch.zeros((), dtype=dtype))  # (h,n,n)


def dense_closed_form(q, k, v, s, do=None, dtype=torch.float64):
    """O = ((QK^T)*M)V and, when ``do`` is given, dQ, dK, dV analytically."""
    q, k, v = (t.to(dtype) for t in (q, k, v))
    n = q.shape[2]
    m = _decay_mask(s, n, dtype)[None]                  # (1,h,n,n)
    a = torch.matmul(q, k.transpose(-1, -2)) * m
    o = torch.matmul(a, v)
    if do is None:
        return o
    do = do.to(dtype)
    da = torch.matmul(do, v.transpose(-1, -2)) * m      # (dO V^T)*M
    dq = torch.matmul(da, k)
    dk = torch.matmul(da.transpose(-1, -2), q)
    dv = torch.matmul(a.transpose(-1, -2), do)
    return o, dq, dk, dv


# ----------------------------------------------------------------------------
# blocked recurrence (O(n)); what every reference kernel computes
# ----------------------------------------------------------------------------
def _pad_blocks(x: torch.Tensor, block: int) -> torch.Tensor:
    n = x.shape[2]
    pad = (-n) % block
    if pad:
        x = torch.nn.functional.pad(x, (0, 0, 0, pad))
    return x


def blocked_forward(q, k, v, s, kv_in=None, block: int = BLOCK, dtype=torch.float32
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block recurrence of lasp/lightning_attention.py:45-83.

    Returns (o, kv_out).  ``kv_in`` (b,h,d,e) is the state arriving from the
    previous sequence-parallel rank, decayed to this rank's first token
    (lasp/lasp_fuse.py:104-111); ``kv_out`` = lambda^n kv_in + local state
    (lasp/lasp_fuse.py:126-127, lasp/lasp_naive.py:565).  A ragged tail is
    zero padded like the masked loads of lightning_attention.py:59-69; the
    outgoing state is always decayed to position n exactly.
    """
    b, h, n, d = q.shape
    e = v.shape[-1]
    q, k, v = (_pad_blocks(t.to(dtype), block) for t in (q, k, v))
    nb = q.shape[2] // block
    sv = s.reshape(1, h, 1, 1).to(dtype)
    r = torch.arange(block, dtype=dtype)
    diff = r[:, None] - r[None, :]
    mask = torch.where(diff >= 0, torch.exp(-sv * diff.clamp(min=0)), torch.zeros((), dtype=dtype))
    q_decay = torch.exp(-sv * r.reshape(1, 1, block, 1))              # lambda^r
    kv = torch.zeros(b, h, d, e, dtype=dtype) if kv_in is None else kv_in.to(dtype).clone()
    o = torch.empty(b, h, nb * block, e, dtype=dtype)
    for t in range(nb):
        sl = slice(t * block, (t + 1) * block)
        ln = min(block, n - t * block)                               # tokens really in the block
        qt, kt, vt = q[:, :, sl], k[:, :, sl], v[:, :, sl]
        k_decay = torch.exp(-sv * (ln - r).clamp(min=0).reshape(1, 1, block, 1))   # lambda^(len-c)
        qk = torch.matmul(qt, kt.transpose(-1, -2)) * mask
        o[:, :, sl] = torch.matmul(qk, vt) + torch.matmul(qt, kv) * q_decay
        kv = torch.exp(-sv * ln) * kv + torch.matmul((kt * k_decay).transpose(-1, -2), vt)
    return o[:, :, :n], kv


def blocked_backward(q, k, v, s, do, kv_in=None, dkv_in=None, block: int = BLOCK,
                     dtype=torch.float32):
    """Backward block recurrences of lasp/lightning_attention.py:154-160 (intra),
    :238-278 (forward sweep, dQ) and :333-393 (reverse sweep, dK, dV, dKV).

    ``kv_in``/``dkv_in`` are the incoming rank states (lasp/lasp_fuse.py:244-246,
    335-344).  Returns (dq, dk, dv, dkv_out) with dkv_out = lambda^n dkv_in +
    local dkv (lasp/lasp_fuse.py:352-353).
    """
    b, h, n, d = q.shape
    e = v.shape[-1]
    q, k, v, do = (_pad_blocks(t.to(dtype), block) for t in (q, k, v, do))
    nb = q.shape[2] // block
    sv = s.reshape(1, h, 1, 1).to(dtype)
    r = torch.arange(block, dtype=dtype)
    diff = r[:, None] - r[None, :]
    mask = torch.where(diff >= 0, torch.exp(-sv * diff.clamp(min=0)), torch.zeros((), dtype=dtype))
    q_decay = torch.exp(-sv * r.reshape(1, 1, block, 1))
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    # forward sweep: dQ needs the prefix state KV_t
    kv = torch.zeros(b, h, d, e, dtype=dtype) if kv_in is None else kv_in.to(dtype).clone()
    for t in range(nb):
        sl = slice(t * block, (t + 1) * block)
        ln = min(block, n - t * block)
        qt, kt, vt, dot = q[:, :, sl], k[:, :, sl], v[:, :, sl], do[:, :, sl]
        k_decay = torch.exp(-sv * (ln - r).clamp(min=0).reshape(1, 1, block, 1))
        dqk = torch.matmul(dot, vt.transpose(-1, -2)) * mask
        dq[:, :, sl] = torch.matmul(dqk, kt) + torch.matmul(dot, kv.transpose(-1, -2)) * q_decay
        kv = torch.exp(-sv * ln) * kv + torch.matmul((kt * k_decay).transpose(-1, -2), vt)
    # reverse sweep: dK, dV need the suffix state dKV_t
    dkv = torch.zeros(b, h, d, e, dtype=dtype) if dkv_in is None else dkv_in.to(dtype).clone()
    for t in reversed(range(nb)):
        sl = slice(t * block, (t + 1) * block)
        ln = min(block, n - t * block)
        qt, kt, vt, dot = q[:, :, sl], k[:, :, sl], v[:, :, sl], do[:, :, sl]
        k_decay = torch.exp(-sv * (ln - r).clamp(min=0).reshape(1, 1, block, 1))
        dqk = torch.matmul(dot, vt.transpose(-1, -2)) * mask
        qk = torch.matmul(qt, kt.transpose(-1, -2)) * mask
        dk[:, :, sl] = (torch.matmul(dqk.transpose(-1, -2), qt)
                        + torch.matmul(vt, dkv.transpose(-1, -2)) * k_decay)
        dv[:, :, sl] = (torch.matmul(qk.transpose(-1, -2), dot)
                        + torch.matmul(kt * k_decay, dkv))
        dkv = torch.exp(-sv * ln) * dkv + torch.matmul((qt * q_decay).transpose(-1, -2), dot)
    return dq[:, :, :n], dk[:, :, :n], dv[:, :, :n], dkv


def fwd_bwd(q, k, v, s, do, block: int = BLOCK, dtype=torch.float32):
    """Single-device forward + backward (the timed CPU baseline)."""
    o, _ = blocked_forward(q, k, v, s, None, block, dtype)
    dq, dk, dv, _ = blocked_backward(q, k, v, s, do, None, None, block, dtype)
    return o, dq, dk, dv


# ----------------------------------------------------------------------------
# sequence-parallel chain, emulated in one process
# ----------------------------------------------------------------------------
def preprocess_qk(x, qk_scale: float = 1.0, feature_map: Optional[str] = None):
    """qk_scale * map(x): what a caller of the reference applies to q and k in front of the operator
    (elu(x)+1 in the no-decay configuration, d^-0.5 elsewhere); lasp/lightning_attention.py:510 takes the result."""
    if feature_map == "elu1":
        x = torch.nn.functional.elu(x) + 1.0
    elif feature_map is not None:
        raise ValueError(feature_map)
    return x * qk_scale


def preprocess_slope(x, qk_scale: float = 1.0, feature_map: Optional[str] = None):
    """d(preprocess_qk(x))/dx, elementwise."""
    if feature_map == "elu1":
        return qk_scale * torch.where(x > 0, torch.ones_like(x), torch.exp(x))
    return torch.full_like(x, qk_scale)


def fwd_bwd_preprocessed(q, k, v, s, do, qk_scale: float = 1.0, feature_map: Optional[str] = None,
                         block: int = BLOCK, dtype=torch.float32):
    """o, dq, dk, dv of the operator evaluated on preprocess_qk(q), preprocess_qk(k), the gradients taken with
    respect to the RAW q and k (chain rule written out): what the kernels with the preprocessing folded into
    their load path must return."""
    qd, kd = q.to(dtype), k.to(dtype)
    o, dqm, dkm, dv = fwd_bwd(preprocess_qk(qd, qk_scale, feature_map), preprocess_qk(kd, qk_scale, feature_map), v, s, do,
                              block=block, dtype=dtype)
    return (o, dqm * preprocess_slope(qd, qk_scale, feature_map), dkm * preprocess_slope(kd, qk_scale, feature_map), dv)


def sp_chain(q, k, v, s, do, sp: int, block: int = BLOCK, dtype=torch.float32):
    """Rank recurrence of lasp/lasp_naive.py:547-568 (forward, rank r -> r+1)
    and :593-616 (backward, rank r -> r-1) over ``sp`` contiguous chunks.

    Returns per-rank lists (o, dq, dk, dv) plus the saved incoming states.
    """
    n = q.shape[2]
    assert n % sp == 0
    nl = n // sp
    chunks = [slice(r * nl, (r + 1) * nl) for r in range(sp)]
    kv = None
    kv_ins, outs = [], []
    for r in range(sp):
        kv_ins.append(None if kv is None else kv.clone())
        o, kv = blocked_forward(q[:, :, chunks[r]], k[:, :, chunks[r]], v[:, :, chunks[r]], s, kv, block, dtype)
        outs.append(o)
    dkv = None
    grads = [None] * sp
    for r in reversed(range(sp)):
        c = chunks[r]
        dq, dk, dv, dkv = blocked_backward(q[:, :, c], k[:, :, c], v[:, :, c], s, do[:, :, c],
                                           kv_ins[r], dkv, block, dtype)
        grads[r] = (dq, dk, dv)
    return outs, grads, kv_ins


def slice_wrapper(fn, q, k, v, *rest):
    """Head-dim slicing of lasp/lightning_attention.py:510-531: for d > 128 the
    op is the sum over 128-wide q,k slices (64-wide when d < 128)."""
    d = q.shape[-1]
    m = 128 if d >= 128 else 64
    arr = [m * i for i in range(d // m + 1)]
    if arr[-1] != d:
        arr.append(d)
    out = 0
    for i in range(len(arr) - 1):
        out = out + fn(q[..., arr[i]:arr[i + 1]], k[..., arr[i]:arr[i + 1]], v, *rest)
    return out


# ----------------------------------------------------------------------------
# accounting shared by bench and tests
# ----------------------------------------------------------------------------
def algorithmic_flops_per_token_head(d: int, e: int, block: int = BLOCK) -> int:
    """fwd 2B(d+e)+4de, bwd 2B(3d+2e)+8de; every required matmul counted once."""
    return 2 * block * (4 * d + 3 * e) + 12 * d * e


def algorithmic_bytes_per_token_head(d: int, e: int, itemsize: int) -> int:
    """fwd reads q,k,v writes o; bwd reads q,k,v,do writes dq,dk,dv."""
    return (6 * d + 5 * e) * itemsize
