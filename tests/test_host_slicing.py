"""Host-side head-dim slicing (lasp_b200._core.sliced_apply) and oracle properties, on the CPU."""
import pytest
import torch
from hypothesis import given, settings, strategies as st

from lasp_b200._core import _cuts, sliced_apply
from oracle import lasp_oracle as O


def test_cuts():
    assert _cuts(64) == [(0, 64)]
    assert _cuts(128) == [(0, 128)]
    assert _cuts(192) == [(0, 128), (128, 192)]
    assert _cuts(256) == [(0, 128), (128, 256)]
    assert _cuts(384) == [(0, 128), (128, 256), (256, 384)]


@pytest.mark.parametrize("d,e", [(64, 64), (256, 64), (128, 192), (256, 256), (160, 320)])
def test_sliced_apply_equals_unsliced_operator(d, e):
    """q/k slices are summed, v slices concatenated, state buffers cut alongside: with an exact per-slice
    operator the sliced result equals the operator on the full head dimensions.  When both widths are
    multiples of 128 the slice pairs are stacked along the batch and go through a single call."""
    b, h, n = 1, 2, 96
    q, k, v, _ = O.make_inputs(3, b, h, n, d, e)
    s = O.baseline_slopes(h)
    kv_in = torch.randn(b, h, d, e, dtype=torch.float64)
    calls = []

    def op(qs, ks, vs, kv):
        assert qs.shape[-1] <= 128 and vs.shape[-1] <= 128 and kv.shape[-2:] == (qs.shape[-1], vs.shape[-1])
        assert kv.shape[0] == qs.shape[0] == vs.shape[0]
        calls.append((qs.shape[0], qs.shape[-1], vs.shape[-1]))
        return O.blocked_forward(qs, ks, vs, s, kv, dtype=torch.float64)[0]

    got = sliced_apply(op, q.double(), k.double(), v.double(), (kv_in,))
    ref = O.blocked_forward(q, k, v, s, kv_in, dtype=torch.float64)[0]
    assert got.shape == ref.shape
    assert O.max_rel_err(got, ref) < 1e-12
    pairs = len(_cuts(d)) * len(_cuts(e))
    if d % 128 == 0 and e % 128 == 0 and pairs > 1:
        assert calls == [(pairs * b, 128, 128)]          # one call: one state hand-over per direction
    else:
        assert len(calls) == pairs


@settings(max_examples=25, deadline=None)
@given(b=st.integers(1, 2), h=st.integers(1, 3), blocks=st.integers(1, 6), sp=st.sampled_from([1, 2, 3]),
       d=st.sampled_from([16, 32, 48]), e=st.sampled_from([16, 32]), seed=st.integers(0, 1000),
       s_scale=st.sampled_from([0.0, 0.05, 1.0]))
def test_rank_chain_equals_whole_sequence(b, h, blocks, sp, d, e, seed, s_scale):
    """Property: cutting the sequence into ranks and passing KV / dKV states reproduces the single-device result
    for any shape, group size and decay (including none)."""
    n = 64 * blocks * sp
    q, k, v, do = O.make_inputs(seed, b, h, n, d, e)
    s = O.baseline_slopes(h) * s_scale
    ref = O.dense_closed_form(q, k, v, s, do)
    outs, grads, _ = O.sp_chain(q, k, v, s, do, sp, dtype=torch.float64)
    assert O.max_rel_err(torch.cat(outs, 2), ref[0]) < 1e-10
    for i in range(3):
        assert O.max_rel_err(torch.cat([g[i] for g in grads], 2), ref[i + 1]) < 1e-10


@settings(max_examples=15, deadline=None)
@given(n=st.integers(1, 200), seed=st.integers(0, 100))
def test_ragged_lengths_blocked_equals_dense(n, seed):
    q, k, v, do = O.make_inputs(seed, 1, 2, n, 16, 16)
    s = O.baseline_slopes(2)
    ref = O.dense_closed_form(q, k, v, s, do)
    got = O.fwd_bwd(q, k, v, s, do, dtype=torch.float64)
    for a, r in zip(got, ref):
        assert O.max_rel_err(a, r) < 1e-10
    # outgoing state is decayed to position n exactly: feeding it to a second segment continues the sequence
    _, kv = O.blocked_forward(q, k, v, s, dtype=torch.float64)
    q2, k2, v2, _ = O.make_inputs(seed + 1, 1, 2, 37, 16, 16)
    o2, _ = O.blocked_forward(q2, k2, v2, s, kv, dtype=torch.float64)
    whole = O.dense_closed_form(torch.cat([q, q2], 2), torch.cat([k, k2], 2), torch.cat([v, v2], 2), s)
    assert O.max_rel_err(o2, whole[:, :, n:]) < 1e-10


def test_layout_check_of_a_call():
    """The guard in front of every launch: tensors must have the row pitch their plan was made for; strides of
    unit dimensions do not count (a chunk cut out of a longer sequence keeps the long sequence's strides)."""
    from types import SimpleNamespace
    from lasp_b200 import engine
    b, h, n = 1, 1, 128
    plan = SimpleNamespace(b=b, h=h, n=n, d=64, e=64, problem=SimpleNamespace(pitch_d=0, pitch_e=0))
    whole = torch.zeros(b, h, 2 * n, 64)
    chunk = whole[:, :, n:]                                   # contiguous rows, batch/head strides of the long tensor
    engine._check_layout(plan, q=chunk, k=chunk.contiguous(), v=chunk, o=None)
    wide = torch.zeros(b, h, n, 256)
    with pytest.raises(ValueError):
        engine._check_layout(plan, q=wide[..., :64])          # row pitch 256, plan says 64
    with pytest.raises(ValueError):
        engine._check_layout(plan, q=torch.zeros(b, h, n, 32))
    sliced = SimpleNamespace(b=2, h=3, n=n, d=128, e=128, problem=SimpleNamespace(pitch_d=256, pitch_e=256))
    wide = torch.zeros(2, 3, n, 256)
    engine._check_layout(sliced, q=wide[..., 128:], dv=wide[..., :128])
    with pytest.raises(ValueError):
        engine._check_layout(sliced, q=wide[..., 128:].contiguous())
