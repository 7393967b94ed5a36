"""GPU parity: the CUDA path (through the ctypes C ABI) against the reference's
golden outputs and against the CPU oracle on seeded inputs.

Gates (max|x - ref| / max|ref|): 1e-3 for fp32 I/O, 2e-2 for bf16/fp16 I/O with
fp32 accumulation.
"""
import pytest
import torch

from oracle import lasp_oracle as O
from tests.helpers import CASES, TOL_BF16, TOL_FP32, case_inputs, golden_tensor, load_golden

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _tol(dtype):
    return TOL_FP32 if dtype == torch.float32 else TOL_BF16


def run_lightning(q, k, v, do, s, dtype, path=None, monkeypatch=None):
    from lasp_b200 import lightning_attn
    if path and monkeypatch:
        monkeypatch.setenv("LASP_B200_PATH", path)
    qd, kd, vd, dod = (t.to(DEV, dtype) for t in (q, k, v, do))
    qd.requires_grad_(True), kd.requires_grad_(True), vd.requires_grad_(True)
    o = lightning_attn(qd, kd, vd, s.to(DEV))
    o.backward(dod)
    torch.cuda.synchronize()
    return o.detach(), qd.grad, kd.grad, vd.grad


def oracle_on_rounded(q, k, v, do, s, dtype):
    """oracle in fp64-accurate fp32 on the inputs as the device sees them"""
    r = [t.to(dtype).float() for t in (q, k, v, do)]
    return O.fwd_bwd(r[0], r[1], r[2], s, r[3])


@pytest.mark.parametrize("name", sorted(CASES["single"]))
def test_lightning_attn_matches_reference_golden(name):
    p = CASES["single"][name]
    q, k, v, do, s = case_inputs(p)
    got = run_lightning(q, k, v, do, s, torch.float32)
    g = load_golden(name)
    for t, key in zip(got, ("o", "dq", "dk", "dv")):
        assert t.shape == g[key].shape
        assert O.max_rel_err(t, golden_tensor(g[key])) < TOL_FP32, key


SHAPES = [
    # b, h, n, d, e
    (1, 1, 64, 16, 16),      # one block, smallest head dims
    (2, 3, 128, 64, 64),
    (1, 2, 65, 32, 48),      # ragged: one token into the second block
    (1, 2, 1, 64, 64),       # a single token
    (2, 2, 333, 128, 64),    # the reference test's d=128, e=64, ragged n
    (1, 4, 1024, 128, 128),
    (1, 2, 512, 96, 112),    # multiples of 16 that are not powers of two
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_fp32_kernels_against_oracle(shape, dtype, monkeypatch):
    b, h, n, d, e = shape
    q, k, v, do = O.make_inputs(100 + n, b, h, n, d, e)
    s = O.baseline_slopes(h)
    got = run_lightning(q, k, v, do, s, dtype, "simt", monkeypatch)
    ref = oracle_on_rounded(q, k, v, do, s, dtype)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert t.dtype == dtype
        assert O.max_rel_err(t, r) < _tol(dtype), (key, shape)


def test_wide_heads_are_sliced(monkeypatch):
    # d = 256 (two q/k slices summed) and e = 192 (two v slices concatenated)
    q, k, v, do = O.make_inputs(5, 1, 2, 256, 256, 192)
    s = O.baseline_slopes(2)
    got = run_lightning(q, k, v, do, s, torch.float32)
    ref = O.dense_closed_form(q, k, v, s, do)
    for t, r in zip(got, ref):
        assert O.max_rel_err(t, r) < TOL_FP32


def test_no_decay_feature_map():
    # LinearTransformer-style config: s = 0, elu(x)+1 on q and k, no 1/sqrt(d)
    q, k, v, do = O.make_inputs(6, 2, 2, 512, 64, 64, scale_qk=False, feature_map="elu1")
    s = torch.zeros(2, 1, 1)
    got = run_lightning(q, k, v, do, s, torch.float32)
    ref = O.fwd_bwd(q, k, v, s, do, dtype=torch.float64)
    for t, r in zip(got, ref):
        assert O.max_rel_err(t, r) < TOL_FP32


def test_baseline_config0_full_size_fp32():
    # b=2, n=2048, h=12, d=e=128, fp32: the reference's CPU-runnable configuration
    q, k, v, do = O.make_inputs(0, 2, 12, 2048, 128, 128)
    s = O.baseline_slopes(12)
    got = run_lightning(q, k, v, do, s, torch.float32)
    ref = O.fwd_bwd(q, k, v, s, do)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, r) < TOL_FP32, key


def _chain_on_one_gpu(q, k, v, do, s, sp, dtype, path):
    """Emulate `sp` sequence-parallel ranks one after another on one device by
    threading kv/dkv states through the C-ABI calls."""
    from lasp_b200 import engine
    b, h, n, d = q.shape
    e = v.shape[-1]
    nl = n // sp
    sd = s.to(DEV)
    parts = [[t[:, :, r * nl:(r + 1) * nl].to(DEV, dtype).contiguous() for r in range(sp)] for t in (q, k, v, do)]
    plan = engine.make_plan(b, h, nl, d, e, dtype, path)
    KV = torch.full((b, h, d, e), float("nan"), device=DEV)
    fws, outs = [], []
    for r in range(sp):
        fw = engine.Forward(plan, parts[0][r], parts[1][r], parts[2][r], sd, kv_in=KV if r > 0 else None,
                            kv_out=KV if r < sp - 1 else None)
        outs.append(fw.run())
        fws.append(fw)
    DKV = torch.full((b, h, d, e), float("nan"), device=DEV)
    grads = [None] * sp
    for r in reversed(range(sp)):
        bw = engine.Backward(plan, parts[0][r], parts[1][r], parts[2][r], parts[3][r], sd, fws[r].ws,
                             dkv_in=DKV if r < sp - 1 else None, dkv_out=DKV if r > 0 else None)
        grads[r] = bw.run()
    torch.cuda.synchronize()
    o = torch.cat(outs, 2)
    dq, dk, dv = (torch.cat([g[i] for g in grads], 2) for i in range(3))
    return o, dq, dk, dv


@pytest.mark.parametrize("sp", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rank_chain_equals_single_device(sp, dtype):
    q, k, v, do = O.make_inputs(20 + sp, 2, 3, 64 * 2 * sp, 64, 32)
    s = O.baseline_slopes(3)
    got = _chain_on_one_gpu(q, k, v, do, s, sp, dtype, "simt")
    ref = oracle_on_rounded(q, k, v, do, s, dtype)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, r) < _tol(dtype), (key, sp)


def test_state_combine_and_outgoing_states():
    from lasp_b200 import engine
    b, h, n, d, e = 2, 3, 200, 32, 48
    q, k, v, do = O.make_inputs(31, b, h, n, d, e)
    s = O.baseline_slopes(h)
    kv_in = torch.randn(b, h, d, e)
    dkv_in = torch.randn(b, h, d, e)
    _, kv_ref = O.blocked_forward(q, k, v, s, kv_in)
    *_, dkv_ref = O.blocked_backward(q, k, v, s, do, kv_in, dkv_in)
    plan = engine.make_plan(b, h, n, d, e, torch.float32, "simt")
    dev = [t.to(DEV) for t in (q, k, v, do)]
    kv_out = torch.empty(b, h, d, e, device=DEV)
    dkv_out = torch.empty(b, h, d, e, device=DEV)
    fw = engine.Forward(plan, dev[0], dev[1], dev[2], s.to(DEV), kv_in=kv_in.to(DEV), kv_out=kv_out)
    fw.run()
    bw = engine.Backward(plan, dev[0], dev[1], dev[2], dev[3], s.to(DEV), fw.ws, dkv_in=dkv_in.to(DEV),
                         dkv_out=dkv_out)
    bw.run()
    assert O.max_rel_err(kv_out, kv_ref) < 1e-5
    assert O.max_rel_err(dkv_out, dkv_ref) < 1e-5
    x_local = torch.randn(b, h, d, e)
    got = engine.state_combine(s.to(DEV), kv_in.to(DEV), x_local.to(DEV), n)
    ref = torch.exp(-s.reshape(1, h, 1, 1) * n) * kv_in + x_local
    assert O.max_rel_err(got, ref) < 1e-6
    assert engine.read_status() == 0


def test_linearity_and_split_property_at_long_sequence():
    # size-independent properties at a TNL-1B-like layer slice: n = 32768 per head
    from lasp_b200 import lightning_attn
    b, h, n, d, e = 1, 2, 32768, 128, 128
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn(b, h, n, d, device=DEV, generator=g) * d ** -0.5
    k = torch.randn(b, h, n, d, device=DEV, generator=g) * d ** -0.5
    v1 = torch.randn(b, h, n, e, device=DEV, generator=g)
    v2 = torch.randn(b, h, n, e, device=DEV, generator=g)
    s = O.baseline_slopes(16)[[0, 15]].to(DEV)
    o1, o2 = lightning_attn(q, k, v1, s), lightning_attn(q, k, v2, s)
    o12 = lightning_attn(q, k, 2.0 * v1 - 0.5 * v2, s)
    assert O.max_rel_err(o12, 2.0 * o1 - 0.5 * o2) < 1e-4
    # two halves chained through the rank state == the whole sequence
    do = torch.randn(b, h, n, e, device=DEV, generator=g)
    whole = _chain_on_one_gpu(q.cpu(), k.cpu(), v1.cpu(), do.cpu(), s.cpu(), 1, torch.float32, "simt")
    halves = _chain_on_one_gpu(q.cpu(), k.cpu(), v1.cpu(), do.cpu(), s.cpu(), 2, torch.float32, "simt")
    for a, bb in zip(whole, halves):
        assert O.max_rel_err(a, bb) < 1e-4


def test_errors_are_raised_not_swallowed():
    from lasp_b200 import _cabi, lightning_attn
    q = torch.randn(1, 1, 64, 24, device=DEV)       # d not a multiple of 16: refused before any library call
    with pytest.raises(ValueError, match="multiple of 16"):
        lightning_attn(q, q, q, torch.zeros(1, 1, 1, device=DEV))
    from lasp_b200 import engine
    with pytest.raises(_cabi.LaspStatusError):      # ... and by the library itself when called directly
        engine.make_plan(1, 1, 64, 24, 24, torch.float32)
    q = torch.randn(1, 2, 64, 32, device=DEV)
    with pytest.raises(ValueError):
        lightning_attn(q, q, q, torch.zeros(3, 1, 1, device=DEV))   # wrong head count
    with pytest.raises(TypeError):
        lightning_attn(q.double(), q.double(), q.double(), torch.zeros(2, 1, 1, device=DEV))


# ---------------------------------------------------------------------------
# tensor-core path (tcgen05 / TMEM / TMA): bf16, d and e in {64, 128}, n >= 128
# ---------------------------------------------------------------------------
TENSOR_SHAPES = [
    (1, 1, 128, 128, 128),     # a single tile
    (2, 3, 256, 128, 128),
    (1, 2, 1024, 128, 128),
    (2, 12, 2048, 128, 128),   # the headline configuration, one rank: six spans of three tiles per sequence
    (2, 2, 333, 128, 64),      # the reference test's d=128, e=64 with a ragged tail
    (1, 3, 1100, 64, 128),     # ragged, 64-wide q/k
    (1, 40, 640, 64, 64),      # more sequences than a span split leaves room for
    (1, 160, 256, 128, 128),   # more sequences than SMs: one span per sequence, several items per CTA
]


@pytest.mark.parametrize("shape", TENSOR_SHAPES)
@pytest.mark.parametrize("slopes", ["baseline", "steep", "zero"])
def test_tensor_kernels_against_oracle(shape, slopes, monkeypatch):
    from lasp_b200 import engine
    b, h, n, d, e = shape
    q, k, v, do = O.make_inputs(300 + n + h, b, h, n, d, e)
    s = {"baseline": O.baseline_slopes(h), "steep": torch.full((h, 1, 1), 0.84),
         "zero": torch.zeros(h, 1, 1)}[slopes]
    assert engine.make_plan(b, h, n, d, e, torch.bfloat16, "auto").path_name == "tensor"
    got = run_lightning(q, k, v, do, s, torch.bfloat16, "tensor", monkeypatch)
    ref = oracle_on_rounded(q, k, v, do, s, torch.bfloat16)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert t.dtype == torch.bfloat16
        assert O.max_rel_err(t, r) < TOL_BF16, (key, shape, slopes)
    assert engine.read_status() == 0


@pytest.mark.parametrize("shape", [(2, 12, 2048, 128, 128), (1, 2, 333, 128, 64), (1, 3, 1100, 64, 128)])
def test_tensor_phases_equal_the_fused_launch(shape):
    """The composite calls run one fused kernel per direction (dQ apart); the separate phases - span totals,
    scan, walk - that a sequence-parallel rank uses must give the same numbers, rank states included."""
    from lasp_b200 import engine
    b, h, n, d, e = shape
    q, k, v, do = (t.to(DEV, torch.bfloat16) for t in O.make_inputs(310 + n, b, h, n, d, e))
    s = O.baseline_slopes(h).to(DEV)
    kv_in, dkv_in = torch.randn(b, h, d, e, device=DEV), torch.randn(b, h, d, e, device=DEV)
    plan = engine.make_plan(b, h, n, d, e, torch.bfloat16, "tensor")
    out = []
    for fused in (True, False):
        kv_out, dkv_out = torch.empty(b, h, d, e, device=DEV), torch.empty(b, h, d, e, device=DEV)
        fw = engine.Forward(plan, q, k, v, s, kv_in=kv_in, kv_out=kv_out)
        bw = engine.Backward(plan, q, k, v, do, s, fw.ws, dkv_in=dkv_in, dkv_out=dkv_out)
        if fused:
            fw.run(), bw.run()
        else:
            fw.chunk_states(), fw.scan(), fw.output()
            bw.chunk_states(), bw.scan(), bw.grads()
        torch.cuda.synchronize()
        out.append((fw.o, bw.dq, bw.dk, bw.dv, kv_out, dkv_out))
    for a, bb, key in zip(out[0], out[1], ("o", "dq", "dk", "dv", "kv_out", "dkv_out")):
        assert O.max_rel_err(a, bb) < (2e-3 if key.endswith("out") else 1e-2), (key, shape)
    assert engine.read_status() == 0


def test_tensor_fused_launch_repeats_on_one_workspace():
    """The fused kernels keep a launch counter and flags in the workspace: many calls on the same workspace,
    interleaved with another problem on its own workspace, stay correct."""
    from lasp_b200 import engine
    b, h, n, d, e = 2, 12, 2048, 128, 128
    q, k, v, do = (t.to(DEV, torch.bfloat16) for t in O.make_inputs(311, b, h, n, d, e))
    s = O.baseline_slopes(h).to(DEV)
    plan = engine.make_plan(b, h, n, d, e, torch.bfloat16)
    fw = engine.Forward(plan, q, k, v, s)
    bw = engine.Backward(plan, q, k, v, do, s, fw.ws)
    other = engine.Forward(engine.make_plan(1, 3, 1100, 64, 128, torch.bfloat16), *(
        t.to(DEV, torch.bfloat16) for t in O.make_inputs(312, 1, 3, 1100, 64, 128)[:3]), O.baseline_slopes(3).to(DEV))
    first = None
    for _ in range(20):
        fw.run(), other.run(), bw.run()
        got = tuple(t.clone() for t in (fw.o, bw.dq, bw.dk, bw.dv))
        if first is None:
            first = got
        for a, bb in zip(first, got):
            assert torch.equal(a, bb)
    ref = oracle_on_rounded(*(t.float().cpu() for t in (q, k, v, do)), s.cpu(), torch.bfloat16)
    for t, r in zip(first, ref):
        assert O.max_rel_err(t, r) < TOL_BF16
    assert engine.read_status() == 0


@pytest.mark.parametrize("shape", [(8, 12, 512, 128, 64), (2, 12, 2048, 128, 128), (1, 3, 1100, 64, 128)])
def test_tensor_kernels_repeat_bit_for_bit_under_load(shape):
    """Races between the kernels' asynchronous agents (TMA, tensor cores, warps) show as run-to-run
    differences: forty forward + backward runs of a shape with many short sequences (the reference test's
    per-rank shape at SP=4), of the headline shape and of a ragged one must agree to the bit."""
    from lasp_b200 import engine
    b, h, n, d, e = shape
    q, k, v, do = (t.to(DEV, torch.bfloat16) for t in O.make_inputs(320 + n, b, h, n, d, e, scale_qk=False))
    s = O.build_slope_tensor_ref(h).to(torch.float32).to(DEV)
    plan = engine.make_plan(b, h, n, d, e, torch.bfloat16)
    kv_out, dkv_out = torch.empty(b, h, d, e, device=DEV), torch.empty(b, h, d, e, device=DEV)
    fw = engine.Forward(plan, q, k, v, s, kv_out=kv_out)
    bw = engine.Backward(plan, q, k, v, do, s, fw.ws, dkv_out=dkv_out)
    first = None
    for _ in range(40):
        for t in (fw.o, bw.dq, bw.dk, bw.dv):
            t.zero_()
        fw.run(), bw.run()
        got = tuple(t.clone() for t in (fw.o, bw.dq, bw.dk, bw.dv, kv_out, dkv_out))
        if first is None:
            first = got
        for a, bb, key in zip(first, got, ("o", "dq", "dk", "dv", "kv_out", "dkv_out")):
            assert torch.equal(a, bb), key
    ref = oracle_on_rounded(*(t.float().cpu() for t in (q, k, v, do)), s.cpu(), torch.bfloat16)
    for t, r, key in zip(first, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, r) < TOL_BF16, key
    assert engine.read_status() == 0


@pytest.mark.parametrize("sp", [2, 4])
def test_tensor_rank_chain_equals_single_device(sp):
    from lasp_b200 import engine
    q, k, v, do = O.make_inputs(40 + sp, 2, 2, 256 * sp, 128, 128)
    s = O.baseline_slopes(16)[[3, 12]]
    got = _chain_on_one_gpu(q, k, v, do, s, sp, torch.bfloat16, "tensor")
    ref = oracle_on_rounded(q, k, v, do, s, torch.bfloat16)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, r) < TOL_BF16, (key, sp)
    assert engine.read_status() == 0


def test_tensor_path_outgoing_states():
    from lasp_b200 import engine
    b, h, n, d, e = 1, 2, 512, 128, 128
    q, k, v, do = O.make_inputs(77, b, h, n, d, e)
    s = O.baseline_slopes(2)
    kv_in, dkv_in = torch.randn(b, h, d, e), torch.randn(b, h, d, e)
    r = [t.to(torch.bfloat16).float() for t in (q, k, v, do)]
    _, kv_ref = O.blocked_forward(r[0], r[1], r[2], s, kv_in)
    *_, dkv_ref = O.blocked_backward(r[0], r[1], r[2], s, r[3], kv_in, dkv_in)
    plan = engine.make_plan(b, h, n, d, e, torch.bfloat16, "tensor")
    dev = [t.to(DEV, torch.bfloat16) for t in (q, k, v, do)]
    kv_out, dkv_out = torch.empty(b, h, d, e, device=DEV), torch.empty(b, h, d, e, device=DEV)
    fw = engine.Forward(plan, dev[0], dev[1], dev[2], s.to(DEV), kv_in=kv_in.to(DEV), kv_out=kv_out)
    fw.run()
    bw = engine.Backward(plan, dev[0], dev[1], dev[2], dev[3], s.to(DEV), fw.ws, dkv_in=dkv_in.to(DEV),
                         dkv_out=dkv_out)
    bw.run()
    # the states are fp32 sums of products of bf16 operands (row decays rounded to bf16 with them)
    e1, e2 = O.max_rel_err(kv_out, kv_ref), O.max_rel_err(dkv_out, dkv_ref)
    print("outgoing state errors", e1, e2)
    assert e1 < 5e-3 and e2 < 5e-3


def test_tensor_long_sequence_tnl1b_slice():
    # TNL-1B attention shape (h=16, d=e=128, b=1), one rank's share at SP=8 of a 131072-token sequence
    b, h, n, d, e = 1, 16, 16384, 128, 128
    q, k, v, do = O.make_inputs(91, b, h, n, d, e)
    s = O.baseline_slopes(h)
    got = run_lightning(q, k, v, do, s, torch.bfloat16)
    ref = oracle_on_rounded(q, k, v, do, s, torch.bfloat16)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, r) < TOL_BF16, key


def test_tensor_wide_qk_is_sliced_bf16():
    # d = 256: two 128-wide q/k slices, each on the tensor-core path, outputs summed
    b, h, n, d, e = 1, 2, 512, 256, 128
    q, k, v, do = O.make_inputs(92, b, h, n, d, e)
    s = O.baseline_slopes(h)
    got = run_lightning(q, k, v, do, s, torch.bfloat16)
    r = [t.to(torch.bfloat16).float() for t in (q, k, v, do)]
    ref = O.dense_closed_form(r[0], r[1], r[2], s, r[3])
    for t, w, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, w) < 2.5e-2, key     # o is a sum of two bf16-rounded slice outputs


@pytest.mark.parametrize("d,e", [(64, 64), (64, 128), (128, 64)])
def test_tensor_head64_variants(d, e):
    """64-wide heads run on the tensor-core kernels too (any mix of 64 and 128 for q/k and v)."""
    from lasp_b200 import engine
    b, h, n = 2, 4, 512
    assert engine.make_plan(b, h, n, d, e, torch.bfloat16).path_name == "tensor"
    q, k, v, do = O.make_inputs(93 + d + e, b, h, n, d, e)
    s = O.baseline_slopes(h)
    got = run_lightning(q, k, v, do, s, torch.bfloat16)
    ref = oracle_on_rounded(q, k, v, do, s, torch.bfloat16)
    for t, r, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, r) < TOL_BF16, (key, d, e)
    assert engine.read_status() == 0


@pytest.mark.parametrize("width", [64, 128, 256])
def test_no_decay_linear_transformer_config_bf16(width):
    """The no-decay (LinearTransformer-style) configuration at reduced length: s = 0, elu(x)+1 feature map on q
    and k (applied by the caller, no 1/sqrt(d)), d = e in {64, 128, 256}, bf16: 64 and 128 on the tensor-core
    kernels, 256 as 128-wide slices of both head dimensions."""
    from lasp_b200 import engine
    b, h, n = 1, 2, 1024
    assert engine.make_plan(b, h, n, min(width, 128), min(width, 128), torch.bfloat16).path_name == "tensor"
    q, k, v, do = O.make_inputs(97 + width, b, h, n, width, width, scale_qk=False, feature_map="elu1")
    s = torch.zeros(h, 1, 1)
    got = run_lightning(q, k, v, do, s, torch.bfloat16)
    r = [t.to(torch.bfloat16).float() for t in (q, k, v, do)]
    ref = O.dense_closed_form(r[0], r[1], r[2], s, r[3])
    gate = TOL_BF16 if width <= 128 else 2.5e-2          # 256: sums of bf16-rounded slice results
    for t, w, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, w) < gate, (key, width)


def run_lightning_fused(q, k, v, do, s, dtype, qk_scale, feature_map):
    from lasp_b200 import lightning_attn_fused
    qd, kd, vd, dod = (t.to(DEV, dtype) for t in (q, k, v, do))
    qd.requires_grad_(True), kd.requires_grad_(True), vd.requires_grad_(True)
    o = lightning_attn_fused(qd, kd, vd, s.to(DEV), qk_scale=qk_scale, feature_map=feature_map)
    o.backward(dod)
    torch.cuda.synchronize()
    return o.detach(), qd.grad, kd.grad, vd.grad


def test_folded_preprocessing_reproduces_the_reference_elu_case():
    """elu(x)+1 folded into the kernels, on the RAW draws of the reference's no-decay case (bf16, tensor-core
    kernels): the output must be the reference's output for the mapped inputs, dv its dv, and dq, dk its
    gradients times the slope of the map."""
    from lasp_b200 import _core
    p = dict(CASES["single"]["lightning_fp32_nodecay_elu"])
    g = load_golden("lightning_fp32_nodecay_elu")
    q, k, v, do, s = case_inputs(dict(p, feature_map=None))
    qb, kb = q.to(torch.bfloat16), k.to(torch.bfloat16)
    assert _core.kernels_preprocess(qb.to(DEV), v.to(DEV, torch.bfloat16), 1.0, "elu1")   # really in the kernels
    o, dq, dk, dv = run_lightning_fused(q, k, v, do, s, torch.bfloat16, 1.0, "elu1")
    assert O.max_rel_err(o, golden_tensor(g["o"])) < TOL_BF16
    assert O.max_rel_err(dv, golden_tensor(g["dv"])) < TOL_BF16
    assert O.max_rel_err(dq, golden_tensor(g["dq"]) * O.preprocess_slope(qb.float(), 1.0, "elu1")) < TOL_BF16
    assert O.max_rel_err(dk, golden_tensor(g["dk"]) * O.preprocess_slope(kb.float(), 1.0, "elu1")) < TOL_BF16


FOLDED = [  # b, h, n, d, e, slopes, scale, map
    (2, 3, 512, 128, 128, "baseline", 128 ** -0.5, None),
    (2, 3, 512, 128, 128, "zero", 1.0, "elu1"),
    (1, 2, 333, 64, 128, "baseline", 0.5, "elu1"),
    (1, 4, 1100, 128, 64, "zero", 64 ** -0.5, "elu1"),
    (2, 12, 2048, 128, 128, "baseline", 128 ** -0.5, "elu1"),     # several spans per sequence: the fused launches
    (4, 40, 256, 64, 64, "steep", 0.25, "elu1"),                  # more sequences than SMs
    (1, 2, 384, 256, 256, "zero", 1.0, "elu1"),                   # 128-wide slices stacked along the batch
]


@pytest.mark.parametrize("b,h,n,d,e,slopes,scale,fmap", FOLDED)
def test_folded_preprocessing_matches_oracle(b, h, n, d, e, slopes, scale, fmap):
    """qk_scale * map(.) of q and k inside the tensor-core kernels, gradients with respect to the raw q, k,
    against the oracle with the chain rule written out (ragged n, both head widths, with and without decay)."""
    from lasp_b200 import _core
    q, k, v, do = O.make_inputs(500 + n + d, b, h, n, d, e, scale_qk=False)
    s = {"baseline": O.baseline_slopes(h), "zero": torch.zeros(h, 1, 1),
         "steep": torch.full((h, 1, 1), 0.6)}[slopes]
    r = [t.to(torch.bfloat16).float() for t in (q, k, v, do)]
    assert _core.kernels_preprocess(q[..., :128].to(DEV, torch.bfloat16), v[..., :128].to(DEV, torch.bfloat16), scale, fmap)
    got = run_lightning_fused(q, k, v, do, s, torch.bfloat16, scale, fmap)
    if d <= 128:
        ref = O.fwd_bwd_preprocessed(r[0], r[1], r[2], s, r[3], scale, fmap)
    else:
        o, dqm, dkm, dv = O.dense_closed_form(O.preprocess_qk(r[0], scale, fmap), O.preprocess_qk(r[1], scale, fmap),
                                              r[2], s, r[3])
        ref = (o, dqm * O.preprocess_slope(r[0], scale, fmap), dkm * O.preprocess_slope(r[1], scale, fmap), dv)
    gate = TOL_BF16 if d <= 128 else 2.5e-2
    for t, w, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, w) < gate, key
    # and the same numbers as the preprocessing done by the caller in front of the plain operator
    qm = O.preprocess_qk(r[0], scale, fmap).to(torch.bfloat16).float()
    km = O.preprocess_qk(r[1], scale, fmap).to(torch.bfloat16).float()
    plain = run_lightning(qm, km, r[2], r[3], s, torch.bfloat16)
    assert O.max_rel_err(got[0], plain[0].float()) < TOL_BF16
    assert O.max_rel_err(got[3], plain[3].float()) < TOL_BF16


def test_folded_preprocessing_falls_back_to_torch_where_the_kernels_cannot():
    """fp32 inputs run on the FFMA kernels, which have no folded preprocessing: same result through torch."""
    from lasp_b200 import _core
    q, k, v, do = O.make_inputs(77, 1, 2, 200, 64, 64, scale_qk=False)
    s = O.baseline_slopes(2)
    assert not _core.kernels_preprocess(q.to(DEV), v.to(DEV), 0.125, "elu1")
    got = run_lightning_fused(q, k, v, do, s, torch.float32, 0.125, "elu1")
    ref = O.fwd_bwd_preprocessed(q, k, v, s, do, 0.125, "elu1")
    for t, w, key in zip(got, ref, ("o", "dq", "dk", "dv")):
        assert O.max_rel_err(t, w) < TOL_FP32, key


def test_wide_heads_run_in_place_and_a_wrong_pitch_is_refused():
    """d = e = 256 in bf16: the 128-wide slice pairs run on the wide tensors in place (row pitch 256), and a tensor
    whose pitch is not the plan's is refused before anything is launched."""
    from lasp_b200 import _core, engine
    b, h, n = 1, 2, 256
    q, k, v, do = (t.to(DEV, torch.bfloat16) for t in O.make_inputs(5, b, h, n, 256, 256))
    assert _core._slices_in_place(q, v, 1.0, None)
    plan = engine.make_plan(b, h, n, 128, 128, torch.bfloat16, pitch_d=256, pitch_e=256)
    s = O.baseline_slopes(h)
    with pytest.raises(ValueError):
        engine.Forward(plan, q[..., :128], k[..., :128], v[..., :128], s)          # o would be a tensor of its own
    with pytest.raises(ValueError):
        engine.Forward(plan, q[..., :128].contiguous(), k[..., :128], v[..., :128], s, o=torch.empty_like(v)[..., :128])
    canary = torch.full_like(v, 7.0)
    fw = engine.Forward(plan, q[..., 128:], k[..., 128:], v[..., :128], s, o=canary[..., 128:])
    fw.run()
    torch.cuda.synchronize()
    assert bool((canary[..., :128] == 7.0).all())                                   # the other half is untouched
    ref = O.blocked_forward(q[..., 128:].float().cpu(), k[..., 128:].float().cpu(), v[..., :128].float().cpu(), s)[0]
    assert O.max_rel_err(canary[..., 128:].float().cpu(), ref) < TOL_BF16
    assert engine.read_status() == 0


def test_exchange_wait_runs_out_and_is_reported():
    """Failure detection without a GPU fault: the last rank of a group of two whose sender never writes.  The
    hand-over kernel's waits are bounded, so it must come back on its own, set the relay bit (4) of the fault
    word, poison the states it could not complete with NaN, and leave the context usable; the host-side check
    turns the bit into an exception."""
    import ctypes as C
    import lasp_b200
    from lasp_b200 import _cabi, engine
    b, h, n, d, e = 1, 2, 256, 64, 64
    q, k, v, do = (t.to(DEV, torch.bfloat16) for t in O.make_inputs(98, b, h, n, d, e))
    s = torch.tensor([0.0, 0.01], device=DEV)
    plan = engine.make_plan(b, h, n, d, e, torch.bfloat16)
    fw = engine.Forward(plan, q, k, v, s)
    fw.chunk_states()
    elems = b * h * d * e
    slots = torch.zeros(2 * 2 * elems * 2, dtype=torch.int32, device=DEV)      # {value, step} words, step 0 = stale
    acks = torch.zeros(2 * 8 * 32, dtype=torch.int32, device=DEV)
    counters = torch.zeros(64, dtype=torch.int32, device=DEV)
    a = _cabi.ExchangeArgs()
    a.ranks, a.position, a.reverse = 2, 1, 0                                    # the last of two: receives only
    a.s, a.ws, a.ws_bytes = s.data_ptr(), fw.ws.data_ptr(), fw.ws.numel()
    a.my_slots, a.my_acks, a.counters = slots.data_ptr(), acks.data_ptr(), counters.data_ptr()
    a.peer_acks[0] = acks.data_ptr()          # the absent sender's acknowledgement words: any writable memory
    a.wait_clocks = 200000                    # about 0.1 ms
    assert engine.read_status() == 0
    engine.exchange_scan(plan, a, torch.device(DEV))
    fw.output()
    torch.cuda.synchronize()
    assert counters[0].item() == 1            # the step was still counted
    assert torch.isnan(fw.o.float()).any()    # a state that never arrived cannot pass for one that did
    with pytest.raises(engine.KernelFault) as info:
        lasp_b200.check_faults()
    assert info.value.word == 4
    # the device is fine: an ordinary call still works and reports no fault
    q2, k2, v2, do2 = O.make_inputs(98, 1, 2, 128, 32, 32)
    got = run_lightning(q2, k2, v2, do2, O.baseline_slopes(2), torch.float32)
    ref = O.fwd_bwd(q2, k2, v2, O.baseline_slopes(2), do2)
    assert O.max_rel_err(got[0], ref[0]) < TOL_FP32
    lasp_b200.check_faults()


def test_fault_watch_raises_at_the_next_call():
    """The operators look at the fault word one step late, without synchronising: a copy of the word to
    pinned memory is queued behind a step and read when the next call starts."""
    from lasp_b200 import engine
    watch = engine._FaultWatch()
    watch.arm(torch.device(DEV))
    torch.cuda.synchronize()
    watch.poll()                               # nothing reported: no exception
    watch.host.fill_(4)                        # what the queued copy would have delivered after a late peer
    watch.event = torch.cuda.Event()
    watch.event.record()
    torch.cuda.synchronize()
    with pytest.raises(engine.KernelFault):
        watch.poll()


@pytest.mark.parametrize("path,dtype,shape", [("tensor", torch.bfloat16, (2, 3, 512, 128, 128)),
                                              ("simt", torch.float32, (1, 2, 333, 64, 48))])
def test_runs_are_bitwise_repeatable(path, dtype, shape, monkeypatch):
    """No atomics or order-dependent reductions on the data path: two runs give identical bits."""
    b, h, n, d, e = shape
    q, k, v, do = O.make_inputs(99, b, h, n, d, e)
    s = O.baseline_slopes(h)
    first = run_lightning(q, k, v, do, s, dtype, path, monkeypatch)
    second = run_lightning(q, k, v, do, s, dtype, path, monkeypatch)
    for a, bb in zip(first, second):
        assert torch.equal(a, bb)


@pytest.mark.parametrize("path,dtype,shape", [("tensor", torch.bfloat16, (1, 2, 256, 128, 128)),
                                              ("simt", torch.float32, (1, 2, 100, 32, 48))])
def test_forward_writes_stay_inside_their_buffers(path, dtype, shape):
    """Canaries around the output and the workspace: nothing is written outside what the caller handed over."""
    from lasp_b200 import engine
    b, h, n, d, e = shape
    q, k, v, _ = O.make_inputs(100, b, h, n, d, e)
    q, k, v = (t.to(DEV, dtype) for t in (q, k, v))
    s = O.baseline_slopes(h).to(DEV)
    plan = engine.make_plan(b, h, n, d, e, dtype, path)
    pad = 4096
    o_buf = torch.full((b * h * n * e + 2 * pad,), 7.0, dtype=dtype, device=DEV)
    ws_buf = torch.full((plan.ws_bytes + 2 * pad,), 0x5A, dtype=torch.uint8, device=DEV)
    o = o_buf[pad:pad + b * h * n * e].view(b, h, n, e)
    ws = ws_buf[pad:pad + plan.ws_bytes]
    ws[:engine.SYNC_BYTES].zero_()     # the fused kernels keep their launch counter and flags there
    kv_out = torch.empty(b, h, d, e, device=DEV)
    engine.Forward(plan, q, k, v, s, kv_out=kv_out, o=o, ws=ws).run()
    torch.cuda.synchronize()
    assert torch.all(o_buf[:pad] == 7.0) and torch.all(o_buf[-pad:] == 7.0)
    assert torch.all(ws_buf[:pad] == 0x5A) and torch.all(ws_buf[-pad:] == 0x5A)
    ref, kv_ref = O.blocked_forward(q.float().cpu(), k.float().cpu(), v.float().cpu(), s.cpu())
    assert O.max_rel_err(o, ref) < _tol(dtype)
    assert O.max_rel_err(kv_out, kv_ref) < 1e-2
