"""The oracle against the reference's own outputs (CPU, no GPU needed).

The fixtures under tests/golden/ were produced by the reference's Triton
kernels run through Triton's interpreter (tests/golden/make_golden.py).
"""
import numpy as np
import pytest
import torch

from oracle import lasp_oracle as O
from tests.helpers import CASES, case_inputs, golden_tensor, input_checksum, load_golden, slopes_for, split

TOL = 2e-6  # fp32 vs fp32, different summation order


@pytest.mark.parametrize("name", sorted(CASES["single"]))
def test_blocked_oracle_matches_reference_lightning(name):
    p = CASES["single"][name]
    q, k, v, do, s = case_inputs(p)
    g = load_golden(name)
    assert abs(input_checksum(q, k, v, do) - float(g["checksum"])) < 1e-6 * float(g["checksum"])

    def op(qs, ks, vs):
        return O.blocked_forward(qs, ks, vs, s)[0]

    o = O.slice_wrapper(op, q, k, v)
    assert O.max_rel_err(o, golden_tensor(g["o"])) < TOL
    # gradients: sum over d-slices is what autograd does in the reference wrapper
    d = p["d"]
    m = 128 if d >= 128 else 64
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.zeros_like(v)
    for lo in range(0, d, m):
        hi = min(lo + m, d)
        gq, gk, gv, _ = O.blocked_backward(q[..., lo:hi], k[..., lo:hi], v, s, do)
        dq[..., lo:hi], dk[..., lo:hi] = gq, gk
        dv += gv
    assert O.max_rel_err(dq, golden_tensor(g["dq"])) < TOL
    assert O.max_rel_err(dk, golden_tensor(g["dk"])) < TOL
    assert O.max_rel_err(dv, golden_tensor(g["dv"])) < TOL


@pytest.mark.parametrize("name", sorted(CASES["single"]))
def test_dense_closed_form_matches_reference_lightning(name):
    p = CASES["single"][name]
    q, k, v, do, s = case_inputs(p)
    g = load_golden(name)
    o, dq, dk, dv = O.dense_closed_form(q, k, v, s, do)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert O.max_rel_err(got, golden_tensor(g[key])) < TOL, key


@pytest.mark.parametrize("name", sorted(CASES["sp"]))
def test_sp_chain_matches_reference_variants(name):
    p = CASES["sp"][name]
    q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"])
    s = slopes_for(p["slopes"], p["h"])
    g = load_golden(name)
    assert abs(input_checksum(q, k, v, do) - float(g["checksum"])) < 1e-6 * float(g["checksum"])
    bf16 = p["dtype"] == "bfloat16"
    # the reference's own variants differ from each other by up to ~7e-3 in bf16
    tol = 1.5e-2 if bf16 else TOL
    for dp_rank in range(p["dp"]):
        cast = (lambda t: t.to(torch.bfloat16).float()) if bf16 else (lambda t: t)
        parts = [[split(cast(t), p["dp"], p["sp"], dp_rank, r) for r in range(p["sp"])] for t in (q, k, v, do)]
        qg, kg, vg, dog = (torch.cat(x, dim=2) for x in parts)
        outs, grads, _ = O.sp_chain(qg, kg, vg, s, dog, p["sp"])
        for sp_rank in range(p["sp"]):
            rank = dp_rank * p["sp"] + sp_rank
            for var in CASES["variants"]:
                ref = {nm: golden_tensor(g[f"rank{rank}_{var}_{nm}"]) for nm in ("o", "dq", "dk", "dv")}
                got = dict(o=outs[sp_rank], dq=grads[sp_rank][0], dk=grads[sp_rank][1], dv=grads[sp_rank][2])
                for nm in ref:
                    assert O.max_rel_err(got[nm], ref[nm]) < tol, (rank, var, nm)


def test_blocked_equals_dense_fp64_long():
    q, k, v, do = O.make_inputs(7, 1, 3, 1000, 64, 48)
    s = O.baseline_slopes(3)
    ref = O.dense_closed_form(q, k, v, s, do)
    got = O.fwd_bwd(q, k, v, s, do, dtype=torch.float64)
    for a, b in zip(got, ref):
        assert O.max_rel_err(a, b) < 1e-12


def test_incoming_states_equal_longer_sequence():
    # running the second half with the first half's state == running the whole sequence
    q, k, v, do = O.make_inputs(8, 2, 2, 384, 32, 32)
    s = O.baseline_slopes(2)
    ref = O.dense_closed_form(q, k, v, s, do)
    outs, grads, _ = O.sp_chain(q, k, v, s, do, 3, dtype=torch.float64)
    assert O.max_rel_err(torch.cat(outs, 2), ref[0]) < 1e-12
    for i in range(3):
        assert O.max_rel_err(torch.cat([g[i] for g in grads], 2), ref[i + 1]) < 1e-12


def test_preprocessed_oracle_against_the_reference_and_autograd():
    """The operator with q,k preprocessing folded in: on the raw inputs of the reference's no-decay elu(x)+1 case
    it must reproduce the reference's output, its dk, dq times the map's slope, and what autograd gives."""
    p = dict(CASES["single"]["lightning_fp32_nodecay_elu"])
    g = load_golden("lightning_fp32_nodecay_elu")
    raw = dict(p, feature_map=None)
    q, k, v, do, s = case_inputs(raw)                      # the same draws, before elu(x)+1
    o, dq, dk, dv = O.fwd_bwd_preprocessed(q, k, v, s, do, 1.0, "elu1")
    assert O.max_rel_err(o, golden_tensor(g["o"])) < TOL
    assert O.max_rel_err(dv, golden_tensor(g["dv"])) < TOL
    assert O.max_rel_err(dq, golden_tensor(g["dq"]) * O.preprocess_slope(q, 1.0, "elu1")) < TOL
    assert O.max_rel_err(dk, golden_tensor(g["dk"]) * O.preprocess_slope(k, 1.0, "elu1")) < TOL
    # and with a scale, against autograd through the dense closed form in fp64
    c = 0.37
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    od = O.dense_closed_form(O.preprocess_qk(qd, c, "elu1"), O.preprocess_qk(kd, c, "elu1"), vd, s)
    od.backward(do.double())
    got = O.fwd_bwd_preprocessed(q, k, v, s, do, c, "elu1", dtype=torch.float64)
    for t, r in zip(got, (od.detach(), qd.grad, kd.grad, vd.grad)):
        assert O.max_rel_err(t, r) < 1e-10


def test_slopes_match_reference_function(golden_dir):
    with np.load(golden_dir + "/build_slope_tensor.npz") as z:
        for key in z.files:
            h = int(key[1:])
            assert np.array_equal(O.build_slope_tensor_ref(h).numpy(), z[key])
    # the two slope rules agree for power-of-two head counts
    for h in (8, 16, 32):
        assert torch.allclose(O.baseline_slopes(h), O.build_slope_tensor_ref(h).float(), rtol=1e-6)


def test_flop_and_byte_accounting():
    assert O.algorithmic_flops_per_token_head(128, 128) == 311296
    assert O.algorithmic_flops_per_token_head(64, 64) == 106496
    assert O.algorithmic_bytes_per_token_head(128, 128, 2) == 2816
