"""Sequence-parallel operators on real GPUs over NCCL (needs >= 2 devices).

Every rank runs the four operators on its (dp_rank, sp_rank) chunk of seeded
global tensors and checks O, dQ, dK, dV against the reference's golden outputs
(tests/golden) or the CPU oracle's rank chain.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import lasp_oracle as O
from tests.helpers import CASES, TOL_BF16, TOL_FP32, golden_tensor, load_golden, slopes_for, split

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_variants(lasp, qi, ki, vi, doi, s):
    bl, h, _, d = qi.shape
    e = vi.shape[-1]
    out = {}
    for var in ("naive", "cache", "fuse", "fuse_parallel"):
        qi.grad = ki.grad = vi.grad = None
        qi.requires_grad_(True), ki.requires_grad_(True), vi.requires_grad_(True)
        KV = torch.full((bl, h, d, e), float("nan"), device=qi.device)
        DKV = torch.full((bl, h, d, e), float("nan"), device=qi.device)
        if var == "naive":
            oi = lasp.lasp_naive(qi, ki, vi, s)
        elif var == "cache":
            oi = lasp.lasp_cache(qi, ki, vi, s, torch.arange(qi.shape[2]).to(qi), KV, DKV)
        else:
            oi = getattr(lasp, "lasp_" + var)(qi, ki, vi, s, KV, DKV)
        oi.backward(doi)
        torch.cuda.synchronize()
        out[var] = dict(o=oi.detach().float().cpu(), dq=qi.grad.float().cpu(), dk=ki.grad.float().cpu(),
                        dv=vi.grad.float().cpu())
        dist.barrier()
    return out


def _worker(rank, world, port, mode, params, errq):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        os.environ["LASP_B200_TRANSPORT"] = params.get("transport", "auto")
        torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))   # the ranks share the host cores
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        import lasp
        from lasp.utils import initialize_lasp
        from lasp_b200 import engine
        p = params
        initialize_lasp(p["dp"], p["sp"])
        dp_rank, sp_rank = rank // p["sp"], rank % p["sp"]
        dtype = getattr(torch, p["dtype"])
        s = slopes_for(p["slopes"], p["h"])
        if mode == "golden":
            q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"])
            qi, ki, vi, doi = (split(t.to(dtype), p["dp"], p["sp"], dp_rank, sp_rank).to(dev) for t in (q, k, v, do))
        else:
            # The global tensors are defined piecewise - one seeded draw per (tensor, global batch row,
            # sequence-parallel chunk) - so that a rank only generates its own chunk plus, for the oracle,
            # the checked heads of its batch rows.
            nl, bl = p["n"] // p["sp"], p["b"] // p["dp"]

            def piece(which, b_global, chunk):
                g = torch.Generator().manual_seed(((p["seed"] * 4 + which) * 4096 + b_global) * 64 + chunk)
                width = p["d"] if which < 2 else p["e"]
                t = torch.randn(p["h"], nl, width, generator=g)
                return t * p["d"] ** -0.5 if (which < 2 and p.get("scale_qk", True)) else t

            rows = [i * p["dp"] + dp_rank for i in range(bl)]   # batch interleaved over dp
            qi, ki, vi, doi = (torch.stack([piece(w, bg, sp_rank) for bg in rows]).to(dtype).to(dev)
                               for w in range(4))
        if mode == "fold":
            # the operator with the q,k preprocessing folded into the kernels, on the raw draws; the oracle chain
            # runs on the preprocessed tensors and its dq, dk take the chain rule afterwards
            import lasp_b200
            c, fmap = p["fold"]
            bl_, h_, _, d_ = qi.shape
            qi.requires_grad_(True), ki.requires_grad_(True), vi.requires_grad_(True)
            KV = torch.full((bl_, h_, d_, p["e"]), float("nan"), device=dev)
            DKV = torch.full((bl_, h_, d_, p["e"]), float("nan"), device=dev)
            oi = lasp_b200.lasp_fuse_parallel_fused(qi, ki, vi, s.to(dev), KV, DKV, qk_scale=c, feature_map=fmap)
            oi.backward(doi)
            torch.cuda.synchronize()
            lasp_b200.check_faults()
            heads = p["check_heads"]
            gq, gk, gv, gdo = (torch.stack([torch.cat([piece(w, bg, r)[heads] for r in range(p["sp"])], 1)
                                            for bg in rows]).to(dtype).float() for w in range(4))
            outs, grads, _ = O.sp_chain(O.preprocess_qk(gq, c, fmap), O.preprocess_qk(gk, c, fmap), gv, s[heads], gdo,
                                        p["sp"])
            mine = slice(sp_rank * nl, (sp_rank + 1) * nl)
            ref = dict(o=outs[sp_rank], dq=grads[sp_rank][0] * O.preprocess_slope(gq[:, :, mine], c, fmap),
                       dk=grads[sp_rank][1] * O.preprocess_slope(gk[:, :, mine], c, fmap), dv=grads[sp_rank][2])
            res = dict(o=oi.detach().float().cpu(), dq=qi.grad.float().cpu(), dk=ki.grad.float().cpu(),
                       dv=vi.grad.float().cpu())
            for nm, t in res.items():
                err = O.max_rel_err(t[:, heads], ref[nm])
                assert err < TOL_BF16, ("fuse_parallel_fused", nm, rank, err)
            assert engine.read_status() == 0
            dist.barrier()
            dist.destroy_process_group()
            return
        got = _run_variants(lasp, qi, ki, vi, doi, s.to(dev))
        if mode == "golden":
            g = load_golden(p["name"])
            tol = 1.5e-2 if dtype == torch.bfloat16 else TOL_FP32
            for var, res in got.items():
                ref_var = "naive" if var == "cache" else var
                for nm, t in res.items():
                    err = O.max_rel_err(t, golden_tensor(g[f"rank{rank}_{ref_var}_{nm}"]))
                    assert err < tol, (var, nm, rank, err)
        else:
            # oracle rank chain on this rank's batch slice, a few heads only (heads are independent)
            heads = p["check_heads"]
            gq, gk, gv, gdo = (torch.stack([torch.cat([piece(w, bg, r)[heads] for r in range(p["sp"])], 1)
                                            for bg in rows]).to(dtype).float() for w in range(4))
            outs, grads, _ = O.sp_chain(gq, gk, gv, s[heads], gdo, p["sp"])
            ref = dict(o=outs[sp_rank], dq=grads[sp_rank][0], dk=grads[sp_rank][1], dv=grads[sp_rank][2])
            tol = TOL_BF16 if dtype != torch.float32 else TOL_FP32
            for var, res in got.items():
                for nm, t in res.items():
                    err = O.max_rel_err(t[:, heads], ref[nm])
                    assert err < tol, (var, nm, rank, err)
        assert engine.read_status() == 0
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        import traceback
        errq.put(f"rank {rank}: {exc}\n{traceback.format_exc()}")
        raise


def _launch(world, mode, params):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    try:
        mp.spawn(_worker, args=(world, _free_port(), mode, params, errq), nprocs=world, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "worker failed")


@pytest.mark.parametrize("transport", ["nvlink", "nccl"])
@pytest.mark.parametrize("name", ["sp2_fp32", "sp4_fp32", "dp2sp2_bf16"])
def test_sequence_parallel_matches_reference_golden(name, transport):
    """transport: the library's relay kernel over peer-mapped memory, or NCCL send/recv"""
    p = dict(CASES["sp"][name], name=name, transport=transport)
    world = p["dp"] * p["sp"]
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, "golden", p)


def _sweep():
    n = _ngpu()
    return [(dp, n // dp) for dp in (1, 2, 4, 8) if n >= 2 and n % dp == 0 and dp <= n]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_dp_sp_sweep_baseline_config1(dtype):
    """The headline configuration: every DP x SP factorisation of the box; per rank b=2,
    2048 tokens, h=12, d=e=128 (bf16: tensor-core path; fp32: FFMA path)."""
    if _ngpu() < 2:
        pytest.skip("needs >= 2 GPUs")
    sweep = _sweep() if dtype == "bfloat16" else _sweep()[:1]   # fp32: the longest chain only
    for dp, sp in sweep:
        p = dict(seed=70 + dp, dp=dp, sp=sp, b=2 * dp, h=12, n=2048 * sp, d=128, e=128, slopes="baseline",
                 dtype=dtype, check_heads=[0, 6, 11])
        _launch(dp * sp, "oracle", p)


def test_reference_test_shape_on_the_whole_box():
    """The shape of the reference's own smoke test (tests/test.py:95 there): global batch 2 per GPU, global
    n = 2048 cut over the SP group, h = 12, d = 128, e = 64, unscaled N(0,1) q and k, build_slope_tensor(12),
    bf16; every DP x SP factorisation of the box."""
    if _ngpu() < 2:
        pytest.skip("needs >= 2 GPUs")
    world = _ngpu()
    for dp, sp in _sweep():
        p = dict(seed=90 + dp, dp=dp, sp=sp, b=2 * world, h=12, n=2048, d=128, e=64, slopes="alibi",
                 dtype="bfloat16", check_heads=[0, 5, 11], scale_qk=False)
        _launch(dp * sp, "oracle", p)


def test_folded_preprocessing_across_ranks():
    """lasp_fuse_parallel_fused on the whole box as one sequence-parallel group: elu(x)+1 and a scale folded into
    the kernels that also hand the rank state over (bf16, config-1 shape per rank, raw N(0,1) q and k)."""
    if _ngpu() < 2:
        pytest.skip("needs >= 2 GPUs")
    sp = _ngpu()
    p = dict(seed=60, dp=1, sp=sp, b=2, h=12, n=2048 * sp, d=128, e=128, slopes="baseline", dtype="bfloat16",
             check_heads=[0, 6, 11], scale_qk=False, fold=(128 ** -0.5, "elu1"))
    _launch(sp, "fold", p)
