"""Host-side logic on CPU: DP x SP mapping and the rank-to-rank message order
of the four sequence-parallel operators, run as gloo ranks.  The kernels are
replaced by tests/fake_engine.py (oracle arithmetic); results are compared with
the reference's own outputs stored under tests/golden/."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import lasp_oracle as O
from tests.helpers import CASES, golden_tensor, load_golden, slopes_for, split


def test_layout_matches_reference_mapping():
    from lasp_b200.utils import dp_sp_layout
    dp_groups, sp_groups = dp_sp_layout(8, 2, 4)
    assert dp_groups == [(0, 4), (1, 5), (2, 6), (3, 7)]          # README example of the reference
    assert sp_groups == [(0, 1, 2, 3), (4, 5, 6, 7)]
    assert dp_sp_layout(8, 8, 1) == ([tuple(range(8))], [(i,) for i in range(8)])
    assert dp_sp_layout(8, 1, 8) == ([(i,) for i in range(8)], [tuple(range(8))])
    with pytest.raises(RuntimeError):
        dp_sp_layout(8, 1, 3)
    with pytest.raises(RuntimeError):
        dp_sp_layout(8, 2, 2)   # dp*sp != world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, errq):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import lasp_b200._core as core
        from tests import fake_engine
        core.ENGINE = fake_engine
        import lasp
        from lasp.utils import (get_data_parallel_rank, get_data_parallel_world_size, get_seq_parallel_receive_rank,
                                get_seq_parallel_send_rank, get_sequence_parallel_rank, get_sequence_parallel_src_rank,
                                get_sequence_parallel_world_size, initialize_lasp, sequence_parallel_is_initialized,
                                get_data_parallel_group, get_data_parallel_src_rank)
        p = CASES["sp"][name]
        assert not sequence_parallel_is_initialized()
        initialize_lasp(p["dp"], p["sp"])
        assert sequence_parallel_is_initialized()
        assert get_sequence_parallel_world_size() == p["sp"] and get_data_parallel_world_size() == p["dp"]
        sp_rank, dp_rank = get_sequence_parallel_rank(), get_data_parallel_rank()
        assert (sp_rank, dp_rank) == (rank % p["sp"], rank // p["sp"])
        assert get_seq_parallel_send_rank() == (rank - 1) % world
        assert get_seq_parallel_receive_rank() == (rank + 1) % world
        assert get_sequence_parallel_src_rank() == dp_rank * p["sp"]
        assert get_data_parallel_src_rank() == sp_rank
        assert dist.get_world_size(group=get_data_parallel_group(True)) == world

        dtype = getattr(torch, p["dtype"])
        q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"])
        s = slopes_for(p["slopes"], p["h"])
        qi, ki, vi, doi = (split(t.to(dtype), p["dp"], p["sp"], dp_rank, sp_rank) for t in (q, k, v, do))
        g = load_golden(name)
        tol = 1.5e-2 if dtype == torch.bfloat16 else 2e-6
        bl, h, d, e = qi.shape[0], p["h"], p["d"], p["e"]
        for var in ("naive", "cache", "fuse", "fuse_parallel"):
            qi.grad = ki.grad = vi.grad = None
            qi.requires_grad_(True), ki.requires_grad_(True), vi.requires_grad_(True)
            KV = torch.full((bl, h, d, e), float("nan"))     # callee must not depend on the contents
            DKV = torch.full((bl, h, d, e), float("nan"))
            if var == "naive":
                oi = lasp.lasp_naive(qi, ki, vi, s)
            elif var == "cache":
                oi = lasp.lasp_cache(qi, ki, vi, s, torch.arange(qi.shape[2]).to(qi), KV, DKV)
            else:
                oi = getattr(lasp, "lasp_" + var)(qi, ki, vi, s, KV, DKV)
            oi.backward(doi)
            ref_var = "naive" if var == "cache" else var
            for nm, t in (("o", oi), ("dq", qi.grad), ("dk", ki.grad), ("dv", vi.grad)):
                ref = golden_tensor(g[f"rank{rank}_{ref_var}_{nm}"])
                err = O.max_rel_err(t.float(), ref)
                assert err < tol, (var, nm, rank, err)
            dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        import traceback
        errq.put(f"rank {rank}: {exc}\n{traceback.format_exc()}")
        raise


@pytest.mark.parametrize("name", ["sp2_fp32", "sp4_fp32", "dp2sp2_bf16"])
def test_sequence_parallel_operators_on_gloo(name):
    p = CASES["sp"][name]
    world = p["dp"] * p["sp"]
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    try:
        mp.spawn(_worker, args=(world, _free_port(), name, errq), nprocs=world, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "worker failed")


def _dead_peer_worker(rank, world, port, resq):
    import datetime
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    import lasp_b200._core as core
    from tests import fake_engine
    core.ENGINE = fake_engine
    import lasp
    from lasp.utils import initialize_lasp
    initialize_lasp(1, 2)
    q, k, v, _ = O.make_inputs(1, 1, 1, 128, 16, 16)
    s = O.baseline_slopes(1)
    if rank == 0:
        resq.put((0, "left"))          # the first rank leaves between steps and never sends its state
        return
    try:
        lasp.lasp_naive(q[:, :, 64:], k[:, :, 64:], v[:, :, 64:], s)
        resq.put((1, "no error"))
    except Exception as exc:  # noqa: BLE001
        resq.put((1, type(exc).__name__))


def test_missing_sender_is_reported_by_a_timeout_not_a_hang():
    """Failure detection on the host: the rank that should send the KV state is gone; the receiver's
    blocking receive ends with an error after the process-group timeout instead of waiting for ever."""
    ctx = mp.get_context("spawn")
    resq = ctx.SimpleQueue()
    mp.spawn(_dead_peer_worker, args=(2, _free_port(), resq), nprocs=2, join=True)
    got = dict(resq.get() for _ in range(2))
    assert got[0] == "left"
    assert got[1] != "no error", "the receive should have timed out"
