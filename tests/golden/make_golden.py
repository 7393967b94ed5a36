"""Generate the golden fixtures in this folder from the reference itself.

Run once, in a container that holds the reference checkout (read-only):

    python tests/golden/make_golden.py /path/to/LASP

The reference's arithmetic lives in Triton kernels; Triton's interpreter
(TRITON_INTERPRET=1) executes them on the CPU, where ``tl.dot`` is exact fp32.
The only harness-side shim is ``torch.cuda.device -> nullcontext`` (the
reference wraps its launches in ``with torch.cuda.device(q.device.index)``,
lasp/lightning_attention.py:414).  Sequence-parallel variants run as gloo
ranks.  Inputs come from ``oracle.lasp_oracle.make_inputs`` (numpy RandomState,
a frozen stream), so the fixtures hold outputs only plus an input checksum.

The fixtures are read by tests/test_oracle_golden.py (oracle vs reference) and
by the GPU parity tests (CUDA path vs reference).
"""
import contextlib
import json
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("OMP_NUM_THREADS", "2")

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from oracle import lasp_oracle as O  # noqa: E402

# case name -> parameters.  ``slopes``: "baseline" = 2^(-8(i+1)/h), "alibi" =
# build_slope_tensor(h), "zero" = no decay.
SINGLE_CASES = {
    "lightning_fp32_d128_e64": dict(seed=0, b=1, h=2, n=128, d=128, e=64, slopes="baseline"),
    "lightning_fp32_ragged_n100": dict(seed=1, b=1, h=2, n=100, d=64, e=64, slopes="alibi"),
    "lightning_fp32_d256_sliced": dict(seed=2, b=1, h=1, n=128, d=256, e=32, slopes="baseline"),
    "lightning_fp32_nodecay_elu": dict(seed=3, b=1, h=2, n=128, d=64, e=64, slopes="zero",
                                       feature_map="elu1", scale_qk=False),
    "lightning_fp32_3blocks_e128": dict(seed=4, b=2, h=1, n=192, d=64, e=128, slopes="baseline"),
}
# sequence-parallel cases: global tensors, split like tests/test.py:48-60 of the reference
SP_CASES = {
    "sp2_fp32": dict(seed=10, dp=1, sp=2, b=1, h=1, n=256, d=64, e=32, slopes="baseline", dtype="float32"),
    "sp4_fp32": dict(seed=11, dp=1, sp=4, b=1, h=1, n=512, d=32, e=32, slopes="alibi", dtype="float32"),
    "dp2sp2_bf16": dict(seed=12, dp=2, sp=2, b=2, h=1, n=256, d=64, e=32, slopes="baseline", dtype="bfloat16"),
}
VARIANTS = ("naive", "fuse", "fuse_parallel")  # lasp_cache reads an uninitialised buffer on CPU; skipped


def slopes_for(kind, h):
    if kind == "baseline":
        return O.baseline_slopes(h)
    if kind == "alibi":
        return O.build_slope_tensor_ref(h).to(torch.float32)
    return torch.zeros(h, 1, 1)


def input_checksum(*ts):
    return float(sum(t.double().abs().sum().item() for t in ts))


def import_reference(path):
    sys.path.insert(0, path)
    torch.cuda.device = lambda *a, **k: contextlib.nullcontext()
    import lasp  # the reference package
    return lasp


def run_single(lasp, p):
    q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"],
                                scale_qk=p.get("scale_qk", True), feature_map=p.get("feature_map"))
    s = slopes_for(p["slopes"], p["h"])
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    o = lasp.lightning_attn(q, k, v, s)
    o.backward(do)
    return dict(o=o.detach().numpy(), dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy(),
                checksum=np.float64(input_checksum(q.detach(), k.detach(), v.detach(), do)))


def split(x, dp, sp, dp_rank, sp_rank):
    # batch interleaved over dp ("(b g) -> g b"), sequence contiguous over sp
    b = x.shape[0]
    x = x.reshape(b // dp, dp, *x.shape[1:])[:, dp_rank]
    nl = x.shape[2] // sp
    return x[:, :, sp_rank * nl:(sp_rank + 1) * nl].clone()


def sp_worker(rank, world, port, ref_path, name, p, outdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lasp = import_reference(ref_path)
    from lasp.utils import initialize_lasp
    initialize_lasp(p["dp"], p["sp"])
    dtype = getattr(torch, p["dtype"])
    q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"])
    s = slopes_for(p["slopes"], p["h"])
    dp_rank, sp_rank = rank // p["sp"], rank % p["sp"]
    qi, ki, vi, doi = (split(t.to(dtype), p["dp"], p["sp"], dp_rank, sp_rank) for t in (q, k, v, do))
    res = {}
    bl, d, e, h = qi.shape[0], p["d"], p["e"], p["h"]
    for var in VARIANTS:
        qi.grad = ki.grad = vi.grad = None
        qi.requires_grad_(True), ki.requires_grad_(True), vi.requires_grad_(True)
        if var == "naive":
            oi = lasp.lasp_naive(qi, ki, vi, s)
        else:
            KV = torch.empty(bl, h, d, e, dtype=torch.float32)
            DKV = torch.empty(bl, h, d, e, dtype=torch.float32)
            oi = getattr(lasp, "lasp_" + var)(qi, ki, vi, s, KV, DKV)
        # lasp_fuse squeezes unit batch/head dims when d <= 64 (lasp/lasp_fuse.py:404);
        # same numbers, so restore the rank-4 shape in the harness
        oi = oi.reshape(doi.shape)
        oi.backward(doi)
        for nm, t in (("o", oi.detach()), ("dq", qi.grad), ("dk", ki.grad), ("dv", vi.grad)):
            t = t.float().numpy() if dtype == torch.float32 else t.view(torch.int16).numpy().view(np.uint16)
            res[f"{var}_{nm}"] = t
        dist.barrier()
    np.savez(os.path.join(outdir, f"_{name}_rank{rank}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/LASP")
    ref_path = sys.argv[1]
    lasp = import_reference(ref_path)
    meta = {"single": SINGLE_CASES, "sp": SP_CASES, "variants": VARIANTS}
    for name, p in SINGLE_CASES.items():
        np.savez(os.path.join(HERE, name + ".npz"), **run_single(lasp, p))
        print("wrote", name, flush=True)
    # slopes of the reference's build_slope_tensor for a range of head counts
    np.savez(os.path.join(HERE, "build_slope_tensor.npz"),
             **{f"h{h}": lasp.utils.build_slope_tensor(h).numpy() for h in (1, 2, 3, 4, 6, 8, 12, 16, 20, 32, 40, 64)})
    for i, (name, p) in enumerate(SP_CASES.items()):
        world = p["dp"] * p["sp"]
        mp.spawn(sp_worker, args=(world, 29610 + i, ref_path, name, p, HERE), nprocs=world, join=True)
        merged = {}
        q, k, v, do = O.make_inputs(p["seed"], p["b"], p["h"], p["n"], p["d"], p["e"])
        merged["checksum"] = np.float64(input_checksum(q, k, v, do))
        for r in range(world):
            f = os.path.join(HERE, f"_{name}_rank{r}.npz")
            with np.load(f) as z:
                for key in z.files:
                    merged[f"rank{r}_{key}"] = z[key]
            os.remove(f)
        np.savez(os.path.join(HERE, name + ".npz"), **merged)
        print("wrote", name, flush=True)
    with open(os.path.join(HERE, "cases.json"), "w") as f:
        json.dump(meta, f, indent=1)


if __name__ == "__main__":
    main()
