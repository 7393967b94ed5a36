"""Benchmark of the LASP linear-attention hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config cfg1|cfg2|cfg3|cfg4-64|...]

Headline workload (--config cfg1, the default): per rank b=2, h=12, 2048 tokens, d=e=128, bf16, seeded
synthetic N(0,1) inputs (q,k scaled by d^-0.5), slopes 2^(-8(i+1)/12).  With N GPUs the N ranks form one
sequence-parallel group (DP=1, SP=N; global sequence 2048*N) unless --dp says otherwise; per-rank work is
fixed (weak scaling).  A step is one forward + one backward of the operator.  The other configurations are
the long-sequence and no-decay shapes (one rank's share of the sequence each); they print the same line.

One JSON line is printed by rank 0:
  value  - tokens/s with inputs resident in HBM (device-timed, max over ranks); the inputs rotate over
           enough independent sets to exceed the L2;
  e2e    - tokens/s through the public operator with pinned HOST buffers: host->device copies of q,k,v,do
           and device->host copies of o,dq,dk,dv are inside the timed region;
  parity - (N > 1) max|x - ref|/max|ref| of O, dQ, dK, dV of one graph-path step and one public-operator
           step against the CPU oracle's rank chain on three heads, max over ranks; the run fails above
           the gate;
  roofline     - the kernel with the largest share of the step against the measured HBM peak;
  cpu_baseline - (N = 1) the CPU oracle (a port of the reference's arithmetic; the reference has no CPU
           implementation) on this box's host cores.

--impl reference times that CPU port alone, with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6
PARITY_GATE = 2e-2
PARITY_HEADS = 3

# name -> per-rank shape (b, h, n, d, e), slopes, scaling of q and k, feature map, description
CONFIGS = {
    "cfg1": dict(b=2, h=12, n=2048, d=128, e=128, slopes="baseline", scale_qk=True, feature_map=None,
                 text="BASELINE config 1: lightning attention fwd+bwd, b=2/rank, h=12, 2048 tokens/rank, d=e=128, "
                      "decay 2^(-8(i+1)/12)"),
    "cfg2": dict(b=1, h=16, n=16384, d=128, e=128, slopes="baseline", scale_qk=True, feature_map=None,
                 text="BASELINE config 2 (TNL-1B layer, b=1, h=16, d=e=128): one rank's 16384 tokens of the "
                      "131072-token sequence at SP=8"),
    "cfg2-sp1": dict(b=1, h=16, n=131072, d=128, e=128, slopes="baseline", scale_qk=True, feature_map=None,
                     text="BASELINE config 2 (TNL-1B layer, b=1, h=16, d=e=128): the whole 131072-token sequence "
                          "on one rank (SP=1)"),
    "cfg3": dict(b=1, h=32, n=65536, d=128, e=128, slopes="baseline", scale_qk=True, feature_map=None,
                 text="BASELINE config 3 (TNL-7B layer, b=1, h=32, d=e=128): one rank's 65536 tokens of the "
                      "524288-token sequence at SP=8"),
    "cfg4-64": dict(b=4, h=16, n=4096, d=64, e=64, slopes="zero", scale_qk=False, feature_map="elu1",
                    text="BASELINE config 4 (no decay, elu(x)+1 on q,k, b=4, h=16), d=e=64: one rank's 4096 tokens "
                         "of the 32768-token sequence at SP=8"),
    "cfg4-128": dict(b=4, h=16, n=4096, d=128, e=128, slopes="zero", scale_qk=False, feature_map="elu1",
                     text="BASELINE config 4 (no decay, elu(x)+1 on q,k, b=4, h=16), d=e=128: one rank's 4096 "
                          "tokens of the 32768-token sequence at SP=8"),
    "cfg4-256": dict(b=4, h=16, n=4096, d=256, e=256, slopes="zero", scale_qk=False, feature_map="elu1",
                     text="BASELINE config 4 (no decay, elu(x)+1 on q,k, b=4, h=16), d=e=256 (128-wide slices of "
                          "both head dimensions): one rank's 4096 tokens of the 32768-token sequence at SP=8"),
}


def env_int(name, default):
    return int(os.environ.get(name, default))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops_sustained"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, 1400.0, "fallback"


def profiled_traffic(kernel: str):
    """dram bytes per launch of `kernel` at the headline configuration, from the ncu capture summarised in
    profiles/dram_traffic_cfg1.json (None when no capture of that kernel is recorded)."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic_cfg1.json")) as f:
            rec = json.load(f)["kernels"].get(kernel)
        return None if rec is None else float(rec["dram_bytes_read"]) + float(rec["dram_bytes_written"])
    except Exception:  # noqa: BLE001
        return None


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.06)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def slopes_for(cfg):
    h = cfg["h"]
    if cfg["slopes"] == "zero":
        return torch.zeros(h, 1, 1)
    i = torch.arange(1, h + 1, dtype=torch.float64)
    return torch.pow(2.0, -8.0 * i / h).float().reshape(h, 1, 1)


def feature(t, cfg):
    return torch.nn.functional.elu(t) + 1.0 if cfg["feature_map"] == "elu1" else t


def qk_preprocessing(cfg):
    """(scale, feature map) that the configuration puts in front of the operator"""
    return (cfg["d"] ** -0.5 if cfg["scale_qk"] else 1.0), cfg["feature_map"]


def make_set(cfg, seed, device, dtype, pinned=False, raw=False):
    """raw: q and k as drawn, for the legs that time the preprocessing too (--qk folded | torch)"""
    b, h, n, d, e = (cfg[x] for x in "bhnde")
    g = torch.Generator().manual_seed(seed)
    scale = d ** -0.5 if cfg["scale_qk"] else 1.0
    q = torch.randn(b, h, n, d, generator=g)
    k = torch.randn(b, h, n, d, generator=g)
    if not raw:
        q, k = feature(q, cfg) * scale, feature(k, cfg) * scale
    v = torch.randn(b, h, n, e, generator=g)
    do = torch.randn(b, h, n, e, generator=g)
    ts = [t.to(dtype) for t in (q, k, v, do)]
    if pinned:
        return [t.pin_memory() for t in ts]
    return [t.to(device) for t in ts]


def parity_piece(cfg, which, b_global, chunk, heads=None):
    """The global tensors of the parity check are defined piecewise - one seeded draw per (tensor, global
    batch row, rank chunk) - so that a rank generates its own chunk plus, for the oracle, the checked
    heads of every chunk; no rank ever builds a global tensor."""
    g = torch.Generator().manual_seed(((7 * 4 + which) * 4096 + b_global) * 64 + chunk)
    width = cfg["d"] if which < 2 else cfg["e"]
    t = torch.randn(cfg["h"], cfg["n"], width, generator=g)
    if which < 2:
        t = feature(t, cfg) * (cfg["d"] ** -0.5 if cfg["scale_qk"] else 1.0)
    return t if heads is None else t[heads]


# ---------------------------------------------------------------------------
# reference arm / cpu baseline: the oracle on the host cores
# ---------------------------------------------------------------------------
def cpu_port_tokens_per_s(cfg, reps, warm=1):
    from oracle import lasp_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    b, h, d, e = cfg["b"], cfg["h"], cfg["d"], cfg["e"]
    n = min(cfg["n"], 2048)                      # a bounded sample: at most 2048 tokens of the rank's chunk
    q, k, v, do = O.make_inputs(0, b, h, n, d, e, scale_qk=cfg["scale_qk"], feature_map=cfg["feature_map"])
    s = slopes_for(cfg)
    for _ in range(warm):
        O.fwd_bwd(q, k, v, s, do)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        O.fwd_bwd(q, k, v, s, do)
        times.append(time.perf_counter() - t0)
    sample = (f"{reps} runs of b={b}, h={h}, {n} tokens, d={d}, e={e} in fp32 (blocked B=64 torch port of the "
              f"reference's kernels, {torch.get_num_threads()} threads), median")
    return b * n / statistics.median(times), torch.get_num_threads(), times, sample


def run_reference(args, cfg):
    if env_int("RANK", 0) != 0:
        return
    value, cores, times, sample = cpu_port_tokens_per_s(cfg, args.steps, max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": metric_name(cfg), "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.median(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["text"] + " - on the host cores", "b": cfg["b"], "h": cfg["h"],
                   "n": min(cfg["n"], 2048), "d": cfg["d"], "e": cfg["e"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def run_reference_triton(args, cfg):
    """Informational, never the reference arm: the reference's own Triton kernels (lightning_attn, single
    device) from the unmodified install under baseline/_ref, JIT-compiled for this GPU by the installed Triton,
    on the same shape, dtype, steps and warm-up.  Prints `unavailable` with the reason when that cannot run."""
    if env_int("RANK", 0) != 0:
        return
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference-triton", "metric": metric_name(cfg), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": cfg["text"] + " - lightning_attn of the reference on one GPU"}}
    try:
        if not os.path.isdir(os.path.join(ref_dir, "lasp")):
            raise RuntimeError("baseline/_ref holds no install of the reference")
        sys.path[:] = [ref_dir] + [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
        for name in [m for m in sys.modules if m == "lasp" or m.startswith("lasp.")]:
            del sys.modules[name]
        import lasp as ref_lasp
        if not os.path.abspath(ref_lasp.__file__).startswith(ref_dir):
            raise RuntimeError(f"imported {ref_lasp.__file__}, not the install under baseline/_ref")
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        q, k, v, do = make_set(cfg, 1000, device, torch.bfloat16)
        s = slopes_for(cfg).to(device)
        for t in (q, k, v):
            t.requires_grad_(True)

        def step():
            q.grad = k.grad = v.grad = None
            ref_lasp.lightning_attn(q, k, v, s).backward(do)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
        line.update(value=cfg["b"] * cfg["n"] / (ms * 1e-3), ms_per_step=ms, higher_is_better=True)
    except BaseException as exc:  # noqa: BLE001  (a Triton compile error must become the line, not a crash)
        line["unavailable"] = f"{type(exc).__name__}: {str(exc).splitlines()[0] if str(exc) else ''}"[:300]
    emit(line)


def metric_name(cfg):
    return (f"fwd+bwd tokens/s, LASP linear attention (b={cfg['b']}/rank, h={cfg['h']}, {cfg['n']} tokens/rank, "
            f"d={cfg['d']}, e={cfg['e']})")


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def bind_to_gpu_numa_node(index):
    """Restricts this process to the CPUs next to GPU `index` (sysfs local_cpulist of its PCI function), so that
    the pinned host buffers allocated afterwards are first touched on that node and the copies do not cross the
    socket interconnect.  Returns the NUMA node, or None when the topology cannot be read."""
    try:
        pr = torch.cuda.get_device_properties(index)
        dev = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(dev + "/local_cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
        with open(dev + "/numa_node") as f:
            return int(f.read().strip())
    except Exception:  # noqa: BLE001
        return None


def run_kernels_only(args, cfg):
    """What a profiler run wants: the launches of W + K steps on rotating input sets, nothing around them."""
    from lasp_b200 import engine
    from lasp_b200.pipeline import FixedStep
    b, h, n, d, e = (cfg[x] for x in "bhnde")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    s = slopes_for(cfg).to(device)
    set_bytes = (2 * d + 2 * e) * 2 * b * h * n
    n_sets = max(2, min(6, int(L2_BYTES * 1.6 // set_bytes) + 1))
    steps = [FixedStep(*make_set(cfg, 1000 + i, device, torch.bfloat16), s) for i in range(n_sets)]
    for i in range(args.warmup + args.steps):
        steps[i % n_sets].run()
    torch.cuda.synchronize()
    emit({"kernels_only": True, "steps": args.steps, "warmup": args.warmup, "launches_per_step":
                      steps[0].launches, "config": args.config, "kernel_faults": engine.read_status()})


def run_ours(args, cfg):
    import torch.distributed as dist
    import lasp_b200
    from lasp_b200 import engine, lasp_fuse_parallel, lightning_attn
    from lasp_b200.utils import initialize_lasp

    b, h, n, d, e = (cfg[x] for x in "bhnde")
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    numa_node = bind_to_gpu_numa_node(local) if world > 1 else None    # before any pinned allocation
    torch.set_num_threads(max(1, min(len(os.sched_getaffinity(0)), (os.cpu_count() or 8) // world)))
    dp = args.dp
    sp = world // dp
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        initialize_lasp(dp, sp)
    dtype = torch.bfloat16
    s = slopes_for(cfg).to(device)
    wide = d > 128 or e > 128                  # head dimensions cut in 128-wide slices by the operator

    # enough independent input sets that a step never finds its inputs in L2
    set_bytes = (2 * d + 2 * e) * 2 * b * h * n
    n_sets = max(2, min(6, int(L2_BYTES * 1.6 // set_bytes) + 1))
    raw_qk = args.qk != "premapped"
    qk_scale, qk_map = qk_preprocessing(cfg) if raw_qk else (1.0, None)
    sets = [make_set(cfg, 1000 * rank + i, device, dtype, raw=raw_qk) for i in range(n_sets)]
    for st in sets:
        for t in st[:3]:
            t.requires_grad_(True)
    KV = torch.empty(b, h, d, e, device=device)
    DKV = torch.empty(b, h, d, e, device=device)

    def operator(q, k, v):
        if args.qk == "folded":      # the kernels preprocess q and k themselves
            if sp > 1:
                return lasp_b200.lasp_fuse_parallel_fused(q, k, v, s, KV, DKV, qk_scale=qk_scale, feature_map=qk_map)
            return lasp_b200.lightning_attn_fused(q, k, v, s, qk_scale=qk_scale, feature_map=qk_map)
        if args.qk == "torch":       # the caller preprocesses them, inside the timed region
            from lasp_b200._core import preprocess_qk
            q, k = preprocess_qk(q, qk_scale, qk_map), preprocess_qk(k, qk_scale, qk_map)
        return lasp_fuse_parallel(q, k, v, s, KV, DKV) if sp > 1 else lightning_attn(q, k, v, s)

    plan = None if wide else engine.make_plan(b, h, n, d, e, dtype)
    graphs = []
    graph_note = "eager operator calls"
    group = None
    if world > 1:
        from lasp_b200.utils import get_sequence_parallel_group
        group = get_sequence_parallel_group()
    if not args.eager and not wide and args.qk != "torch":
        # the launches of a step go through the C ABI and are replayed from a CUDA graph, one per input set
        from lasp_b200.pipeline import FixedStep
        side = torch.cuda.Stream()
        try:
            fixed_steps = [FixedStep(q.detach(), k.detach(), v.detach(), do, s, group, qk_scale=qk_scale,
                                     feature_map=qk_map) for q, k, v, do in sets]
            usable = 1
        except Exception as exc:  # noqa: BLE001  (no peer-mapped exchange here: time the eager NCCL path)
            graph_note = f"eager operator calls ({type(exc).__name__}: {exc})"[:200]
            fixed_steps, usable = [], 0
        flag = torch.tensor([usable], device=device)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)      # all ranks take the same route
        for fixed in (fixed_steps if flag.item() else []):
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fixed.run()
            torch.cuda.current_stream().wait_stream(side)
            if world > 1:
                torch.cuda.synchronize()
                dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fixed.run()
            graphs.append((g, fixed))

    # ---- parity before anything is timed (N > 1): graph path and public operator against the oracle chain
    parity = None
    if world > 1 and args.qk == "premapped":
        from oracle import lasp_oracle as O
        from lasp_b200.pipeline import FixedStep
        dp_rank, sp_rank = rank // sp, rank % sp
        rows = [i * dp + dp_rank for i in range(b)]                      # batch interleaved over dp
        mine = [torch.stack([parity_piece(cfg, w, bg, sp_rank) for bg in rows]).to(dtype).to(device) for w in range(4)]
        heads = sorted({0, h // 2, h - 1})[:PARITY_HEADS]
        glob = [torch.stack([torch.cat([parity_piece(cfg, w, bg, r, heads) for r in range(sp)], 1) for bg in rows])
                .to(dtype).float() for w in range(4)]
        outs, grads, _ = O.sp_chain(glob[0], glob[1], glob[2], slopes_for(cfg)[heads], glob[3], sp)
        ref = dict(o=outs[sp_rank], dq=grads[sp_rank][0], dk=grads[sp_rank][1], dv=grads[sp_rank][2])
        errs = {}

        def record(tag, o, dq, dk, dv):
            for name, t in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                errs[name] = max(errs.get(name, 0.0), O.max_rel_err(t[:, heads].float().cpu(), ref[name]))

        if graphs:
            step0 = FixedStep(mine[0], mine[1], mine[2], mine[3], s, group)
            step0.run()
            torch.cuda.synchronize()
            record("graph path", *step0.outputs)
        qp, kp, vp = (t.clone().requires_grad_(True) for t in mine[:3])
        op = operator(qp, kp, vp)
        op.backward(mine[3])
        torch.cuda.synchronize()
        record("operator", op.detach(), qp.grad, kp.grad, vp.grad)
        lasp_b200.check_faults()
        worst = torch.tensor([errs[k] for k in ("o", "dq", "dk", "dv")], device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        parity = {k: float(x) for k, x in zip(("o", "dq", "dk", "dv"), worst.tolist())}
        parity.update(gate=PARITY_GATE, heads=heads, reference="CPU oracle rank chain (fp32) on the bf16-rounded inputs",
                      paths=["graph of C-ABI launches", "lasp_fuse_parallel"] if graphs else ["lasp_fuse_parallel"])
        if max(worst.tolist()) > PARITY_GATE or any(x != x for x in worst.tolist()):
            if rank == 0:
                emit({"error": "parity gate exceeded", "parity": parity})
            raise SystemExit(3)

    def step(i):
        if graphs:
            graphs[i % n_sets][0].replay()
            return
        q, k, v, do = sets[i % n_sets]
        q.grad = k.grad = v.grad = None
        operator(q, k, v).backward(do)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    sync_all()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tokens_per_step = b * dp * n * sp
    with ClockSampler(local) as clocks:
        sync_all()
        start.record()
        for i in range(args.steps):
            step(args.warmup + i)
        stop.record()
        sync_all()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms_per_step = ms.item() / args.steps
        # The timed region can be too short for nvidia-smi to sample.  Keep the same steps running for about a
        # second under the sampler: its clocks and throttle reasons are those of this load, and the longer
        # window gives a sustained figure next to the timed one (the one to trust when they differ).
        extra = int(min(20000, max(args.steps, 1000.0 / max(ms_per_step, 1e-3))))
        t2 = torch.tensor([extra], device=device)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MIN)
        extra = int(t2.item())
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for i in range(extra):
            step(i)
        e2.record()
        sync_all()
        ms_sus = torch.tensor([s2.elapsed_time(e2)], device=device)
        if world > 1:
            dist.all_reduce(ms_sus, op=dist.ReduceOp.MAX)
    value = tokens_per_step / (ms_per_step * 1e-3)
    sustained = {"value": tokens_per_step / (ms_sus.item() / extra * 1e-3), "unit": UNIT, "steps": extra,
                 "ms_per_step": ms_sus.item() / extra}

    # ---- end to end through the public operator with host buffers ---------
    host_in = make_set(cfg, 5000 + rank, device, dtype, pinned=True, raw=raw_qk)
    host_out = [torch.empty_like(t).pin_memory() for t in host_in]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def e2e_step():
        q, k, v, do = (t.to(device, non_blocking=True) for t in host_in)
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        o = operator(q, k, v)
        o.backward(do)
        for dst, src in zip(host_out, (o.detach(), q.grad, k.grad, v.grad)):
            dst.copy_(src, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 20))

    def timed(fn_loop):
        sync_all()
        start.record()
        fn_loop()
        stop.record()
        sync_all()
        t = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return tokens_per_step / (t.item() / e2e_steps * 1e-3)

    for _ in range(3):
        e2e_step()
    e2e_serial = timed(lambda: [e2e_step() for _ in range(e2e_steps)])

    def e2e_pipelined_loop():
        """Same work per step, but the copy-in of step i+1 and the copy-out of step i-1 run on their own
        streams next to the compute of step i (two device input buffers; PCIe is full duplex)."""
        cur = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        dev_in = [[torch.empty(t.shape, dtype=t.dtype, device=device) for t in host_in] for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        keep = [None, None]
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        for i in range(e2e_steps):
            j = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(in_free[j])        # step i-2 has finished with buffer set j
                for dst, src in zip(dev_in[j], host_in):
                    dst.copy_(src, non_blocking=True)
                in_ready[j].record(s_in)
            cur.wait_event(in_ready[j])
            q, k, v = (t.detach().requires_grad_(True) for t in dev_in[j][:3])
            o = operator(q, k, v)
            o.backward(dev_in[j][3])
            in_free[j].record(cur)
            outs = (o.detach(), q.grad, k.grad, v.grad)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(host_out, outs):
                    src.record_stream(s_out)           # the allocator must not reuse it before the copy-out ran
                    dst.copy_(src, non_blocking=True)
            keep[j] = outs
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)

    e2e_modes = {"serial (copy in, compute, copy out)": e2e_serial}
    try:
        e2e_pipelined_loop()                           # warm-up of the streams and buffers
        e2e_modes["copies overlapped with compute on side streams"] = timed(e2e_pipelined_loop)
    except Exception as exc:  # noqa: BLE001  (keep the serial number)
        e2e_modes[f"pipelined variant failed: {type(exc).__name__}"] = 0.0
    e2e_mode = max(e2e_modes, key=e2e_modes.get)
    e2e_value = e2e_modes[e2e_mode]

    # ---- the kernels of a step one by one: which dominates, and its roofline ----
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    kernels, roofline = None, None
    if not wide and plan.path_name == "tensor":
        fws, bws = [], []
        for q, k, v, do in sets:
            fw = engine.Forward(plan, q.detach(), k.detach(), v.detach(), s)
            fw.run()
            bw = engine.Backward(plan, q.detach(), k.detach(), v.detach(), do, s, fw.ws)
            bw.run()
            fws.append(fw), bws.append(bw)
        torch.cuda.synchronize()
        reps = 8 * n_sets

        def launch_us(fn):
            """average device time of one launch: a graph of back-to-back launches rotating over the input sets"""
            kg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(kg):
                for i in range(reps):
                    fn(i % n_sets)
            kg.replay()
            torch.cuda.synchronize()
            start.record()
            kg.replay()
            stop.record()
            torch.cuda.synchronize()
            return 1e3 * start.elapsed_time(stop) / reps

        per_token_head = {   # algorithmic bytes per token and head: every tensor of the launch touched once
            "k_walk_out<fused> (forward: q,k,v -> o)": ((2 * d + 2 * e) * 2, lambda i: fws[i].run()),
            "k_walk_out<dq> (do,v,k -> dq)": ((2 * d + 2 * e) * 2, lambda i: bws[i].dq_only()),
            "k_walk_dkv<fused> (q,k,v,do -> dk,dv)": ((3 * d + 3 * e) * 2, lambda i: bws[i].dkv_only()),
        }
        kernels = {}
        for name, (bytes_per, fn) in per_token_head.items():
            us = launch_us(fn)
            kernels[name] = {"us_per_launch": us, "algorithmic_bytes": bytes_per * b * h * n,
                             "achieved_gbs": bytes_per * b * h * n / (us * 1e-6) / 1e9}
        top = max(kernels, key=lambda k_: kernels[k_]["us_per_launch"])
        step_bytes = (6 * d + 5 * e) * 2 * b * h * n
        step_flops = (2 * 64 * (4 * d + 3 * e) + 12 * d * e) * b * h * n
        traffic = profiled_traffic(top.split(" ")[0]) if args.config == "cfg1" else None
        roofline = {"bound": "hbm", "kernel": top, "achieved": kernels[top]["achieved_gbs"], "peak": hbm_peak,
                    "unit": "GB/s", "frac": kernels[top]["achieved_gbs"] / hbm_peak, "peak_source": peak_kind,
                    "traffic": traffic, "traffic_source": "profiles/dram_traffic_cfg1.json" if traffic else None,
                    "kernel_us": kernels[top]["us_per_launch"],
                    "algorithmic_bytes_per_launch": kernels[top]["algorithmic_bytes"],
                    "step_hbm_frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
                    "step_tensor_frac": step_flops / (ms_per_step * 1e-3) / 1e12 / tensor_peak}

    fault_t = torch.tensor([engine.read_status(clear=False)], device=device)
    if world > 1:
        dist.all_reduce(fault_t, op=dist.ReduceOp.MAX)
    fault_word = int(fault_t.item())     # 0 = no bounded wait ran out on any rank
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    launches = graphs[0][1].launches if graphs else (3 if not wide else 3 * ((d + 127) // 128) * ((e + 127) // 128))
    line = {
        "metric": metric_name(cfg), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["text"], "name": args.config, "qk_preprocessing": args.qk,
                   "parallelism": f"dp{dp}xsp{sp}",
                   "global_batch": b * dp, "global_seq_len": n * sp,
                   "kernel_path": "tensor (128-wide slices)" if wide else plan.path_name,
                   "launch": f"cuda graph of the {graphs[0][1].launches} C-ABI launches of a step" if graphs
                   else graph_note,
                   "transport": ("nvlink hand-over kernel" if graphs else "nccl or nvlink (operator default)")
                   if world > 1 else "none",
                   "l2": f"inputs rotate over {n_sets} independent sets ({n_sets * set_bytes / 1e6:.0f} MB) > L2"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "mode": e2e_mode, "serial_value": e2e_serial,
                "pcie_gbs_per_rank": (h2d + d2h) * e2e_value / tokens_per_step / 1e9,
                "host_numa_node_of_rank0": numa_node},
        "gpu_launches": launches * args.steps,
        "kernel_faults": fault_word,
        "clocks": clocks.summary(), "sustained": sustained,
    }
    if roofline is not None:
        line["roofline"] = roofline
        line["kernels"] = kernels
    if parity is not None:
        line["parity"] = parity
    if world == 1:
        cpu_value, cores, _, sample = cpu_port_tokens_per_s(cfg, 3)
        line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries print to stdout too (NCCL its version, for one): everything but the result line goes to stderr."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text)


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--config", default="cfg1", choices=sorted(CONFIGS))
    ap.add_argument("--dp", type=int, default=1, help="data-parallel size; sequence-parallel size = gpus / dp")
    ap.add_argument("--eager", action="store_true", help="time the public operator launch by launch (no CUDA graph)")
    ap.add_argument("--qk", default="premapped", choices=["premapped", "folded", "torch"],
                    help="where the configuration's preprocessing of q and k (1/sqrt(d), elu(x)+1) happens: before the "
                         "timed region (as BASELINE words it), inside the kernels, or as torch operations of the caller "
                         "inside the timed region")
    ap.add_argument("--kernels-only", action="store_true",
                    help="W + K steps of the C-ABI launches on one GPU and nothing else (the target of profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    cfg = CONFIGS[args.config]
    if args.impl == "reference":
        run_reference(args, cfg)
    elif args.impl == "reference-triton":
        run_reference_triton(args, cfg)
    elif args.kernels_only:
        run_kernels_only(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
