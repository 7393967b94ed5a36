"""Benchmark of the LASP linear-attention hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the headline configuration): per rank b=2, h=12, 2048 tokens, d=e=128, bf16,
seeded synthetic N(0,1) inputs (q,k scaled by d^-0.5), slopes 2^(-8(i+1)/12).
With N GPUs the N ranks form one sequence-parallel group (DP=1, SP=N; global
sequence 2048*N) unless --dp says otherwise; per-rank work is fixed (weak
scaling).  A step is one forward + one backward of the operator.

One JSON line is printed by rank 0:
  value  - tokens/s with inputs resident in HBM (device-timed, max over ranks);
           the inputs rotate over enough independent sets to exceed the L2;
  e2e    - tokens/s through the public operator with pinned HOST buffers:
           host->device copies of q,k,v,do and device->host copies of
           o,dq,dk,dv are inside the timed region;
  roofline     - the dominant kernel (backward gradients) against measured HBM peak;
  cpu_baseline - the CPU oracle (a port of the reference's arithmetic; the
           reference has no CPU implementation) on this box's host cores.

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

# headline configuration, per rank
B, H, N_LOCAL, D, E = 2, 12, 2048, 128, 128
METRIC = "fwd+bwd tokens/s, LASP linear attention (b=2/rank, h=12, 2048 tokens/rank, d=e=128)"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (backward gradients) on this
# workload, from one ncu capture: 75.7 MB read (q,k,v,do and the two state tensors) + 5.6 MB written back by
# kernel end (most of dq,dk,dv still sits in L2)
DOMINANT_KERNEL_TRAFFIC_BYTES = 81.3e6


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


def slopes(h):
    i = torch.arange(1, h + 1, dtype=torch.float64)
    return torch.pow(2.0, -8.0 * i / h).float().reshape(h, 1, 1)


def make_set(seed, device, dtype, pinned=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, N_LOCAL, D, generator=g) * D ** -0.5
    k = torch.randn(B, H, N_LOCAL, D, generator=g) * D ** -0.5
    v = torch.randn(B, H, N_LOCAL, E, generator=g)
    do = torch.randn(B, H, N_LOCAL, E, generator=g)
    ts = [t.to(dtype) for t in (q, k, v, do)]
    if pinned:
        return [t.pin_memory() for t in ts]
    return [t.to(device) for t in ts]


# ---------------------------------------------------------------------------
# reference arm / cpu baseline: the oracle on the host cores
# ---------------------------------------------------------------------------
def cpu_port_tokens_per_s(reps, warm=1):
    from oracle import lasp_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, do = O.make_inputs(0, B, H, N_LOCAL, D, E)
    s = O.baseline_slopes(H)
    for _ in range(warm):
        O.fwd_bwd(q, k, v, s, do)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        O.fwd_bwd(q, k, v, s, do)
        times.append(time.perf_counter() - t0)
    return B * N_LOCAL / statistics.median(times), torch.get_num_threads(), times


def run_reference(args):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    value, cores, times = cpu_port_tokens_per_s(args.steps, max(1, min(args.warmup, 2)))
    sample = (f"each step = one rank's chunk (b={B},h={H},n={N_LOCAL},d=e={D}) in fp32, blocked (B=64) torch port "
              f"of the reference's kernels; {args.steps} steps, median")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.median(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BASELINE config 1 per-rank chunk on CPU", "b": B, "h": H, "n": N_LOCAL, "d": D,
                   "e": E},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from lasp_b200 import engine, lasp_fuse_parallel, lightning_attn
    from lasp_b200.utils import initialize_lasp

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dp = args.dp
    sp = world // dp
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        initialize_lasp(dp, sp)
    dtype = torch.bfloat16
    s = slopes(H).to(device)

    # enough independent input sets that a step never finds its inputs in L2
    set_bytes = (2 * D + 2 * E) * 2 * B * H * N_LOCAL
    n_sets = max(2, int(L2_BYTES * 1.6 // set_bytes) + 1)
    sets = [make_set(1000 * rank + i, device, dtype) for i in range(n_sets)]
    for st in sets:
        for t in st[:3]:
            t.requires_grad_(True)
    KV = torch.empty(B, H, D, E, device=device)
    DKV = torch.empty(B, H, D, E, device=device)

    plan = engine.make_plan(B, H, N_LOCAL, D, E, dtype)
    graphs = []
    graph_note = "eager operator calls"
    if not args.eager:
        # the launches of a step (6 kernels; 10 with the two state totals and the two
        # state exchanges of a sequence-parallel rank) go through the C ABI and are replayed
        # from a CUDA graph, one graph per input set
        from lasp_b200.pipeline import FixedStep
        from lasp_b200.utils import get_sequence_parallel_group
        group = get_sequence_parallel_group() if world > 1 else None
        side = torch.cuda.Stream()
        try:
            fixed_steps = [FixedStep(q.detach(), k.detach(), v.detach(), do, s, group) for q, k, v, do in sets]
            usable = 1
        except Exception as exc:  # noqa: BLE001  (no peer-mapped exchange here: time the eager NCCL path)
            graph_note = f"eager operator calls ({type(exc).__name__}: {exc})"[:200]
            fixed_steps, usable = [], 0
        if usable and world > 1:
            # self-check of the exchange before anything is timed: one eager step; a bounded wait that ran out
            # (fault word != 0 on any rank) sends every rank down the NCCL route instead
            fixed_steps[0].run()
            torch.cuda.synchronize()
            if engine.read_status(clear=True) != 0:
                usable = 0
                graph_note = "eager operator calls over NCCL (the exchange self-check reported a fault)"
        flag = torch.tensor([usable], device=device)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)      # all ranks take the same route
        if world > 1 and not flag.item():
            from lasp_b200 import comm
            comm._relay_unavailable = True                   # the operators now use NCCL send/recv
            if usable:
                graph_note = "eager operator calls over NCCL (the exchange self-check failed on another rank)"
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

    def step(i):
        if graphs:
            graphs[i % n_sets][0].replay()
            return
        q, k, v, do = sets[i % n_sets]
        q.grad = k.grad = v.grad = None
        if sp > 1:
            o = lasp_fuse_parallel(q, k, v, s, KV, DKV)
        else:
            o = lightning_attn(q, k, v, s)
        o.backward(do)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    sync_all()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tokens_per_step = B * dp * N_LOCAL * sp
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
        # The timed region lasts a few milliseconds, too short for nvidia-smi to sample.  Keep the same
        # steps running for about a second under the sampler: its clocks and throttle reasons are those of
        # this load, and the longer window gives a sustained figure next to the timed one.
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
    host_in = make_set(5000 + rank, device, dtype, pinned=True)
    host_out = [torch.empty_like(t).pin_memory() for t in host_in]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def e2e_step():
        q, k, v, do = (t.to(device, non_blocking=True) for t in host_in)
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        o = lasp_fuse_parallel(q, k, v, s, KV, DKV) if sp > 1 else lightning_attn(q, k, v, s)
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
            o = lasp_fuse_parallel(q, k, v, s, KV, DKV) if sp > 1 else lightning_attn(q, k, v, s)
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

    e2e_mode = "serial (copy in, compute, copy out)"
    e2e_value = e2e_serial
    try:
        e2e_pipelined_loop()                           # warm-up of the streams and buffers
        piped = timed(e2e_pipelined_loop)
        if piped > e2e_value:
            e2e_value, e2e_mode = piped, "copies overlapped with compute on side streams"
    except Exception as exc:  # noqa: BLE001  (keep the serial number)
        e2e_mode += f"; pipelined variant failed: {type(exc).__name__}"

    # ---- dominant kernel alone: backward gradients --------------------------
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    fws, bws = [], []
    for q, k, v, do in sets:
        fw = engine.Forward(plan, q.detach(), k.detach(), v.detach(), s)
        fw.run()
        bw = engine.Backward(plan, q.detach(), k.detach(), v.detach(), do, s, fw.ws)
        bw.chunk_states(), bw.scan()
        fws.append(fw), bws.append(bw)
    for bw in bws:
        bw.grads()
    torch.cuda.synchronize()
    reps = 8 * n_sets

    def launch_ms(fn):
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
        return start.elapsed_time(stop) / reps

    kernel_ms = launch_ms(lambda i: bws[i].grads())
    phases = None
    if args.phases:
        phases = {name: 1e3 * launch_ms(fn) for name, fn in (
            ("fwd_chunk_states_us", lambda i: fws[i].chunk_states()), ("fwd_scan_us", lambda i: fws[i].scan()),
            ("fwd_output_us", lambda i: fws[i].output()), ("bwd_chunk_states_us", lambda i: bws[i].chunk_states()),
            ("bwd_scan_us", lambda i: bws[i].scan()), ("bwd_grads_us", lambda i: bws[i].grads()))}
    kernel_bytes = (4 * D + 3 * E) * 2 * B * H * N_LOCAL      # reads q,k,v,do; writes dq,dk,dv
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    step_bytes = (6 * D + 5 * E) * 2 * B * H * N_LOCAL
    step_flops = (2 * 64 * (4 * D + 3 * E) + 12 * D * E) * B * H * N_LOCAL

    fault_t = torch.tensor([engine.read_status(clear=False)], device=device)
    if world > 1:
        dist.all_reduce(fault_t, op=dist.ReduceOp.MAX)
    fault_word = int(fault_t.item())     # 0 = no bounded wait ran out on any rank
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    cpu_value, cores, _ = cpu_port_tokens_per_s(3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "BASELINE config 1: lightning attention fwd+bwd, b=2/rank, h=12, 2048 tokens/rank, "
                               "d=e=128, decay 2^(-8(i+1)/12)", "parallelism": f"dp{dp}xsp{sp}",
                   "global_batch": B * dp, "global_seq_len": N_LOCAL * sp, "kernel_path": plan.path_name,
                   "launch": f"cuda graph of the {graphs[0][1].launches} C-ABI launches" if graphs
                   else graph_note,
                   "transport": ("nvlink exchange kernel" if graphs else "nccl or nvlink (operator default)")
                   if world > 1 else "none",
                   "l2": f"inputs rotate over {n_sets} independent sets ({n_sets * set_bytes / 1e6:.0f} MB) > L2"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "mode": e2e_mode, "serial_value": e2e_serial},
        "gpu_launches": (graphs[0][1].launches if graphs else 6) * args.steps,
        "kernel_faults": fault_word,
        "clocks": clocks.summary(), "sustained": sustained,
        "roofline": {"bound": "hbm", "kernel": f"bwd_grads ({plan.path_name})", "achieved": achieved,
                     "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_kind,
                     "traffic": DOMINANT_KERNEL_TRAFFIC_BYTES, "kernel_ms": kernel_ms,
                     "algorithmic_bytes_per_launch": kernel_bytes,
                     "step_hbm_frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
                     "step_tensor_frac": step_flops / (ms_per_step * 1e-3) / 1e12 / tensor_peak},
        "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"3 runs of one rank's chunk (b={B},h={H},n={N_LOCAL},d=e={D}) fp32, median"},
    }
    print(json.dumps(line), flush=True)
    if phases is not None:
        print(json.dumps({"phases": phases, "note": "device time per launch of each of the six kernels, L2-cold"}),
              flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dp", type=int, default=1, help="data-parallel size; sequence-parallel size = gpus / dp")
    ap.add_argument("--eager", action="store_true", help="time the public operator launch by launch (no CUDA graph)")
    ap.add_argument("--phases", action="store_true", help="also print a second JSON line with the time of each kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
