#!/usr/bin/env python
"""Benchmark of the bytecode-interpreter hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--programs all|none]

Headline workload: the conductor-lowered RMSNorm bytecode program over x fp32 [16384, 4096] (the configuration the
metric is quoted on), one "step" = one pass of the program over the whole batch. With N > 1 (launched by torchrun, one
process per GPU) the batch is N times as large and sharded by rows: every rank runs its own 16384-row shard (weak scaling),
with no data-path collective, and the reported value is all ranks' bytes divided by the slowest rank's device time.

Prints ONE JSON line. `value` is achieved HBM GB/s = algorithmic bytes / device time with inputs resident in HBM;
`e2e` is the same metric through the public executor API with HOST buffers (pinned host -> device copy of the inputs and
device -> host copy of the result inside the timed region). `roofline` relates the kernel to the measured copy bandwidth,
`cpu_baseline` times the reference's CPU path (torch eager, the oracle its tests use) on a bounded sample of the same
workload, and `programs` carries the other named programs for context.

--impl reference runs only that CPU path, with the same metric and config, on this box's host cores.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_HBM_GBS = 6650.0   # an earlier copy-bandwidth measurement on B200, used only when MEASURED_PEAKS.json is absent
NOMINAL_HBM_GBS = 8000.0
L2_BYTES = 126 * 1024 * 1024
# DRAM bytes per leading unit (row / matrix) of one launch, from the ncu captures summarised under profiles/ (small cases of
# the same kernels; traffic grows in proportion to the units): dram__bytes_read.sum per unit as captured, plus the unit's
# output bytes for the write side -- in the captures part of the output is still dirty in L2 when the kernel ends (89 MB
# of 134 MB written for RMSNorm), so dram__bytes_write.sum itself understates what a launch eventually writes.
NCU_DRAM_BYTES_PER_UNIT = {"rmsnorm": 143289088 / 8192 + 16384, "bmm4x4": 134688512 / 1048576 + 64, "inv4x4": 67286016 / 1048576 + 64}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.device_index), "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        torch.cuda.set_device(local)
        # the data path has no collective: the process group only carries the barrier and the max-over-ranks of the timing,
        # so the CPU backend is enough (and nothing but the JSON line reaches stdout)
        dist.init_process_group("gloo")
    return rank, world, local


def pin_to_gpu_numa_node(local: int):
    """Run this rank's host threads on the CPUs next to its GPU, so that the pinned host buffers of the end-to-end leg
    (allocated afterwards, first touch) and the copies' staging live on the GPU's own NUMA node instead of all ranks sharing
    node 0. Returns a short description, or None when the topology cannot be read."""
    try:
        prop = torch.cuda.get_device_properties(local)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = f.read().strip()
        return f"gpu {local} ({bdf}): numa node {node}, {len(cpus)} cpus"
    except Exception:
        return None


def barrier(world: int):
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_device(fn, steps: int, world: int) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the current stream, barrier + synchronize on both sides,
    max over ranks."""
    stream = torch.cuda.current_stream()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    barrier(world)
    return max_over_ranks(start.elapsed_time(stop), world)


# ---------------------------------------------------------------------------------------------------- CPU baseline

def cpu_reference(name: str, budget_s: float, steps: int = 1, warmup: int = 1):
    """Times the reference's CPU path for `name` -- torch eager on fp32 CPU tensors with all host threads, the expression
    the reference's tests use as their oracle -- on a bounded sample of the workload. Returns (GB/s, description, cores, ms)."""
    from gint_b200.workloads import EAGER, FULL_SIZES, make_workload
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    full_leading, inner = FULL_SIZES[name]
    sample = {"add": full_leading, "rmsnorm": 2048, "bmm4x4": 524288, "inv4x4": 524288, "graph": 8192, "graph_gathered": 8192}[name]
    wl = make_workload(name, sample, inner, device="cpu")
    fn = EAGER[name]
    for _ in range(max(1, warmup)):
        fn(wl.tensors)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < max(steps, 1) or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        fn(wl.tensors)
        times.append(time.perf_counter() - t0)
        if len(times) >= steps and time.perf_counter() >= t_end:
            break
    best = min(times)
    gbs = wl.algorithmic_bytes / best / 1e9
    desc = f"torch eager fp32 on CPU, {sample} of {full_leading} leading units x {inner}, best of {len(times)}"
    return gbs, desc, torch.get_num_threads(), statistics.mean(times) * 1e3, wl


def oracle_port_speed(wl_cpu, budget_rows: int = 256):
    """The C restatement of the interpreter (oracle/), timed on a few hundred logical programs: context for the
    torch-eager baseline, not a baseline itself."""
    from oracle import oracle
    st = wl_cpu.steps[0]
    grid = min(st.grid_dim, budget_rows)
    threads = os.cpu_count() or 1
    t0 = time.perf_counter()
    oracle.execute(st.program.bytecode, [vars(t) for t in st.program.tensor_infos], [wl_cpu.tensors[r] for r in st.roles], grid,
                   input_indices=st.program.input_indices, threads=threads)
    dt = time.perf_counter() - t0
    bytes_ = wl_cpu.algorithmic_bytes * grid / st.grid_dim
    return {"value": bytes_ / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{grid} logical programs of the same bytecode through oracle/gint_oracle.c"}


# ---------------------------------------------------------------------------------------------------- GPU side

def graph_replay_us(wls, ex, steps: int) -> float:
    """Device time per pass with the host taken out: all buffer sets' launches captured once into a CUDA graph (the launch
    entry point allocates nothing and copies nothing, so it can be captured) and the replays timed with CUDA events."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for wl in wls:
            wl.run(ex, side.cuda_stream)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for wl in wls:
                wl.run(ex, torch.cuda.current_stream().cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / (steps * len(wls))


def host_dispatch_us(wls, ex, stream: int, reps: int = 200) -> float:
    """Host time per call of the launch path (argument conversion, cache lookup, the C call), device idle-time excluded:
    wall clock over a burst of launches that are not waited for."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(reps):
        wls[i % len(wls)].run(ex, stream)
    dt = time.perf_counter() - t0
    torch.cuda.synchronize()
    n_launch = sum(wls[i % len(wls)].launches_per_run() for i in range(reps))
    return dt * 1e6 / n_launch


LEAN = False


def run_program_bench(name: str, world: int, rank: int, steps: int, warmup: int, peak_gbs: float, impl: str = "b200"):
    """Device-resident timing of one named program at its benchmark size (sharded `world` ways). impl "reference_kernel" runs
    the same buffers through the reference's own executor and sm_100 kernels (baseline/_ref)."""
    from gint_b200 import get_executor
    from gint_b200.workloads import FULL_SIZES, make_workload
    ex = get_executor()
    if impl == "reference_kernel":
        from baseline import ref_harness
    leading, inner = FULL_SIZES[name]
    seed = 42 + rank
    # a+b is 12 MB and would sit in L2: rotate over enough independent buffer sets to exceed it
    n_sets = 1
    wls = [make_workload(name, leading, inner, device="cuda", seed=seed)]
    if wls[0].algorithmic_bytes < 2 * L2_BYTES:
        n_sets = int(2 * L2_BYTES // wls[0].algorithmic_bytes) + 1
        wls += [make_workload(name, leading, inner, device="cuda", seed=seed + 1000 + i) for i in range(n_sets - 1)]
    stream = torch.cuda.current_stream().cuda_stream
    state = {"i": 0}

    # the executor's plan API: the steps of one pass are lowered once, a pass is then one library call (gint_execute_plan)
    plans = [wl.plan(ex) for wl in wls] if impl == "b200" else None

    def step():
        wl = wls[state["i"] % n_sets]
        if impl == "reference_kernel":
            ref_harness.run_workload(wl, stream)
        else:
            plan = plans[state["i"] % n_sets]
            if plan is None:               # gathered rows: plain executor calls
                wl.run(ex, stream)
            else:
                if wl.pre is not None:
                    wl.pre(wl.tensors)
                plan.run(stream)
        state["i"] += 1
    for _ in range(max(3, warmup, n_sets)):   # every buffer set once at least: its program is built on first use
        step()
    # a pass of a few microseconds is timed over many passes per step, so that the start-up of the first launch and the
    # two event records do not weigh on it
    probe = time_device(step, 3, world) / 3
    passes = 1 if probe > 0.05 else 40
    launches0 = ex.launches
    ms = time_device(step, steps * passes, world) / passes
    launches = (ex.launches - launches0) // passes
    wl = wls[0]
    total_bytes = wl.algorithmic_bytes * world
    per_step_ms = ms / steps
    st = wl.steps[0]
    if impl == "reference_kernel":
        return {"ms_per_step": per_step_ms, "gbs": total_bytes / (per_step_ms * 1e-3) / 1e9,
                "kernels": [ref_harness.variant_of(s_.program) for s_ in wl.steps],
                "frac_of_measured_peak": total_bytes / (per_step_ms * 1e-3) / 1e9 / (peak_gbs * world)}, wls
    info = ex.launch_info(st.program, [wl.tensors[r] for r in st.roles], st.grid_dim)
    split = {}
    if wl.pre is None and world == 1 and plans[0] is not None and not LEAN:
        # host and device separated: the event-timed figure above includes whatever the host fails to hide
        try:
            split = {"device_us_per_launch": graph_replay_us(wls, ex, max(10, steps)),
                     "host_dispatch_us_per_launch": host_dispatch_us(wls, ex, stream)}
            split["gbs_device_only"] = wl.algorithmic_bytes / wl.launches_per_run() / (split["device_us_per_launch"] * 1e-6) / 1e9
        except Exception as e:   # context only
            split = {"split_error": str(e)[:200]}
    return {
        **split,
        "ms_per_step": per_step_ms,
        "gbs": total_bytes / (per_step_ms * 1e-3) / 1e9,
        "elements_per_s": wl.elements * world / (per_step_ms * 1e-3),
        "algorithmic_bytes": total_bytes,
        "launches": launches,
        "launches_per_step": wl.launches_per_run(),
        "l2": "inputs larger than L2" if n_sets == 1 else f"rotating {n_sets} buffer sets (> 2x L2)",
        "passes_per_timed_step": passes,
        "geometry": {k: info[k] for k in ("pool_size", "tiles_per_warp", "grid_blocks", "regs_per_thread", "blocks_per_sm", "smem_bytes")},
        "frac_of_measured_peak": total_bytes / (per_step_ms * 1e-3) / 1e9 / (peak_gbs * world),
        "frac_of_8TBs": total_bytes / (per_step_ms * 1e-3) / 1e9 / (NOMINAL_HBM_GBS * world),
    }, wls


def run_e2e(name: str, world: int, rank: int, steps: int, warmup: int, overlapped: bool = True):
    """Same metric through the public API with HOST buffers: every step copies the inputs from pinned host memory,
    runs the program and copies the result back."""
    from gint_b200 import get_executor
    from gint_b200.workloads import FULL_SIZES, make_workload
    ex = get_executor()
    leading, inner = FULL_SIZES[name]
    wl = make_workload(name, leading, inner, device="cuda", seed=42 + rank)
    in_roles = [r for r in wl.tensors if r not in wl.outputs and r not in ("g", "x_rows")]
    host_in = {r: wl.tensors[r].cpu().pin_memory() for r in in_roles}
    host_out = {r: torch.empty(wl.tensors[r].shape, dtype=wl.tensors[r].dtype).pin_memory() for r in wl.outputs}
    stream = torch.cuda.current_stream().cuda_stream
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())

    single = overlapped and len(wl.steps) == 1 and wl.pre is None
    if single:   # the executor's host-data call: transfers overlapped with the kernels, range by range
        st = wl.steps[0]
        dev = [wl.tensors[r] for r in st.roles]
        ins = {i: host_in[r] for i, r in enumerate(st.roles) if r in host_in}
        outs = {i: host_out[r] for i, r in enumerate(st.roles) if r in host_out}

        def step():
            ex.execute_streamed(st.program, dev, st.grid_dim, ins, outs, n_chunks=16)
    else:
        def step():
            for r in in_roles:
                wl.tensors[r].copy_(host_in[r], non_blocking=True)
            wl.run(ex, stream)
            for r in wl.outputs:
                host_out[r].copy_(wl.tensors[r], non_blocking=True)
    for _ in range(max(1, min(warmup, 3))):
        step()
    ms = time_device(step, steps, world)
    per_step = ms / steps
    return {"value": wl.algorithmic_bytes * world / (per_step * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": per_step,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "api": "B200Executor.execute_streamed (16 ranges, copies overlapped with kernels)" if single else "B200Executor.execute between whole-tensor copies"}


def run_strong_scaling(name: str, world: int, rank: int, steps: int, warmup: int):
    """The FIXED benchmark configuration cut `world` ways by its leading dimension: every rank launches its contiguous range of
    the full-size program's logical grid with gint_execute_range (same program, same descriptors, no collective) on rows it holds.
    Time = slowest rank; value = the whole fixed batch's bytes over that time."""
    from gint_b200 import get_executor
    from gint_b200.host.executor import _convert_arg
    from gint_b200.shard import shard_range
    from gint_b200.workloads import FULL_SIZES, make_workload
    ex = get_executor()
    leading, inner = FULL_SIZES[name]
    wl = make_workload(name, leading, inner, device="cuda", seed=42)     # same seed everywhere: one batch, replicated for simplicity
    if len(wl.steps) != 1 or wl.pre is not None:
        return None
    st = wl.steps[0]
    args = [_convert_arg(wl.tensors[r]) for r in st.roles]
    first, count = shard_range(st.grid_dim, world, rank)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        ex.execute_range(st.program, args, first, count, cuda_stream=stream)
    for _ in range(max(3, warmup)):
        step()
    ms = time_device(step, steps, world) / steps
    return {"ms_per_step": ms, "gbs": wl.algorithmic_bytes / (ms * 1e-3) / 1e9, "scaling": "strong",
            "what": f"{leading} leading units in total, {world} contiguous ranges of the one program's grid (gint_execute_range)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="rmsnorm", choices=["add", "rmsnorm", "bmm4x4", "inv4x4", "graph", "graph_gathered"])
    ap.add_argument("--programs", default="all", choices=["all", "none"], help="also time the other named programs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--leading", type=int, default=0, help="override the leading dimension (a recorded size; small profiler captures)")
    ap.add_argument("--lean", action="store_true", help="device-timed leg only: no end-to-end, reference-kernel, host/device split or CPU legs (profiler captures)")
    opts = ap.parse_args()
    global LEAN
    LEAN = opts.lean
    warmup = max(opts.warmup, 3)
    peak, peak_kind = measured_peak()
    metric = "achieved HBM GB/s per bytecode program (algorithmic bytes / device time)"
    name = opts.workload
    from gint_b200.workloads import FULL_SIZES
    if opts.leading:
        FULL_SIZES[name] = (opts.leading, FULL_SIZES[name][1])
    leading, inner = FULL_SIZES[name]
    config = {"workload": {"add": "configs[0] a+b fp32 [1048576]", "rmsnorm": "configs[1] RMSNorm x fp32 [16384,4096], conductor-lowered bytecode (363 insns)",
                           "bmm4x4": "configs[2] batched 4x4 matmul [4194304,4,4]", "inv4x4": "configs[3] batched 4x4 inverse [4194304,4,4]",
                           "graph": "configs[4] conductor graph x [65536,1024]",
                           "graph_gathered": "configs[4] conductor graph x [65536,1024], gather folded into the fused program"}[name],
              "leading": leading, "inner": inner, "sharding": f"{opts.gpus} rank(s), each running its own {leading}-unit shard of a {opts.gpus * leading}-unit batch; no collective"}

    if opts.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        if rank != 0:
            return 0
        gbs, desc, cores, ms, _ = cpu_reference(name, budget_s=20.0, steps=opts.steps if opts.steps < 20 else 20, warmup=min(warmup, 3))
        line = {"impl": "reference", "metric": metric, "value": gbs, "unit": "GB/s", "n_gpus": opts.gpus, "steps": opts.steps,
                "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic (seeded)", "config": config,
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "reference", "sample": desc},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "the reference has no CPU bytecode executor; its CPU path for these programs is the torch-eager "
                        "expression its tests use as oracle"}
        print(json.dumps(line))
        return 0

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: gint_b200 has no CPU path"}))
        return 1
    rank, world, local = dist_setup(opts.gpus)
    torch.cuda.set_device(local)
    numa = pin_to_gpu_numa_node(local) if world > 1 else None

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    res, wls = run_program_bench(name, world, rank, opts.steps, warmup, peak)
    clocks = sampler.stop() if sampler else None
    del wls
    torch.cuda.empty_cache()
    if opts.lean:
        e2e = None
    else:
        e2e = run_e2e(name, world, rank, max(3, min(opts.steps, 10)), warmup)
        torch.cuda.empty_cache()
        e2e["unoverlapped"] = {k: v for k, v in run_e2e(name, world, rank, max(3, min(opts.steps, 10)), warmup, overlapped=False).items()
                               if k in ("value", "ms_per_step", "api")}
        torch.cuda.empty_cache()

    programs = {}
    if opts.programs == "all":
        # the five named programs, and the conductor graph once more with its gather folded into the fused program's loads
        for other in ("add", "rmsnorm", "bmm4x4", "inv4x4", "graph", "graph_gathered"):
            if other == name:
                programs[other] = res
                continue
            r, w_ = run_program_bench(other, world, rank, max(10, min(opts.steps, 30)), warmup, peak)
            programs[other] = r
            del w_
            torch.cuda.empty_cache()
    # the reference's own kernels (its sm_100 build of geval_s7 / geval_l12, through its unmodified executor), same buffers and
    # timing: what this library replaces, on this box
    ref_kernel_note = None
    if world == 1 and not opts.lean:
        try:
            from baseline import ref_harness
            if not ref_harness.available():
                ref_kernel_note = ref_harness.why_unavailable()
            else:
                for other in (("add", "rmsnorm", "bmm4x4", "inv4x4", "graph") if opts.programs == "all" else (name,)):
                    r, w_ = run_program_bench(other, world, rank, max(5, min(opts.steps, 20)), warmup, peak, impl="reference_kernel")
                    (programs[other] if other in programs else res)["reference_kernel"] = r
                    del w_
                    torch.cuda.empty_cache()
        except Exception as e:
            ref_kernel_note = f"{type(e).__name__}: {str(e)[:300]}"
    strong = run_strong_scaling(name, world, rank, max(10, min(opts.steps, 30)), warmup) if world > 1 else None

    if rank == 0:
        line = {
            "metric": metric, "value": res["gbs"], "unit": "GB/s", "n_gpus": world, "steps": opts.steps, "warmup": warmup,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic (seeded)",
            "config": config, "l2": res["l2"], "elements_per_s": res["elements_per_s"], "geometry": res["geometry"],
            "clocks": clocks, "e2e": e2e, "gpu_launches": res["launches"],
            "roofline": {"bound": "hbm", "achieved": res["gbs"] / world, "peak": peak, "unit": "GB/s",
                         "frac": res["gbs"] / world / peak, "peak_kind": f"of {peak_kind}", "frac_of_8TBs": res["frac_of_8TBs"],
                         "traffic": (NCU_DRAM_BYTES_PER_UNIT[name] * leading) if name in NCU_DRAM_BYTES_PER_UNIT else None,
                         "traffic_source": "ncu dram__bytes_read per row of the 8192-row capture (profiles/) + output bytes per row, x rows of this launch",
                         "algorithmic_bytes_per_launch": res["algorithmic_bytes"] // world,
                         "kernel_ms": res["ms_per_step"] / res["launches_per_step"]},
            "programs": {k: {kk: vv for kk, vv in v.items() if kk not in ("launches",)} for k, v in programs.items()},
        }
        if "reference_kernel" in res:
            line["reference_kernel"] = res["reference_kernel"]
        if ref_kernel_note:
            line["reference_kernel_unavailable"] = ref_kernel_note
        if strong is not None:
            line["strong_scaling"] = strong
        if numa:
            line["host_placement"] = numa
        if not opts.no_cpu and not opts.lean:
            gbs, desc, cores, ms, wl_cpu = cpu_reference(name, budget_s=10.0)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "reference", "sample": desc}
            try:
                line["cpu_oracle_port"] = oracle_port_speed(wl_cpu)
            except Exception as e:  # the port is context only
                line["cpu_oracle_port"] = {"error": str(e)}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
