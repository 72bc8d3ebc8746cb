#!/usr/bin/env python
"""Benchmark of the recurrent hot path: fwd+bwd tokens/s (B*T per second).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C2|C3|C4|C5] [--impl ours|reference|reference_gpu]

One JSON line on stdout (rank 0).  A "step" is one forward + backward pass of the whole sequence:
frnn_forward + frnn_backward + frnn_finalize_grads through the C ABI on device-resident buffers (`value`), and the same
step through the public `flashrnn()` API with pinned HOST inputs, host->device copies and a device->host read of the
gradients inside the timed region (`e2e`).  The headline workload is the LSTM configuration (C2); the other benchmark
configurations ride along in `workloads` (same harness, device-resident inputs).  The timed region is a series of
blocks of K steps (at least three blocks and half a second); `ms_per_step` is the median block, max over ranks.

With N > 1 every rank runs the headline workload on its own batch shard (weak scaling: global batch = N x workload
batch) and the fp32 dR || db are all-reduced with NCCL inside the step; `workloads` then holds the Elman configuration
batch-sharded weak (1024 rows per GPU) and strong (1024 rows in all) and the GRU configuration head-sharded, each with
the time the same workload takes on rank 0 alone.

`--impl reference` times the CPU restatement of the reference's `vanilla` backend (oracle/vanilla_port.py) on the host
cores on a bounded sample of the same workload.  `--impl reference_gpu` times the reference's own CUDA backend
(`cuda_fused`; `cuda` for the GRU), imported unmodified from baseline/_ref, on the same GPU and inputs.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

# name -> (function, B, T, N, D, states fp32)
WORKLOADS = {
    "C2": ("lstm", 16, 1024, 4, 256, False),
    "C3": ("gru", 32, 2048, 8, 128, False),
    "C4": ("slstm", 8, 4096, 4, 192, True),
    "C5": ("elman", 1024, 2048, 16, 64, False),
    "C5s": ("elman", 1024, 256, 16, 64, False),  # C5 with T cut to 256 (2.1 GB resident): the size ncu captures use
    "LB": ("lstm", 1024, 512, 16, 64, False),    # large-batch LSTM (the reference's batch-size sweeps): 16-row tiles, HBM-side regime
    "LBs": ("lstm", 512, 128, 16, 64, False),    # LB cut to 0.7 GB resident (512 CTAs, same tile): the size ncu captures use
    "LBm": ("lstm", 1024, 64, 16, 64, False),    # LB with T cut to 64 (1.3 GB resident, 128 CTAs of 128 rows): ncu captures of the memory-bound case
    "GB": ("gru", 1024, 512, 16, 64, False),     # large-batch GRU, as LB
    # the head-dim sweep of the reference's README figure (LSTM bf16 B16 T1024, head_dim x heads = 768)
    "H16": ("lstm", 16, 1024, 48, 16, False), "H32": ("lstm", 16, 1024, 24, 32, False), "H64": ("lstm", 16, 1024, 12, 64, False),
    "H128": ("lstm", 16, 1024, 6, 128, False), "H256": ("lstm", 16, 1024, 3, 256, False), "H768": ("lstm", 16, 1024, 1, 768, False),
}
DIMS = {"lstm": (4, 4, 4, 2), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1), "slstm": (4, 4, 4, 4)}
METRIC = "fwd+bwd tokens/sec (B*T/s)"
# DRAM bytes (read + write) of ONE launch of the reverse time loop, from an `ncu --set full` capture of
# `python bench.py --steps 2 --warmup 1 --no-cpu` on a B200; reported with its provenance, for the kernel build named.
NCU_TRAFFIC = {"C2": {"bytes": 237_750_016 + 105_541_632, "source": "ncu --set full capture of frnn_bwd_kernel<lstm,KT16,NT1,MPW2> on this "
                      "command line with --steps 1 --min-seconds 0, 2026-11-25 (the kernel has not changed since)"}}
# fwd+bwd of the reference's own CUDA backend on a B200 of this pool, measured by `bench.py --impl reference_gpu`
# (tokens/s; None: not measured).  The live arm is the source of truth; this record lets the default line carry the ratio.
REFERENCE_GPU_RECORD = {
    "C2": {"value": 1549168.3, "unit": "tokens/s", "ms_per_step": 10.576,
           "source": "`bench.py --impl reference_gpu --steps 10` on a B200 of this pool, 2026-11-25: the reference's cuda_fused backend "
                     "(unmodified, baseline/_ref, its own JIT build and tiling search), bf16, same seeded inputs, median of 5 blocks of "
                     "10 steps, CUDA events, SM clock 1965 MHz, no throttle reason"},
}


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1407.4))), "measured"
    return 6650.0, 1400.0, "fallback"


def make_inputs(function, B, T, N, D, f32_states, device, seed=0, edt=torch.bfloat16):
    """Seeded synthetic inputs with the shapes and distributions of the named configuration (``edt``: the 16-bit type).
    Generated on ``device`` (the large configurations would take the host cores tens of seconds)."""
    Gr, Gw, Gt, S = DIMS[function]
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *shape: torch.randn(*shape, generator=g, device=device)
    Wx = rn(B, T, Gw, N, D).to(edt)
    R = (rn(Gr, N, D, D) / D ** 0.5).to(edt)
    b = 0.1 * rn(Gt, N, D)
    if function == "gru":
        b.zero_()
    if function == "slstm":
        b.zero_()
        b[1] = 3.0 + 3.0 * torch.rand(N, D, generator=g, device=device)
    b = b.to(edt)
    sdt = torch.float32 if f32_states else edt
    s0 = (0.1 * rn(S, B, 1, N, D) if function == "lstm" else torch.zeros(S, B, 1, N, D, device=device)).to(sdt)
    return [Wx, R, b, s0]


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML from a background thread while the timed region
    runs (every ~4 ms; only reads, no setting is touched)."""

    REASONS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index: int):
        self.idx, self.samples, self.mask, self.max_mhz = gpu_index, [], 0, None
        self._stop = threading.Event()
        self._th = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(physical_index(gpu_index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:  # no NVML: the line then carries empty clock fields
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception:
                break
            time.sleep(0.004)

    def __enter__(self):
        if self.nv is not None:
            self._th = threading.Thread(target=self._run, daemon=True)
            self._th.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=2)

    def summary(self):
        sm = sorted(self.samples)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": [n for n, bit in self.REASONS if self.mask & bit], "samples": len(sm)}


def physical_index(gpu_index: int) -> int:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible and len(visible.split(",")) > gpu_index and visible.split(",")[gpu_index].isdigit():
        return int(visible.split(",")[gpu_index])
    return gpu_index


def bind_to_gpu_numa_node(gpu_index: int):
    """Restricts this process to the host cores of the NUMA node its GPU hangs off, so that the pinned staging buffers
    allocated afterwards (first touch) sit in that node's memory.  Returns the node, or None when the box does not say."""
    try:
        import pynvml

        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(physical_index(gpu_index))).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        bus = bus[-12:] if len(bus) > 12 else bus  # 00000000:1b:00.0 -> 0000:1b:00.0
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
        if node < 0:
            # sysfs does not say (containers often hide it): ask NVML for the cores closest to the GPU
            ncpu = os.cpu_count() or 1
            words = pynvml.nvmlDeviceGetCpuAffinity(pynvml.nvmlDeviceGetHandleByIndex(physical_index(gpu_index)), (ncpu + 63) // 64)
            near = {64 * i + j for i, w in enumerate(words) for j in range(64) if (int(w) >> j) & 1}
            allowed = near & os.sched_getaffinity(0)
            if allowed and allowed != os.sched_getaffinity(0):
                os.sched_setaffinity(0, allowed)
                return f"nvml affinity: {len(allowed)} cores"
            return None
        cpus = set()
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return node
    except Exception:
        pass
    return None


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(function, B, T, N, D, target_seconds=8.0, reps=2):
    """fwd+bwd of the reference's CPU algorithm (torch restatement, autograd backward, all host threads) on a
    bounded sample: same cell, N, D; batch and T cut so that one pass takes about `target_seconds`."""
    from oracle.vanilla_port import vanilla_fwbw

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Gr = DIMS[function][0]
    Bs = B
    while Bs > 1 and Bs * N * Gr * D * D * 4 * 16 > 8e9:  # autograd keeps ~B*N*Gr*D*D*4 bytes per time step
        Bs //= 2

    def one(Ts):
        Wx, R, b, s0 = (t.float() for t in make_inputs(function, Bs, Ts, N, D, True, "cpu"))
        t0 = time.perf_counter()
        vanilla_fwbw(Wx, R, b, s0, function)
        return time.perf_counter() - t0

    one(2)
    per_step = max(one(4) / 4, 1e-6)
    mem_cap = int(6e9 // max(1, Bs * N * Gr * D * D * 4))
    Ts = int(max(4, min(T, 128, mem_cap, target_seconds / per_step)))
    best = min(one(Ts) for _ in range(reps))
    return {"value": Bs * Ts / best, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{function} fp32 B={Bs} T={Ts} N={N} D={D} fwd+bwd (loss=sum(h)), best of {reps}", "seconds": best}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    function, B, T, N, D, f32 = WORKLOADS[args.workload]
    vals = []
    per = max(0.5, min(8.0, 120.0 / (args.warmup + args.steps)))  # whole run stays within a few minutes
    for i in range(args.warmup + args.steps):
        r = cpu_sample(function, B, T, N, D, target_seconds=per, reps=1)
        if i >= args.warmup:
            vals.append(r)
    v = sum(x["value"] for x in vals) / len(vals)
    sec = sum(x["seconds"] for x in vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {function} B={B} T={T} N={N} D={D} (CPU sample, see cpu_baseline.sample)"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": vals[0]["cores"], "kind": "port", "sample": vals[0]["sample"]},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------------ reference on the GPU
def run_reference_gpu(args):
    """fwd+bwd of the reference's own CUDA backend on this GPU: the unmodified package from baseline/_ref through its
    public `flashrnn()` call (protocol of its speed_experiments/kernel_speed_benchmark.py:237-248: bf16, inputs that
    require grad, loss = h.sum()), CUDA events, its JIT build and tiling search excluded by warm-up.  One attempt: a
    failing build, tiling solve or launch prints an `unavailable` line."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    function, B, T, N, D, f32 = WORKLOADS[args.workload]
    backend = "cuda" if function == "gru" else "cuda_fused"  # the reference runs the GRU on its alternating backend only
    base = {"impl": "reference_gpu", "metric": METRIC, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {function} fwd+bwd B={B} T={T} N={N} D={D}, loss=sum(h), reference backend '{backend}'"}}
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "flashrnn").exists():
        print(json.dumps({**base, "unavailable": "baseline/_ref holds no reference install"}), flush=True)
        return 0
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", str(ROOT / "baseline" / "_ref_ext"))  # the reference's JIT builds land here
    os.environ.setdefault("CONSTRINT_CACHE_DIR", str(ROOT / "baseline" / "_ref_ext" / "constrint"))
    Path(os.environ["TORCH_EXTENSIONS_DIR"]).mkdir(parents=True, exist_ok=True)
    t_start = time.time()
    try:
        sys.path.insert(0, str(ref_root))
        for m in [m for m in sys.modules if m == "flashrnn" or m.startswith("flashrnn.")]:
            del sys.modules[m]
        from flashrnn import flashrnn as ref_flashrnn  # the reference, unmodified

        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        Wx, R, b, s0 = make_inputs(function, B, T, N, D, False, dev, seed=0)
        Wx.requires_grad_(True), R.requires_grad_(True), b.requires_grad_(True)

        def step():
            Wx.grad = R.grad = b.grad = None
            h, _ = ref_flashrnn(Wx, R, b, s0, function=function, backend=backend, dtype="bfloat16")
            h[0].sum().backward()

        step()  # JIT build + tiling search
        torch.cuda.synchronize()
        build_s = time.time() - t_start
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        ev = lambda: torch.cuda.Event(enable_timing=True)
        blocks = []
        with ClockSampler(0) as clk:
            t0 = time.time()
            while len(blocks) < 3 or (time.time() - t0 < 0.5 and len(blocks) < 50):
                e0, e1 = ev(), ev()
                e0.record()
                for _ in range(args.steps):
                    step()
                e1.record()
                torch.cuda.synchronize()
                blocks.append(e0.elapsed_time(e1) / args.steps)
        ms = statistics.median(blocks)
        line = {**base, "value": B * T / (ms * 1e-3), "ms_per_step": ms, "ms_per_step_best": min(blocks), "blocks": len(blocks),
                "build_and_first_call_s": build_s, "clocks": clk.summary(), "torch_extensions_dir": os.environ["TORCH_EXTENSIONS_DIR"]}
    except BaseException as e:  # noqa: BLE001 - every failure of the reference becomes its own `unavailable` line
        line = {**base, "unavailable": f"{type(e).__name__}: {str(e)[:400]}", "after_s": time.time() - t_start}
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------------ GPU arm
class Job:
    """Process-wide state of the GPU arm."""

    def __init__(self, args):
        from flashrnn_b200 import _native as nv

        self.nv, self.L, self.args = nv, nv.lib(), args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device: flashrnn_b200 has no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.stream = torch.cuda.current_stream(self.dev)
        self.sp = ctypes.c_void_p(self.stream.cuda_stream)
        self.f16 = args.dtype == "float16"
        self.f32io = args.dtype == "float32"  # the float32 loops (CUDA cores): everything, states included, fp32
        self.edt = torch.float32 if self.f32io else (torch.float16 if self.f16 else torch.bfloat16)
        self.hbm_peak, self.tc_peak, self.peak_source = measured_peaks()

    def barrier(self, group=True):
        if self.dist is not None and group:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values, group=True):
        if self.dist is None or not group:
            return list(values)
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]


def measure(job: Job, function, B, T, N, D, f32, *, allreduce, group=True, cluster_size=0, batch_tile=0, floor=True,
            min_seconds=None, keep=None):
    """The C-ABI step (forward, reverse loop, dR, [all-reduce,] cast) of one workload on resident buffers.
    ``group``: the ranks run it together (barriers, max over ranks); False: this rank alone.  Returns a dict of timings;
    ``keep`` (a dict) receives the tensors for a caller that goes on to use them."""
    nv, L, dev, stream, sp, args = job.nv, job.L, job.dev, job.stream, job.sp, job.args
    min_seconds = args.min_seconds if min_seconds is None else min_seconds
    Gr, Gw, Gt, S = DIMS[function]
    f32 = f32 or job.f32io
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, f32, dev, seed=job.rank, edt=job.edt)
    sdt = torch.float32 if f32 else job.edt
    esz, ssz = (4 if job.f32io else 2), (4 if f32 else 2)
    E = B * T * N * D
    prob = nv.make_problem(function, B, T, N, D, f32, True, f16=job.f16, f32=job.f32io)
    plan = nv.query(prob, cluster_size, batch_tile)
    states = torch.empty(S, B, T, N, D, device=dev, dtype=sdt)
    cache = torch.empty(max(16, int(plan.cache_bytes)), device=dev, dtype=torch.uint8)
    ws = torch.empty(int(plan.workspace_bytes), device=dev, dtype=torch.uint8)
    dstates = torch.zeros_like(states)
    dstates[0] = 1.0  # loss = sum(h)
    dWx, ds0 = torch.empty_like(Wx), torch.empty_like(s0)
    dR, db = torch.empty_like(R), torch.empty_like(b)
    goff, gcnt = int(plan.grads_offset), int(plan.grads_count)
    grads = ws[goff:goff + 4 * gcnt].view(torch.float32)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    fa = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), P(ws))
    ba = nv.FrnnBwdArgs(P(R), P(s0), P(states), P(cache), P(dstates), P(dWx), P(ds0), P(ws))
    ev = lambda: torch.cuda.Event(enable_timing=True)
    do_allreduce = allreduce and job.dist is not None and group

    def step(rec=None, pl=plan):
        if rec: rec[0].record(stream)
        nv.check("frnn_forward", L.frnn_forward(ctypes.byref(pl), ctypes.byref(fa), sp))
        if rec: rec[1].record(stream)
        nv.check("frnn_backward_parts", L.frnn_backward_parts(ctypes.byref(pl), ctypes.byref(ba), sp, 1))
        if rec: rec[2].record(stream)
        nv.check("frnn_backward_parts", L.frnn_backward_parts(ctypes.byref(pl), ctypes.byref(ba), sp, 2))
        if rec: rec[3].record(stream)
        if do_allreduce:
            job.dist.all_reduce(grads)
        nv.check("frnn_finalize_grads", L.frnn_finalize_grads(ctypes.byref(pl), P(grads), P(dR), P(db), sp))

    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    job.barrier(group)
    # ---- timed region: blocks of `steps` steps, at least 3 and at least `min_seconds`; the number of blocks is fixed
    # from the warm-up's pace so that every rank runs the same count
    e0, e1 = ev(), ev()
    e0.record(stream)
    step()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    est = job.max_over_ranks([e0.elapsed_time(e1)], group)[0]
    nblocks = int(min(50, max(3, -(-min_seconds * 1e3 // max(1e-3, est * args.steps)))))
    recs = [[[ev() for _ in range(4)] for _ in range(args.steps)] for _ in range(nblocks)]
    marks = [ev() for _ in range(nblocks + 1)]
    with ClockSampler(job.local) as clk:
        job.barrier(group)
        marks[0].record(stream)
        for bi in range(nblocks):
            for i in range(args.steps):
                step(recs[bi][i])
            marks[bi + 1].record(stream)
        job.barrier(group)
    block_ms = job.max_over_ranks([marks[i].elapsed_time(marks[i + 1]) / args.steps for i in range(nblocks)], group)
    ms = statistics.median(block_ms)
    st = nv.FrnnDevStatus()
    nv.check("frnn_read_device_status", L.frnn_read_device_status(P(ws), sp, ctypes.byref(st)))
    if st.code != 0:
        raise RuntimeError(f"device-side wait expired (step {st.where}, cta {st.cta}); results invalid")
    flat = [r for blk in recs for r in blk]
    fwd_ms = statistics.median(r[0].elapsed_time(r[1]) for r in flat)
    bwd_ms = statistics.median(r[1].elapsed_time(r[2]) for r in flat)
    dr_ms = statistics.median(r[2].elapsed_time(r[3]) for r in flat)

    # ---- floor of the serial chain: the same loops with the gate arithmetic taken out (frnn_plan.probe_noop_cell)
    chain = None
    wide = plan.batch_tile == 128
    if floor and not wide:
        probe = nv.FrnnPlan.from_buffer_copy(plan)
        probe.probe_noop_cell = 1
        if (L.frnn_forward(ctypes.byref(probe), ctypes.byref(fa), sp) == 0 and
                L.frnn_backward_parts(ctypes.byref(probe), ctypes.byref(ba), sp, 1) == 0):  # else: no probe for this tile
            k = max(5, args.steps)
            ef = [ev() for _ in range(3)]
            for _ in range(2):
                L.frnn_forward(ctypes.byref(probe), ctypes.byref(fa), sp)
                L.frnn_backward_parts(ctypes.byref(probe), ctypes.byref(ba), sp, 1)
            ef[0].record(stream)
            for _ in range(k):
                nv.check("floor fwd", L.frnn_forward(ctypes.byref(probe), ctypes.byref(fa), sp))
            ef[1].record(stream)
            for _ in range(k):
                nv.check("floor bwd", L.frnn_backward_parts(ctypes.byref(probe), ctypes.byref(ba), sp, 1))
            ef[2].record(stream)
            torch.cuda.synchronize(dev)
            ff, fb = ef[0].elapsed_time(ef[1]) / k, ef[1].elapsed_time(ef[2]) / k
            chain = {"ms": ff + fb, "forward_ms": ff, "backward_ms": fb, "us_per_time_step": {"forward": 1e3 * ff / T, "backward": 1e3 * fb / T},
                     "frac_of_loops": (ff + fb) / (fwd_ms + bwd_ms),
                     "what": "2T dependent steps of the same loops with the gate arithmetic replaced by a pass-through "
                             "(exchange wait, matrix product, barriers, copies remain)"}
            step()  # leave real results behind
            torch.cuda.synchronize(dev)

    bwd_bytes = E * (S * ssz + S * ssz + Gw * esz)  # reverse loop: reads dstates and states, writes dWx
    fwd_bytes = E * (Gw * esz + S * ssz)            # forward loop: reads Wx, writes states
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    out = {
        "ms_per_step": ms, "ms_per_step_best": min(block_ms), "blocks": nblocks, "timed_seconds": sum(block_ms) * args.steps * 1e-3,
        "kernel_ms": {"forward_loop": fwd_ms, "backward_loop": bwd_ms, "recurrent_grad": dr_ms},
        "us_per_time_step": {"forward": 1e3 * fwd_ms / T, "backward": 1e3 * bwd_ms / T},
        "tile": {"cluster_size": plan.cluster_size, "units_per_cta": plan.units_per_cta, "batch_tile": plan.batch_tile, "threads": plan.threads,
                 "wide_forward": int(plan.wide_forward)},  # 1: forward loop on the 128-row tcgen05 kernel (LSTM, head dim 64)
        "roofline": {
            "bound": "hbm", "kernel": "wide_bwd_elman_kernel (reverse time loop, dR and db inside)" if wide else "frnn_bwd_kernel (reverse time loop)",
            "achieved": achieved, "peak": job.hbm_peak, "unit": "GB/s", "frac": achieved / job.hbm_peak, "peak_source": job.peak_source,
            "traffic": None, "traffic_source": None, "algorithmic_bytes_per_launch": bwd_bytes,
            "forward_loop": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / job.hbm_peak,
                             "algorithmic_bytes_per_launch": fwd_bytes},
            "whole_step": {"hbm_frac": (fwd_bytes + bwd_bytes) / (ms * 1e-3) / 1e9 / job.hbm_peak,
                           "tensor_frac": None if job.f32io else (6.0 * E * Gr * D / (ms * 1e-3) / 1e12) / job.tc_peak,
                           # float32 loops: FFMA on the CUDA cores; nominal 148 SMs x 128 lanes x 2 flop x max SM clock
                           "fp32_cuda_core_frac": (6.0 * E * Gr * D / (ms * 1e-3) / 1e12) / (148 * 128 * 2 * 1.965e-3) if job.f32io else None},
            "chain_floor": chain,
            "note": "streams one 16 KB tile per operand, step and CTA; HBM-bound" if wide else
                    "the serial chain of 2T dependent steps (chain_floor), not HBM or the tensor pipe, bounds this workload"},
        "clocks": clk.summary(), "launches_per_step": 3 if wide else 6,
    }
    if keep is not None:
        keep.update(Wx=Wx, R=R, b=b, s0=s0, gcnt=gcnt)
    return out


def measure_e2e(job: Job, function, tensors, gcnt, allreduce):
    """The same step through the public API with pinned HOST inputs: H2D of Wx/R/b/s0 and D2H of loss + dR/db inside
    the timed region, every step.  Inputs are double-buffered on the device: the copy of step i+1 (own stream) overlaps
    the kernels of step i, as an input pipeline with pinned memory does."""
    from flashrnn_b200 import flashrnn

    dev, stream, args, dist = job.dev, job.stream, job.args, job.dist
    ev = lambda: torch.cuda.Event(enable_timing=True)
    numa = bind_to_gpu_numa_node(job.local)
    hostW = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in tensors]
    host_out = torch.empty(gcnt, dtype=job.edt).pin_memory()
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [[torch.empty_like(t) for t in tensors] for _ in range(2)]
    ready = [ev(), ev()]   # inputs of the slot have landed
    free = [ev(), ev()]    # the step that used the slot has been queued behind (its kernels no longer read the inputs)

    def e2e_copy(slot, after=None):
        with torch.cuda.stream(copy_stream):
            if after is not None:
                copy_stream.wait_event(after)
            for dst, src in zip(bufs[slot], hostW):
                dst.copy_(src, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_compute(slot):
        stream.wait_event(ready[slot])
        w, r, bb, s = (t.detach() for t in bufs[slot])
        w.requires_grad_(True); r.requires_grad_(True); bb.requires_grad_(True)
        out, _ = flashrnn(w, r, bb, s, function=function, dtype=args.dtype,
                          grad_allreduce_group=(True if dist is not None and allreduce else None))
        loss = out[0].float().sum()
        loss.backward()
        host_out[: r.numel()].copy_(r.grad.reshape(-1), non_blocking=True)
        host_out[r.numel():].copy_(bb.grad.reshape(-1), non_blocking=True)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        free[slot].record(stream)

    def e2e_run(k, start):
        e2e_copy(0, after=start)
        for i in range(k):
            if i + 1 < k:
                e2e_copy((i + 1) & 1, after=free[(i + 1) & 1] if i >= 1 else None)
            e2e_compute(i & 1)

    warm = ev()
    warm.record(stream)
    e2e_run(2, warm)
    job.barrier()
    k2 = max(1, min(args.steps, 10))
    blocks = []
    for _ in range(3):
        e2, e3 = ev(), ev()
        job.barrier()
        e2.record(stream)
        e2e_run(k2, e2)
        e3.record(stream)
        job.barrier()
        blocks.append(e2.elapsed_time(e3) / k2)
    e2e_ms = statistics.median(job.max_over_ranks(blocks))
    h2d = sum(t.numel() * t.element_size() for t in hostW)
    d2h = host_out.numel() * host_out.element_size() + 4
    # what the host side of this box delivers when all ranks copy at once: the same bytes, copies only
    job.barrier()
    c0, c1 = ev(), ev()
    c0.record(copy_stream)
    for _ in range(4):
        e2e_copy(0)
    c1.record(copy_stream)
    job.barrier()
    copy_ms = job.max_over_ranks([c0.elapsed_time(c1) / 4])[0]
    return {"ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "h2d_only_ms_per_step": copy_ms, "h2d_gbs_per_gpu_all_ranks_copying": h2d / (copy_ms * 1e-3) / 1e9, "numa_node": numa}


def tokens_per_s(B, T, ranks, ms):
    return ranks * B * T / (ms * 1e-3)


def run_ours(args):
    job = Job(args)
    world, rank, dist = job.world, job.rank, job.dist
    function, B, T, N, D, f32 = WORKLOADS[args.workload]
    Gr, Gw, Gt, S = DIMS[function]
    # --shard batch (default): every rank runs the whole workload on its own batch shard (weak scaling; one all-reduce of
    # dR||db per step).  --shard heads: the ranks split the N independent heads of ONE workload (strong scaling, no
    # collective: dR/db stay sharded like R/b); the tokens of the job are B*T whatever the number of ranks.
    by_heads = args.shard == "heads" and world > 1
    if by_heads:
        if N % world:
            raise SystemExit(f"--shard heads needs the {N} heads of {args.workload} to divide by {world} ranks")
        N = N // world
    keep = {}
    head = measure(job, function, B, T, N, D, f32, allreduce=not by_heads, cluster_size=args.cluster_size,
                   batch_tile=args.batch_tile, keep=keep)
    e2e = measure_e2e(job, function, [keep[k] for k in ("Wx", "R", "b", "s0")], keep["gcnt"], allreduce=not by_heads)
    keep.clear()
    torch.cuda.empty_cache()

    # ---- the other benchmark configurations, same harness (device-resident inputs)
    extra = {}
    if not args.headline_only:
        def entry(m, Bw, Tw, ranks, **more):
            return {"value": tokens_per_s(Bw, Tw, ranks, m["ms_per_step"]), "unit": "tokens/s", **more, **m}

        if world == 1:
            for name in ("C3", "C4", "C5", "LB", "GB"):
                if name == args.workload:
                    continue
                fn, Bw, Tw, Nw, Dw, f32w = WORKLOADS[name]
                m = measure(job, fn, Bw, Tw, Nw, Dw, f32w, allreduce=False)
                extra[name] = entry(m, Bw, Tw, 1, workload=f"{fn} fwd+bwd B={Bw} T={Tw} N={Nw} D={Dw}, loss=sum(h)")
                torch.cuda.empty_cache()
        else:
            fn, Bw, Tw, Nw, Dw, f32w = WORKLOADS["C5"]
            solo = measure(job, fn, Bw, Tw, Nw, Dw, f32w, allreduce=False, group=False, floor=False) if rank == 0 else None
            job.barrier()
            solo_ms = job.max_over_ranks([solo["ms_per_step"] if solo else 0.0])[0]
            torch.cuda.empty_cache()
            m = measure(job, fn, Bw, Tw, Nw, Dw, f32w, allreduce=True, floor=False)
            extra["C5_weak"] = entry(m, Bw, Tw, world, workload=f"{fn} B={Bw} per GPU (global {Bw * world}) T={Tw} N={Nw} D={Dw}, "
                                     f"batch-sharded x{world}, NCCL all-reduce of dR||db", scaling="weak", one_gpu_ms_per_step=solo_ms,
                                     efficiency=solo_ms / m["ms_per_step"])
            torch.cuda.empty_cache()
            if Bw % world == 0:
                Bl = Bw // world
                strong = {}
                for label, bt in (("table", 0), ("rows128", 128), ("rows8", 8)):
                    try:
                        strong[label] = measure(job, fn, Bl, Tw, Nw, Dw, f32w, allreduce=True, floor=False, batch_tile=bt)
                    except Exception as e:  # noqa: BLE001 - a tile that does not exist for this shard size
                        strong[label] = {"unavailable": str(e)[:200]}
                    torch.cuda.empty_cache()
                m = strong["table"]
                extra["C5_strong"] = entry(m, Bl, Tw, world, workload=f"{fn} global B={Bw} ({Bl} per GPU) T={Tw} N={Nw} D={Dw}, "
                                           f"batch-sharded x{world}, NCCL all-reduce of dR||db", scaling="strong",
                                           one_gpu_ms_per_step=solo_ms, efficiency=solo_ms / (world * m["ms_per_step"]),
                                           other_tiles_ms_per_step={k: v.get("ms_per_step") for k, v in strong.items() if k != "table"})
            fn, Bw, Tw, Nw, Dw, f32w = WORKLOADS["C3"]
            if Nw % world == 0:
                solo = measure(job, fn, Bw, Tw, Nw, Dw, f32w, allreduce=False, group=False, floor=False) if rank == 0 else None
                job.barrier()
                solo_ms = job.max_over_ranks([solo["ms_per_step"] if solo else 0.0])[0]
                m = measure(job, fn, Bw, Tw, Nw // world, Dw, f32w, allreduce=False)
                extra["C3_heads"] = entry(m, Bw, Tw, 1, workload=f"{fn} B={Bw} T={Tw} D={Dw}, {Nw} heads split over {world} GPUs "
                                          f"({Nw // world} each), no collective", scaling="strong", one_gpu_ms_per_step=solo_ms,
                                          efficiency=solo_ms / (world * m["ms_per_step"]))
                torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    tok_ranks = 1 if by_heads else world  # ranks whose tokens add up (head shards work on the same tokens)
    ms = head["ms_per_step"]
    value = tokens_per_s(B, T, tok_ranks, ms)
    roof = head["roofline"]
    tr = NCU_TRAFFIC.get(args.workload) if (world == 1 and not args.cluster_size and not args.batch_tile and not job.f16 and not job.f32io) else None
    if tr:
        roof["traffic"], roof["traffic_source"] = tr["bytes"], tr["source"]
    nsteps = args.steps * head["blocks"]
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if by_heads else "weak",
        "vs_baseline": None,
        "dtype": "f32" if job.f32io else ("f16" if job.f16 else "bf16"), "data": "synthetic",
        "config": {"workload": f"{args.workload}: {function} fwd+bwd B={B} T={T} N={N} D={D} per GPU, loss=sum(h), "
                               f"states {'f32' if (f32 or job.f32io) else ('f16' if job.f16 else 'bf16')}", "global_batch": tok_ranks * B,
                   "parallelism": (f"head-sharded x{world} ({N} of {N * world} heads per GPU), no collective" if by_heads else
                                   f"batch-sharded x{world}, NCCL all-reduce of fp32 dR||db") if world > 1 else "single GPU",
                   "tile": head["tile"],
                   "timed_region": f"{head['blocks']} blocks of {args.steps} steps ({head['timed_seconds']:.2f} s); ms_per_step = median block, "
                                   f"max over ranks",
                   "l2": "working set per step (Wx+states+cache+dWx > 400 MB for C2) exceeds the 126 MB L2; no explicit flush"},
        "ms_per_step_best": head["ms_per_step_best"],
        "kernel_ms": head["kernel_ms"], "us_per_time_step": head["us_per_time_step"],
        "roofline": roof,
        "e2e": {"value": tokens_per_s(B, T, tok_ranks, e2e["ms_per_step"]), "unit": "tokens/s", **e2e},
        "gpu_launches": head["launches_per_step"] * nsteps,
        "clocks": head["clocks"],
    }
    rec = REFERENCE_GPU_RECORD.get(args.workload)
    if rec and world == 1:
        line["gpu_baseline"] = {**rec, "ratio": value / rec["value"]}
    if extra:
        line["workloads"] = extra
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = {k: v for k, v in cpu_sample(function, B, T, N, D).items() if k != "seconds"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--cluster-size", dest="cluster_size", type=int, default=0)
    ap.add_argument("--batch-tile", dest="batch_tile", type=int, default=0)
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="N > 1 GPUs: batch shards (weak scaling, default) or head shards of one workload (strong scaling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--headline-only", action="store_true", help="skip the `workloads` object (the other configurations)")
    ap.add_argument("--min-seconds", dest="min_seconds", type=float, default=0.5,
                    help="length of the timed region per workload (blocks of --steps steps are repeated until it is reached; "
                         "0 = three blocks, for runs under a profiler)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"],
                    help="element type of Wx/R/b/gradients (the baseline metric is quoted in bfloat16; float32 = the "
                         "accurate CUDA-core loops)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference_gpu":
        return run_reference_gpu(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
