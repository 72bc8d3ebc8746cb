#!/usr/bin/env python
"""Benchmark of the recurrent hot path: fwd+bwd tokens/s (B*T per second) of the LSTM headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C2|C3|C4|C5] [--impl ours|reference]

One JSON line on stdout (rank 0).  A "step" is one forward + backward pass of the whole sequence:
frnn_forward + frnn_backward + frnn_finalize_grads through the C ABI on device-resident buffers (`value`),
and the same step through the public `flashrnn()` API with pinned HOST inputs, host->device copies and a
device->host read of the gradients inside the timed region (`e2e`).  With N > 1 every rank runs the workload on
its own batch shard (weak scaling: global batch = N x workload batch) and the fp32 dR || db are all-reduced with
NCCL inside the step.  `--impl reference` times the CPU restatement of the reference's `vanilla` backend
(oracle/vanilla_port.py) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
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
}
DIMS = {"lstm": (4, 4, 4, 2), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1), "slstm": (4, 4, 4, 4)}
METRIC = "fwd+bwd tokens/sec (B*T/s)"
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the reverse time loop, from an `ncu --set full` capture
# of this command on a B200 (summary: profiles/ncu_full_C2_kernels.md).  Only workloads that were captured are listed.
NCU_TRAFFIC_BYTES = {"C2": 237_129_984 + 105_455_360}


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1407.4))), "measured"
    return 6650.0, 1400.0, "fallback"


def make_inputs(function, B, T, N, D, f32_states, device, seed=0, edt=torch.bfloat16):
    """Seeded synthetic inputs with the shapes and distributions of the named configuration (``edt``: the 16-bit type)."""
    Gr, Gw, Gt, S = DIMS[function]
    g = torch.Generator(device="cpu").manual_seed(seed)
    Wx = torch.randn(B, T, Gw, N, D, generator=g).to(edt)
    R = (torch.randn(Gr, N, D, D, generator=g) / D ** 0.5).to(edt)
    b = 0.1 * torch.randn(Gt, N, D, generator=g)
    if function == "gru":
        b.zero_()
    if function == "slstm":
        b.zero_()
        b[1] = 3.0 + 3.0 * torch.rand(N, D, generator=g)
    b = b.to(edt)
    sdt = torch.float32 if f32_states else edt
    s0 = (0.1 * torch.randn(S, B, 1, N, D, generator=g) if function == "lstm" else torch.zeros(S, B, 1, N, D)).to(sdt)
    return [t.to(device) if device != "cpu" else t for t in (Wx, R, b, s0)]


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
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[gpu_index]) if visible and visible.split(",")[gpu_index].isdigit() else gpu_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
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


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args):
    from flashrnn_b200 import _native as nv
    from flashrnn_b200 import flashrnn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: flashrnn_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

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
    f16 = args.dtype == "float16"
    edt = torch.float16 if f16 else torch.bfloat16
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, f32, dev, seed=rank, edt=edt)
    sdt = torch.float32 if f32 else edt
    esz, ssz = 2, (4 if f32 else 2)
    E = B * T * N * D

    # ---- C-ABI step on resident buffers
    prob = nv.make_problem(function, B, T, N, D, f32, True, f16=f16)
    plan = nv.query(prob, args.cluster_size, args.batch_tile)
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
    stream = torch.cuda.current_stream(dev)
    sp = ctypes.c_void_p(stream.cuda_stream)
    fa = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), P(ws))
    ba = nv.FrnnBwdArgs(P(R), P(s0), P(states), P(cache), P(dstates), P(dWx), P(ds0), P(ws))
    L = nv.lib()
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step(rec=None):
        if rec: rec[0].record(stream)
        nv.check("frnn_forward", L.frnn_forward(ctypes.byref(plan), ctypes.byref(fa), sp))
        if rec: rec[1].record(stream)
        nv.check("frnn_backward_parts", L.frnn_backward_parts(ctypes.byref(plan), ctypes.byref(ba), sp, 1))
        if rec: rec[2].record(stream)
        nv.check("frnn_backward_parts", L.frnn_backward_parts(ctypes.byref(plan), ctypes.byref(ba), sp, 2))
        if rec: rec[3].record(stream)
        if dist is not None and not by_heads:
            dist.all_reduce(grads)
        nv.check("frnn_finalize_grads", L.frnn_finalize_grads(ctypes.byref(plan), P(grads), P(dR), P(db), sp))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    recs = [[ev() for _ in range(4)] for _ in range(args.steps)]
    e0, e1 = ev(), ev()
    with ClockSampler(local) as clk:
        barrier()
        e0.record(stream)
        for i in range(args.steps):
            step(recs[i])
        e1.record(stream)
        barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    st = nv.FrnnDevStatus()
    nv.check("frnn_read_device_status", L.frnn_read_device_status(P(ws), sp, ctypes.byref(st)))
    if st.code != 0:
        raise RuntimeError(f"device-side wait expired (step {st.where}, cta {st.cta}); results invalid")
    fwd_ms = sum(r[0].elapsed_time(r[1]) for r in recs) / args.steps
    bwd_ms = sum(r[1].elapsed_time(r[2]) for r in recs) / args.steps
    dr_ms = sum(r[2].elapsed_time(r[3]) for r in recs) / args.steps

    # ---- end to end through the public API with host inputs
    hostW = [t.cpu().pin_memory() for t in (Wx, R, b, s0)]
    host_out = torch.empty(gcnt, dtype=edt).pin_memory()
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()

    # Inputs are double-buffered on the device: the H2D copy of step i+1 (own stream) overlaps the kernels of step i,
    # as an input pipeline with pinned memory does; every step's inputs still cross PCIe inside the timed region.
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [[torch.empty_like(t) for t in (Wx, R, b, s0)] for _ in range(2)]
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
                          grad_allreduce_group=(True if dist is not None and not by_heads else None))
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
    barrier()
    k2 = max(1, min(args.steps, 10))
    e2, e3 = ev(), ev()
    e2.record(stream)
    e2e_run(k2, e2)
    e3.record(stream)
    barrier()
    e2e_ms = e2.elapsed_time(e3) / k2
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = sum(t.numel() * t.element_size() for t in hostW)
    d2h = host_out.numel() * 2 + 4

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    hbm_peak, tc_peak, which = measured_peaks()
    tok_ranks = 1 if by_heads else world  # ranks whose tokens add up (head shards work on the same tokens)
    # algorithmic traffic of the dominant kernel (the reverse time loop): reads dstates and states, writes dWx
    bwd_bytes = E * (S * ssz + S * ssz + Gw * esz)
    fwd_bytes = E * (Gw * esz + S * ssz)
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    wide = plan.batch_tile == 128  # tcgen05 loops: forward, reverse loop (with dR and db inside), cast = 3 launches per step
    line = {
        "metric": METRIC, "value": tok_ranks * B * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if by_heads else "weak",
        "vs_baseline": None,
        "dtype": "f16" if f16 else "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {function} fwd+bwd B={B} T={T} N={N} D={D} per GPU, loss=sum(h), "
                               f"states {'f32' if f32 else ('f16' if f16 else 'bf16')}", "global_batch": tok_ranks * B,
                   "parallelism": (f"head-sharded x{world} ({N} of {N * world} heads per GPU), no collective" if by_heads else
                                   f"batch-sharded x{world}, NCCL all-reduce of fp32 dR||db") if world > 1 else "single GPU",
                   "tile": {"cluster_size": plan.cluster_size, "units_per_cta": plan.units_per_cta, "batch_tile": plan.batch_tile,
                            "threads": plan.threads},
                   "l2": "working set per step (Wx+states+cache+dWx > 400 MB for C2) exceeds the 126 MB L2; no explicit flush"},
        "kernel_ms": {"forward_loop": fwd_ms, "backward_loop": bwd_ms, "recurrent_grad": dr_ms},
        "us_per_time_step": {"forward": 1e3 * fwd_ms / T, "backward": 1e3 * bwd_ms / T},
        "roofline": {"bound": "hbm", "kernel": "wide_bwd_elman_kernel (reverse time loop, dR and db inside)" if wide
                     else "frnn_bwd_kernel (reverse time loop)", "achieved": achieved, "peak": hbm_peak,
                     "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": which, "traffic": None,
                     "algorithmic_bytes_per_launch": bwd_bytes,
                     "forward_loop": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "algorithmic_bytes_per_launch": fwd_bytes},
                     "tensor_frac_whole_step": (6.0 * E * Gr * D / (ms * 1e-3) / 1e12) / tc_peak,
                     "note": "streams one 16 KB tile per operand, step and CTA; HBM-bound" if wide else
                     "the serial chain of 2T dependent steps, not HBM or the tensor pipe, bounds this workload"},
        "e2e": {"value": tok_ranks * B * T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": (3 if wide else 6) * args.steps,
        "clocks": clk.summary(),
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = {k: v for k, v in cpu_sample(function, B, T, N, D).items() if k != "seconds"}
    line["roofline"]["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--cluster-size", dest="cluster_size", type=int, default=0)
    ap.add_argument("--batch-tile", dest="batch_tile", type=int, default=0)
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="N > 1 GPUs: batch shards (weak scaling, default) or head shards of one workload (strong scaling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16"],
                    help="16-bit element type of Wx/R/b/gradients (the baseline metric is quoted in bfloat16)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
