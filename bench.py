#!/usr/bin/env python
"""Benchmark of the DDF forward at the ddf_resnet50 stage shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload op|model|backward|sfnorm|probe] [--detail PATH]

One "step" is the whole sweep: 7 stage shapes x {bf16, f16} x {mul, add} = 28
DDF forward calls at B = 128, k = 3, d = 1 (stride-1 shapes (C,H) = (64,56),
(128,28), (256,14), (512,7); stride-2 shapes (128,56), (256,28), (512,14)).
Inputs are seeded synthetic tensors: x ~ relu(N(0,1)), filters ~ N(0,1/9).

Prints ONE JSON line.  `value` is algorithmic GB moved per second over the
whole step with inputs resident in HBM, the step replayed from a CUDA graph and
timed with CUDA events; `e2e` is the same sweep through `ddf_host_async` with pinned
host buffers (host<->device copies inside the timed region); `roofline`
describes the kernel instance that takes the largest share of the step (against the
HBM roof and, in `fma_issue_roof`, against the issue rate of the mixed-precision FMA that
the library's probe kernel measures in the same run);
`cpu_baseline` is the CPU oracle (a port of the reference's arithmetic: the
reference has no CPU implementation) on a bounded sample.  With N > 1 every rank
runs the same sweep on its own GPU (the op shards along the batch with no
collective) and the value is the aggregate.

The same line also carries, beside the headline: `backward` (configs[2]: all three
gradients, 16 cases, GB/s and fraction of the HBM roofline per case), `model`
(ddf_mul_resnet50 inference, float16, GLOBAL batch 256 split over the N ranks, images/s),
`launch_floor_us` (an empty kernel replayed from a CUDA graph) and, per shape,
`floor_ratio` = (launch floor + bytes / peak) / measured time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(64, 56, 1), (128, 28, 1), (256, 14, 1), (512, 7, 1), (128, 56, 2), (256, 28, 2), (512, 14, 2)]
BATCH = 128
K, D = 3, 1
L2_BYTES = 126 * 1024 * 1024
MODEL_CFG = {"ddf_mul_resnet50": (torch.float16, 256), "ddf_add_resnet101": (torch.bfloat16, 512)}


def algorithmic_bytes(B, C, H, s, es, k=K):
    oh = H // s
    return es * (B * C * H * H + B * C * k * k + B * k * k * oh * oh + B * C * oh * oh)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_case(C, H, s, dtype, B, device, seed, k=K):
    g = torch.Generator().manual_seed(seed)
    oh = H // s
    x = torch.randn(B, C, H, H, generator=g).relu_().to(dtype)
    cf = (torch.randn(B, C, k, k, generator=g) / 3).to(dtype)
    sf = (torch.randn(B, k * k, oh, oh, generator=g) / 3).to(dtype)
    if device is None:
        return x, cf, sf
    return x.to(device), cf.to(device), sf.to(device)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.idx)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    p = [q.strip() for q in line.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        sm.append(float(p[1])); smax.append(float(p[2]))
                    except ValueError:
                        continue
                    for n, v in zip(names, p[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        hot = [v for v in sm if v >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(hot) if hot else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------ CPU legs
def cpu_sweep_seconds(sample_batch, threads=None, min_seconds=0.0):
    """Times the float32 CPU oracle over the sweep's 7 shapes x 2 modes at the given batch,
    repeating the whole sweep until `min_seconds` of CPU work have been timed.  Returns
    (seconds, 2-byte algorithmic bytes, threads used, repetitions)."""
    from oracle import ddf_oracle
    # All host cores unless told otherwise: torchrun exports OMP_NUM_THREADS=1 to its workers,
    # which would otherwise leave the CPU arm on a single thread.
    ddf_oracle.set_threads(threads or len(os.sched_getaffinity(0)))
    used = ddf_oracle.max_threads()
    inputs = [make_case(C, H, s, torch.float32, sample_batch, None, 10 + i) for i, (C, H, s) in enumerate(SHAPES)]
    for (x, cf, sf), (_C, _H, s) in zip(inputs, SHAPES):
        ddf_oracle.forward(x[:1], cf[:1], sf[:1], K, D, s, "mul")  # page in
    total_s, total_b, reps = 0.0, 0, 0
    while reps == 0 or total_s < min_seconds:
        for (x, cf, sf), (C, H, s) in zip(inputs, SHAPES):
            for mode in ("mul", "add"):
                t0 = time.perf_counter()
                ddf_oracle.forward(x, cf, sf, K, D, s, mode)
                total_s += time.perf_counter() - t0
                total_b += algorithmic_bytes(sample_batch, C, H, s, 2)
        reps += 1
    return total_s, total_b, used, reps


def run_reference(args, rank, world):
    """The reference has no CPU implementation of the op (its entry points raise on
    CPU tensors), so this arm times the CPU oracle -- a port of the reference's
    arithmetic -- on all host threads, on a bounded sample of the same sweep."""
    if rank != 0:
        return
    # one step = the full-size sweep (B = 128: 0.4 GB of float32 inputs per shape set, far larger
    # than the host caches); at least about five seconds of CPU work are timed in all
    sample_batch = BATCH
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_sweep_seconds(8)
    secs, nbytes, used, reps = 0.0, 0, 1, 0
    for i in range(args.steps):
        s_, b_, used, r_ = cpu_sweep_seconds(sample_batch, min_seconds=5.0 / args.steps)
        secs += s_; nbytes += b_; reps += r_
    gbs = nbytes / secs / 1e9
    line = {
        "impl": "reference", "metric": "ddf_forward_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (the CPU port has no 2-byte path; bytes counted at 2 bytes/element)",
        "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": used, "kind": "port",
                         "sample": f"7 shapes x (mul, add) at the full B={sample_batch}, float32, {reps} sweeps, "
                                   f"{secs:.1f} s, {os.cpu_count()} logical CPUs, OpenMP threads={used}"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def kernel_name(H, stride):
    """Which forward kernel serves a 2-byte sweep shape (see row_inst.inc: every shape of the sweep)."""
    return "row_kernel"


def workload_config():
    return {"workload": "configs[1]: DDF forward sweep at ddf_resnet50 stage shapes",
            "batch": BATCH, "kernel_size": K, "dilation": D,
            "shapes_C_H_stride": SHAPES, "io_dtypes": ["bf16", "f16"], "combine": ["mul", "add"],
            "calls_per_step": len(SHAPES) * 4,
            "l2": "inputs larger than L2: a step touches 0.87 GB of distinct tensors and the "
                  "two calls that share inputs (mul, add) are 13 calls (>0.4 GB) apart"}


# ------------------------------------------------------------------------------ GPU legs
def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from ddfnet_b200 import _lib, ddf
    from ddfnet_b200.host import ddf_host_async

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L = _lib.load()
    peak, peak_kind = peaks()

    # resident inputs, one set per (dtype, shape); outputs preallocated by the op
    cases = []  # (mode, dtname, C, H, s, x, cf, sf)
    tensors = {}
    for dtname, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        for i, (C, H, s) in enumerate(SHAPES):
            tensors[(dtname, C, H, s)] = make_case(C, H, s, dtype, BATCH, dev, 100 + i)
    for mode in ("mul", "add"):
        for dtname in ("bf16", "f16"):
            for (C, H, s) in SHAPES:
                cases.append((mode, dtname, C, H, s) + tensors[(dtname, C, H, s)])
    step_bytes = sum(algorithmic_bytes(BATCH, C, H, s, 2) for (_, _, C, H, s, *_r) in cases)

    def step():
        outs = []
        for (mode, _dt, _C, _H, s, x, cf, sf) in cases:
            outs.append(ddf(x, cf, sf, K, D, s, mode))
        return outs

    with torch.no_grad():
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        # the step as a CUDA graph: 28 launches replayed without host work between them
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            keep = step()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        torch.cuda.synchronize()

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        n0 = L.ddf_b200_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        elapsed_ms = e0.elapsed_time(e1)
        # graph replays do not pass through the library's host-side counter
        launches = (L.ddf_b200_launch_count() - n0) + args.steps * len(cases)

        # per-call durations: each call replayed alone from its own graph over rotating
        # buffer sets larger than L2, timed with CUDA events
        floor_us = launch_floor_us(L)
        # issue rate of the mixed-precision FMA (warp instructions per ns per SM), measured live by the
        # library's probe kernel: the second roof of the 2-byte stride-1 shapes (18 FMA operations per output)
        fma_rate = mixed_fma_rate(L, dev) if rank == 0 and not args.quick else None
        sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
        per_shape = []
        if rank == 0 and not args.quick:
            for (mode, dtname, C, H, s, x, cf, sf) in cases:
                nb = algorithmic_bytes(BATCH, C, H, s, 2)
                nsets = min(24, max(3, (2 * L2_BYTES) // nb + 2))
                sets = [(x, cf, sf)] + [(x.clone(), cf.clone(), sf.clone()) for _ in range(nsets - 1)]
                for st in sets:
                    ddf(*st, K, D, s, mode)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    held = [ddf(*st, K, D, s, mode) for st in sets]
                for _ in range(3):
                    g.replay()
                reps = 5
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(reps):
                    g.replay()
                b.record()
                torch.cuda.synchronize()
                us = a.elapsed_time(b) * 1e3 / (reps * nsets)
                per_shape.append({"C": C, "H": H, "stride": s, "dtype": dtname, "combine": mode,
                                  "us": round(us, 3), "bytes": nb, "gbs": round(nb / us / 1e3, 1),
                                  "frac": round(nb / us / 1e3 / peak, 4),
                                  "floor_ratio": round((floor_us + nb / peak / 1e3) / us, 4)})
                del g, held, sets
        clocks = sampler.stop() if rank == 0 else None

        # end to end through the host-buffer API: pinned inputs up, result down, every call
        e2e_steps = max(1, min(args.steps, 3))
        host_sets = {}
        for dtname, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16)):
            for i, (C, H, s) in enumerate(SHAPES):
                x, cf, sf = make_case(C, H, s, dtype, BATCH, None, 100 + i)
                oh = H // s
                # one output buffer per combine mode: the asynchronous calls of a step overlap
                host_sets[(dtname, C, H, s)] = (x.pin_memory(), cf.pin_memory(), sf.pin_memory(),
                                                {m: torch.empty(BATCH, C, oh, oh, dtype=dtype, pin_memory=True)
                                                 for m in ("mul", "add")})
        h2d = sum(sum(t.numel() * t.element_size() for t in v[:3]) for v in host_sets.values()) * 2
        d2h = sum(o.numel() * o.element_size() for v in host_sets.values() for o in v[3].values())

        def e2e_step():
            # the 28 calls of a step are issued asynchronously (uploads, kernels and downloads
            # of neighbouring calls overlap) and the step ends when every result is in host memory
            pending = []
            for (mode, dtname, C, H, s, *_r) in cases:
                hx, hcf, hsf, hout = host_sets[(dtname, C, H, s)]
                pending.append(ddf_host_async(hx, hcf, hsf, K, D, s, mode, out=hout[mode], device=dev))
            for h_ in pending:
                h_.wait()

        e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b.record()
        torch.cuda.synchronize()
        e2e_ms = max(a.elapsed_time(b), (time.perf_counter() - t0) * 1e3)

        # the copies alone (same pinned buffers, same bytes, no kernels): what the host side
        # of this box delivers to this rank while all ranks copy at once
        up = {k_: tuple(torch.empty_like(t, device=dev) for t in v[:3]) for k_, v in host_sets.items()}
        dn = {k_: {m: torch.empty_like(o, device=dev) for m, o in v[3].items()} for k_, v in host_sets.items()}
        s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

        def copy_step():
            with torch.cuda.stream(s_up):
                for _rep in range(2):          # every input set is uploaded once per combine mode
                    for k_, v in host_sets.items():
                        for src, dst in zip(v[:3], up[k_]):
                            dst.copy_(src, non_blocking=True)
            with torch.cuda.stream(s_dn):
                for k_, v in host_sets.items():
                    for m, o in v[3].items():
                        o.copy_(dn[k_][m], non_blocking=True)
            s_up.synchronize()
            s_dn.synchronize()

        copy_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            copy_step()
        copy_ms = (time.perf_counter() - t0) * 1e3
        del up, dn

    # configs[2] backward on rank 0 (the other ranks wait), then the model at global batch 256
    backward = None
    model = None
    if not args.quick:
        if rank == 0:
            backward = measure_backward(L, dev, peak, max(2, min(args.steps, 5)), with_sweep_shapes=False)
        if world > 1:
            dist.barrier()
        del graph, keep, tensors, cases
        torch.cuda.empty_cache()
        model = measure_model(rank, world, local_rank, "ddf_mul_resnet50", max(5, min(args.steps, 20)), 3)

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms, copy_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, copy_ms = t.tolist()
    if rank != 0:
        return

    ms_per_step = elapsed_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * step_bytes / (e2e_ms / e2e_steps * 1e-3) / 1e9
    copy_value = world * step_bytes / (copy_ms / e2e_steps * 1e-3) / 1e9

    # dominant kernel instance = largest share of the step
    roof = None
    if per_shape:
        dom = max(per_shape, key=lambda r: r["us"])
        roof = {"bound": "hbm",
                "kernel": f"{kernel_name(dom['H'], dom['stride'])} fwd C={dom['C']} H={dom['H']} "
                          f"s={dom['stride']} {dom['dtype']} {dom['combine']}",
                "achieved": dom["gbs"], "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                "frac": round(dom["gbs"] / peak, 4), "frac_of_8000": round(dom["gbs"] / 8000.0, 4),
                "traffic": None, "us_per_launch": dom["us"], "algorithmic_bytes": dom["bytes"]}
        if fma_rate:
            # the same launch against the FMA-issue roof: k*k taps x 2 FMA operations per output
            oh = dom["H"] // dom["stride"]
            ops = BATCH * dom["C"] * oh * oh * 2 * K * K
            fma_us = ops / 32 / (sm_count * fma_rate) / 1e3
            roof["fma_issue_roof"] = {"rate_warp_instr_per_ns_per_sm": fma_rate, "floor_us": round(fma_us, 2),
                                      "hbm_floor_us": round(dom["bytes"] / peak / 1e3, 2),
                                      "frac": round(fma_us / dom["us"], 4)}
        # DRAM bytes per launch of that kernel from the committed ncu capture, if any
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                tj = json.load(f)
            key = f"{dom['C']}x{dom['H']}s{dom['stride']}"
            if key in tj:
                roof["traffic"] = tj[key]

    cpu = None
    if not args.quick:
        cpu_sweep_seconds(8)
        secs, nbytes, used, reps = cpu_sweep_seconds(BATCH, min_seconds=10.0)
        cpu = {"value": round(nbytes / secs / 1e9, 3), "unit": "GB/s", "cores": used, "kind": "port",
               "sample": f"7 shapes x (mul, add) at the full B={BATCH}, float32 CPU oracle, {reps} sweeps, "
                         f"{secs:.1f} s, {os.cpu_count()} logical CPUs, OpenMP threads={used}"}

    line = {
        "metric": "ddf_forward_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16+f16 I/O, f32 arithmetic", "data": "synthetic",
        "config": workload_config(),
        "frac_of_measured_peak": round(value / world / peak, 4),
        "frac_of_8000": round(value / world / 8000.0, 4),
        "roofline": roof, "cpu_baseline": cpu,
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "per_rank_h2d_gbs": round(h2d / (e2e_ms / e2e_steps * 1e-3) / 1e9, 2),
                "per_rank_d2h_gbs": round(d2h / (e2e_ms / e2e_steps * 1e-3) / 1e9, 2),
                "copies_only": {"value": round(copy_value, 2), "unit": "GB/s",
                                "what": "the same pinned-buffer uploads and downloads with no kernels, all ranks "
                                        "at once: the ceiling the host side of this box sets",
                                "e2e_over_copies_only": round(e2e_value / copy_value, 3)}},
        "launch_floor_us": round(floor_us, 3) if per_shape else None,
        "backward": backward, "model": model,
        "gpu_launches": int(launches), "clocks": clocks,
        "per_shape": per_shape,
    }
    print(json.dumps(line))
    if args.detail:
        with open(args.detail, "w") as f:
            json.dump(line, f, indent=1)


def measure_backward(L, dev, peak, steps, with_sweep_shapes=True):
    """configs[2]: DDF backward (all three gradients) at B=64, C=256, 28x28, k in
    {3, 5}, d in {1, 2}, stride 1, mul and add, float32 and bfloat16, through the
    C ABI with caller-allocated outputs and workspace.  Per case: its own CUDA
    graph over rotating buffer sets larger than L2, CUDA events."""
    from ddfnet_b200 import _lib
    B, C, H = 64, 256, 28
    rows, total_bytes, total_us = [], 0, 0.0

    def time_case(Bc, Cc, Hc, k, d, s2, comb, dtc, dtype, es, seed):
        oh = Hc // s2
        g = torch.Generator().manual_seed(seed)
        mk = lambda *shape: torch.randn(*shape, generator=g)
        base = (mk(Bc, Cc, oh, oh), mk(Bc, Cc, Hc, Hc).relu_(), mk(Bc, Cc, k, k) / 3, mk(Bc, k * k, oh, oh) / 3)
        nb = es * (Bc * Cc * oh * oh + 2 * Bc * Cc * Hc * Hc + 2 * Bc * Cc * k * k + 2 * Bc * k * k * oh * oh)
        nsets = max(3, (2 * L2_BYTES) // nb + 2)
        sets = []
        for _ in range(nsets):
            go, x, cf, sf = (t.to(dev, dtype) for t in base)
            sets.append((go, x, cf, sf, torch.empty_like(x), torch.empty_like(cf), torch.empty_like(sf)))
        out = {}
        for mode, cmb in comb:
            wsb = int(L.ddf_b200_backward_workspace(Bc, Cc, Hc, Hc, k, d, s2, cmb, dtc, _lib.VARIANT_AUTO))
            ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)

            def call(st):
                go, x, cf, sf, gx, gcf, gsf = st
                _lib.check(L.ddf_b200_backward(
                    go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(), gx.data_ptr(),
                    gcf.data_ptr(), gsf.data_ptr(), ws.data_ptr(), wsb, Bc, Cc, Hc, Hc, k, d, s2, cmb,
                    dtc, _lib.VARIANT_AUTO, torch.cuda.current_stream().cuda_stream))

            for st in sets:
                call(st)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for st in sets:
                    call(st)
            for _ in range(3):
                gr.replay()
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            for _ in range(steps):
                gr.replay()
            b_.record()
            torch.cuda.synchronize()
            out[mode] = (a_.elapsed_time(b_) * 1e3 / (steps * nsets), nb, wsb)
            del gr
        del sets
        return out

    for dtname, dtype, dtc in (("f32", torch.float32, _lib.F32), ("bf16", torch.bfloat16, _lib.BF16)):
        es = 4 if dtname == "f32" else 2
        for k in (3, 5):
            for d in (1, 2):
                res = time_case(B, C, H, k, d, 1, (("mul", _lib.MUL), ("add", _lib.ADD)), dtc, dtype, es, 300 + k + d)
                for mode, (us, nb, _w) in res.items():
                    rows.append({"dtype": dtname, "k": k, "d": d, "combine": mode, "us": round(us, 2),
                                 "bytes": nb, "gbs": round(nb / us / 1e3, 1),
                                 "frac": round(nb / us / 1e3 / peak, 4)})
                    total_bytes += nb
                    total_us += us
    # The sweep's own shapes (bf16, mul, k = 3), not part of `value`.
    shape_rows = []
    if with_sweep_shapes:
        for (C2, H2, s2) in SHAPES:
            res = time_case(B, C2, H2, 3, 1, s2, (("mul", _lib.MUL),), _lib.BF16, torch.bfloat16, 2, 700 + C2 + s2)
            us, nb, wsb = res["mul"]
            shape_rows.append({"C": C2, "H": H2, "stride": s2, "us": round(us, 1), "gbs": round(nb / us / 1e3, 1),
                               "frac": round(nb / us / 1e3 / peak, 4),
                               "filter_gradients": "streaming" if wsb > 0 else "generic"})
    return {"value": round(total_bytes / total_us / 1e3, 1), "unit": "GB/s",
            "workload": "configs[2]: DDF backward, B=64, C=256, 28x28, k 3/5, d 1/2, mul/add, f32 + bf16; "
                        "rotating buffer sets larger than L2",
            "ms_all_cases": round(total_us / 1e3, 4), "min_frac": min(r["frac"] for r in rows),
            "frac": round(total_bytes / total_us / 1e3 / peak, 4),
            "per_case": rows, "sweep_shapes_bf16_mul_B64": shape_rows}


def run_backward(args, rank, world, local_rank):
    from ddfnet_b200 import _lib
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L = _lib.load()
    peak, peak_kind = peaks()
    r = measure_backward(L, dev, peak, args.steps)
    if rank == 0:
        print(json.dumps({
            "metric": "ddf_backward_hbm_gbs", "value": r["value"], "unit": "GB/s",
            "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": r["ms_all_cases"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32+bf16 I/O, f32 arithmetic", "data": "synthetic",
            "config": {"workload": r["workload"]},
            "peak": peak, "peak_kind": f"of {peak_kind}", "min_frac": r["min_frac"], "per_case": r["per_case"],
            "sweep_shapes_bf16_mul_B64": r["sweep_shapes_bf16_mul_B64"]}))


def run_sfnorm(args, rank, world, local_rank):
    """Forward with the spatial FilterNorm fused into the kernel (ddf_sfnorm) against the
    module sequence it replaces (FilterNorm as torch ops, then ddf), at the sweep's shapes."""
    from ddfnet_b200 import ddf, ddf_sfnorm
    from ddfnet_b200.modules import FilterNorm
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peak, peak_kind = peaks()
    rows = []
    scale = 2.0 ** 0.5 / K
    norm = FilterNorm(1, K, "spatial", "relu")
    for (C, H, s) in SHAPES:
        for dtname in ("bf16", "f16"):
            dtype = {"bf16": torch.bfloat16, "f16": torch.float16}[dtname]
            nb = algorithmic_bytes(BATCH, C, H, s, 2)
            nsets = max(3, (2 * L2_BYTES) // nb + 2)
            sets = [make_case(C, H, s, dtype, BATCH, dev, 500 + i) for i in range(nsets)]
            times = {}
            for label, fn in (("fused", lambda x, cf, raw: ddf_sfnorm(x, cf, raw, K, 1, s, "mul", scale)),
                              ("module_sequence", lambda x, cf, raw: ddf(x, cf, norm(raw), K, 1, s, "mul"))):
                with torch.no_grad():
                    for st in sets:
                        fn(st[0], st[1], st[2])
                    torch.cuda.synchronize()
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        for st in sets:
                            fn(st[0], st[1], st[2])
                    for _ in range(3):
                        gr.replay()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(args.steps):
                        gr.replay()
                    b.record()
                    torch.cuda.synchronize()
                    times[label] = a.elapsed_time(b) * 1e3 / (args.steps * nsets)
            rows.append({"C": C, "H": H, "stride": s, "dtype": dtname, "bytes": nb,
                         "fused_us": round(times["fused"], 2),
                         "module_sequence_us": round(times["module_sequence"], 2),
                         "fused_gbs": round(nb / times["fused"] / 1e3, 1)})
            del sets
    tot_b = sum(r["bytes"] for r in rows)
    tot_f = sum(r["fused_us"] for r in rows)
    tot_m = sum(r["module_sequence_us"] for r in rows)
    if rank == 0:
        print(json.dumps({
            "metric": "ddf_forward_sfnorm_hbm_gbs", "value": round(tot_b / tot_f / 1e3, 1), "unit": "GB/s",
            "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": round(tot_f / 1e3, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16+f16 I/O, f32 arithmetic", "data": "synthetic",
            "config": {"workload": "DDF forward with the spatial FilterNorm fused, sweep shapes, mul, B=128",
                       "l2": "rotating buffer sets larger than L2"},
            "module_sequence_ms_per_step": round(tot_m / 1e3, 4),
            "peak": peak, "peak_kind": f"of {peak_kind}", "per_shape": rows}))


def run_nhwc(args, rank, world, local_rank):
    """Per-layer sweep of the channels_last forward as the network harness calls it: raw 16-map
    spatial-filter tensor, bias + FilterNorm + per-channel scale/shift + ReLU inside the kernel.
    Bytes are the sweep's algorithmic bytes (9 filter maps); the kernel reads the 16-map tensor."""
    from ddfnet_b200.nhwc import ddf_nhwc
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peak, peak_kind = peaks()
    rows = []
    scale = 2.0 ** 0.5 / K
    for mode in ("mul", "add"):
        for (C, H, s) in SHAPES:
            for dtname in ("bf16", "f16"):
                dtype = {"bf16": torch.bfloat16, "f16": torch.float16}[dtname]
                nb = algorithmic_bytes(BATCH, C, H, s, 2)
                nsets = max(3, (2 * L2_BYTES) // nb + 2)
                sets = []
                for i in range(nsets):
                    x, cf, sf = make_case(C, H, s, dtype, BATCH, dev, 700 + i)
                    sf16 = torch.zeros(sf.shape[0], 16, sf.shape[2], sf.shape[3], dtype=dtype, device=dev)
                    sf16[:, :K * K] = sf
                    sets.append((x.contiguous(memory_format=torch.channels_last), cf,
                                 sf16.contiguous(memory_format=torch.channels_last)))
                bias = torch.zeros(K * K, dtype=torch.float32, device=dev)
                osc = torch.ones(C, dtype=torch.float32, device=dev)
                osh = torch.zeros(C, dtype=torch.float32, device=dev)

                def fn(st):
                    return ddf_nhwc(st[0], st[1], st[2], K, 1, s, mode, sf_bias=bias, sf_norm_scale=scale,
                                    out_scale=osc, out_shift=osh, relu=True)
                with torch.no_grad():
                    for st in sets:
                        fn(st)
                    torch.cuda.synchronize()
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        for st in sets:
                            fn(st)
                    for _ in range(3):
                        gr.replay()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(args.steps):
                        gr.replay()
                    b.record()
                    torch.cuda.synchronize()
                us = a.elapsed_time(b) * 1e3 / (args.steps * nsets)
                rows.append({"C": C, "H": H, "stride": s, "dtype": dtname, "combine": mode, "bytes": nb,
                             "us": round(us, 2), "gbs": round(nb / us / 1e3, 1),
                             "frac": round(nb / us / 1e3 / peak, 4)})
                del sets
    tot_b = sum(r["bytes"] for r in rows)
    tot_t = sum(r["us"] for r in rows)
    if rank == 0:
        print(json.dumps({
            "metric": "ddf_forward_nhwc_hbm_gbs", "value": round(tot_b / tot_t / 1e3, 1), "unit": "GB/s",
            "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": round(tot_t / 1e3, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16+f16 I/O, f32 arithmetic", "data": "synthetic",
            "config": {"workload": "channels_last DDF forward with bias, FilterNorm, scale/shift and ReLU fused, "
                                   "sweep shapes, mul and add, B=128",
                       "l2": "rotating buffer sets larger than L2"},
            "peak": peak, "peak_kind": f"of {peak_kind}", "per_shape": rows}))


def measure_model(rank, world, local_rank, name, steps, warmup, channels_last=True, fold_bn="fused",
                  unfused_norm=False, no_graph=False):
    """Whole-network inference throughput (images/s) of the DDF-ResNet harness at the
    model's GLOBAL batch, batch-sharded over the ranks (strong scaling); logits are
    all-gathered once, outside the timed region, for checking."""
    import torch.distributed as dist
    from ddfnet_b200.resnet import MODELS
    from ddfnet_b200.shard import batch_slice, gather_batch

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dtype, gbatch = MODEL_CFG[name]
    lo, hi = batch_slice(gbatch, rank, world)
    torch.manual_seed(0)
    model = MODELS[name]().to(dev).eval()
    if fold_bn:
        from ddfnet_b200.resnet import fold_batchnorm
        fold_batchnorm(model, fuse_activations=fold_bn == "fused")
    model = model.to(dtype)
    if channels_last:
        model = model.to(memory_format=torch.channels_last)
    for m in model.ddf_layers():
        m.fuse_filter_norm = not unfused_norm
        m.fuse_channel_branch = not unfused_norm
    g = torch.Generator().manual_seed(1)
    x = torch.randn(gbatch, 3, 224, 224, generator=g)[lo:hi].to(dev, dtype)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        for _ in range(max(warmup, 3)):
            y = model(x)
        torch.cuda.synchronize()
        # The whole network as one CUDA graph: at 32 images per GPU the ~300 small
        # kernels of a forward pass are otherwise bound by launch overhead.
        graphed = False
        if not no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    model(x)
                torch.cuda.current_stream().wait_stream(side)
                with torch.cuda.graph(graph):
                    y = model(x)
                graph.replay()
                torch.cuda.synchronize()
                graphed = True
            except Exception as e:  # fall back to eager launches
                print(f"# graph capture failed, timing eager launches: {e}", file=sys.stderr)
        run = graph.replay if graphed else (lambda: model(x))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            run()
        b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = a.elapsed_time(b)
        if not graphed:
            y = model(x)
        logits = gather_batch(y.float(), gbatch)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    return {"name": name, "images_per_s": round(gbatch * steps / (ms * 1e-3), 1), "global_batch": gbatch,
            "per_gpu_batch": hi - lo, "ms_per_step": round(ms / steps, 3), "steps": steps,
            "dtype": str(dtype).replace("torch.", ""), "scaling": "strong", "cuda_graph": graphed,
            "flags": {"filter_branches": "reference module sequence (torch ops)" if unfused_norm
                      else "spatial FilterNorm fused into the DDF kernel, channel branch as one kernel",
                      "memory_format": "channels_last around the DDF layers" if channels_last else "NCHW",
                      "batchnorm": {None: "as built", "plain": "folded into the preceding convolutions",
                                    "fused": "folded; conv+bias(+shortcut)+ReLU as single cuDNN calls"}[fold_bn]},
            "logits_finite": bool(torch.isfinite(logits).all()), "logits_shape": list(logits.shape)}


def run_model(args, rank, world, local_rank):
    r = measure_model(rank, world, local_rank, args.model, args.steps, args.warmup, args.channels_last,
                      args.fold_bn, args.unfused_norm, args.no_graph)
    if rank == 0:
        print(json.dumps({
            "metric": f"{r['name']}_images_per_s", "value": r["images_per_s"],
            "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": r["dtype"], "data": "synthetic",
            "config": {"workload": f"{r['name']} inference, global batch {r['global_batch']}, 224x224, random init",
                       "per_gpu_batch": r["per_gpu_batch"], "cuda_graph": r["cuda_graph"], **r["flags"]},
            "logits_finite": r["logits_finite"], "logits_shape": r["logits_shape"]}))


def launch_floor_us(L, reps=200):
    """Time per launch of an empty kernel replayed from a CUDA graph."""
    g = torch.cuda.CUDAGraph()
    stream = torch.cuda.current_stream()
    L.ddf_b200_noop(stream.cuda_stream)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        for _ in range(50):
            L.ddf_b200_noop(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        g.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps // 50):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps // 50 * 50)


def mixed_fma_rate(L, dev):
    """Issue rate of fma.rn.f32.bf16 (three distinct register operands), warp instructions per ns per SM."""
    import ctypes
    from ddfnet_b200 import _lib
    nbytes = int(L.ddf_b200_rate_probe_bytes())
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    v = ctypes.c_double(0.0)
    _lib.check(L.ddf_b200_rate_probe(2, scratch.data_ptr(), nbytes, 1024, ctypes.byref(v),
                                     torch.cuda.current_stream().cuda_stream))
    return round(v.value, 3)


def run_probe(args, rank, world, local_rank):
    """Instruction issue rates and the launch floor (the numbers the roofline discussion uses)."""
    import ctypes
    from ddfnet_b200 import _lib
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L = _lib.load()
    nbytes = int(L.ddf_b200_rate_probe_bytes())
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    names = ["ffma_repeated_multiplicands", "ffma_three_distinct_registers", "mixed_fma_bf16", "mixed_fma_f16",
             "fma_f32x2", "lop3"]
    rates = {}
    for mode, nm in enumerate(names):
        v = ctypes.c_double(0.0)
        _lib.check(L.ddf_b200_rate_probe(mode, scratch.data_ptr(), nbytes, 1024, ctypes.byref(v),
                                         torch.cuda.current_stream().cuda_stream))
        rates[nm] = round(v.value, 3)
    if rank == 0:
        print(json.dumps({"metric": "warp_instructions_per_ns_per_sm", "rates": rates,
                          "launch_floor_us": round(launch_floor_us(L), 3),
                          "note": "4 schedulers per SM at 1.965 GHz issue at most 7.86 warp instructions per ns"}))


def run_ncu_case(spec):
    """C,H,stride,dtype,combine followed by any of: backward, nhwc, k=5, d=2."""
    from ddfnet_b200 import ddf
    parts = spec.split(",")
    C, H, s = int(parts[0]), int(parts[1]), int(parts[2])
    dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[parts[3]]
    mode = parts[4]
    flags = parts[5:]
    backward, nhwc = "backward" in flags, "nhwc" in flags
    k = next((int(f[2:]) for f in flags if f.startswith("k=")), K)
    d = next((int(f[2:]) for f in flags if f.startswith("d=")), D)
    dev = torch.device("cuda:0")
    B = 64 if backward else BATCH
    sets = [make_case(C, H, s, dtype, B, dev, 7 + i, k=k) for i in range(3)]
    if backward:
        go = torch.randn(B, C, H // s, H // s, device=dev).to(dtype)
        for i in range(6):
            xs = [t.detach().requires_grad_() for t in sets[i % 3]]
            ddf(*xs, k, d, s, mode).backward(go)
    elif nhwc:
        # channels_last input and spatial filter (the filter's tap axis padded to 16, as the
        # spatial branch's convolution produces it): the layout-native kernel
        from ddfnet_b200.nhwc import ddf_nhwc
        cl = []
        for x, cf, sf in sets:
            sf16 = torch.zeros(sf.shape[0], 16, sf.shape[2], sf.shape[3], dtype=sf.dtype, device=dev)
            sf16[:, :k * k] = sf
            cl.append((x.contiguous(memory_format=torch.channels_last), cf,
                       sf16.contiguous(memory_format=torch.channels_last)))
        for i in range(6):
            ddf_nhwc(*cl[i % 3], k, d, s, mode)
    else:
        with torch.no_grad():
            for i in range(6):
                ddf(*sets[i % 3], k, d, s, mode)
    torch.cuda.synchronize()
    print("ok")


def run_model_reference(args, rank, world):
    """CPU baseline of the whole-network workload: the same nn.Module in float32 on
    the host cores, with the DDF op served by the CPU oracle's unfold composite (a
    port: the reference has no CPU op).  Reduced batch, stated in the line."""
    if rank != 0:
        return
    import ddfnet_b200.modules as modules
    from ddfnet_b200.resnet import MODELS
    from oracle import ddf_oracle

    name = args.model
    batch = 8
    torch.set_num_threads(len(os.sched_getaffinity(0)))  # launchers may export OMP_NUM_THREADS=1
    orig = modules.ddf
    modules.ddf = lambda x, cf, sf, k, d, s, comb: ddf_oracle.composite_forward(x, cf, sf, k, d, s, comb)
    try:
        torch.manual_seed(0)
        model = MODELS[name]().eval()
        for m in model.ddf_layers():   # the reference's module sequence, op by op
            m.fuse_filter_norm = False
            m.fuse_channel_branch = False
        x = torch.randn(batch, 3, 224, 224, generator=torch.Generator().manual_seed(1))
        with torch.no_grad():
            for _ in range(max(1, min(args.warmup, 1))):
                model(x)
            t0 = time.perf_counter()
            steps = max(1, min(args.steps, 3))
            for _ in range(steps):
                model(x)
            secs = time.perf_counter() - t0
    finally:
        modules.ddf = orig
    val = batch * steps / secs
    print(json.dumps({
        "impl": "reference", "metric": f"{name}_images_per_s", "value": round(val, 2), "unit": "images/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": round(secs / steps * 1e3, 1),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "float32",
        "data": "synthetic",
        "config": {"workload": f"{name} inference on CPU, batch {batch}, 224x224, random init"},
        "cpu_baseline": {"value": round(val, 2), "unit": "images/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": f"batch {batch}, float32, {os.cpu_count()} logical CPUs"},
        "e2e": {"value": round(val, 2), "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="op", choices=["op", "model", "backward", "sfnorm", "nhwc", "probe"])
    ap.add_argument("--model", default="ddf_mul_resnet50", choices=sorted(MODEL_CFG))
    ap.add_argument("--quick", action="store_true",
                    help="op workload: skip the per-call timings and the CPU baseline (scaling runs)")
    ap.add_argument("--no-graph", action="store_true", help="model workload: eager launches")
    ap.add_argument("--unfused-norm", action="store_true",
                    help="model workload: run both filter branches as the reference's module sequence "
                         "(FilterNorm and the channel branch as separate torch ops)")
    ap.add_argument("--channels-last", action="store_true",
                    help="model workload: convolutions in channels_last; each DDFPack converts to NCHW and back")
    ap.add_argument("--fold-bn", nargs="?", const="plain", default=None, choices=["plain", "fused"],
                    help="model workload: fold every BatchNorm that follows a convolution into it; "
                         "'fused' also uses cuDNN's fused conv+bias(+add)+ReLU calls")
    ap.add_argument("--detail", default=None, help="also write the JSON, indented, to this file")
    ap.add_argument("--ncu-case", default=None, metavar="C,H,stride,dtype,combine[,backward][,nhwc][,k=5][,d=2]",
                    help="profiling aid: run only this case, 6 launches over 3 rotating buffer "
                         "sets at B=128 (B=64 for backward), print nothing but 'ok'")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if args.workload == "model":
            run_model_reference(args, rank, world)
        else:
            run_reference(args, rank, world)
        return
    if args.ncu_case:
        run_ncu_case(args.ncu_case)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the op)")
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "model":
            run_model(args, rank, world, local_rank)
        elif args.workload == "backward":
            run_backward(args, rank, world, local_rank)
        elif args.workload == "sfnorm":
            run_sfnorm(args, rank, world, local_rank)
        elif args.workload == "nhwc":
            run_nhwc(args, rank, world, local_rank)
        elif args.workload == "probe":
            run_probe(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
