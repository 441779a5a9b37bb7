#!/usr/bin/env python
"""Benchmark of the fused Conv2D path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

A *step* is one forward pass of the hot path over one batch of synthetic input: layout repack + weight prepack +
tensor-core convolution with fused bias + ReLU (exactly what one gie::Conv2D::forward call does).  The default
workload is the FP16 3x3 convolution the headline metric is quoted on (N=32, C=256, 14x14, K=256).  With N GPUs every
rank runs the same work on its own replica (weak scaling, no collective on the data path); the reported value is the
whole-job TFLOP/s = N * K * FLOPs / max-over-ranks device time.  One JSON line is printed by rank 0.

`--impl reference` times the reference library's own CPU convolution (oracle/_ref, or the C restatement when the
reference could not be compiled) on the host cores for the same metric; that is the only place besides the
`cpu_baseline` leg where anything under oracle/ is executed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures summarised
# under profiles/ (None where no capture exists yet).
NCU_TRAFFIC_BYTES = {"c2": 4470784,             # profiles/conv_tc_kernel_c2_fp16.md
                     "c3_fp16": 51898880}       # profiles/conv_tc_kernel_c3_fp16.md

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and all(t.strip().isdigit() for t in vis.split(",")) else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr is not None:
            self._stop.set()
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def time_rmsnorm(torch, pkg, steps, warmup):
    """Fused residual-add + RMSNorm, BF16 8192 x 4096, FP32 gamma = 1 + N(0, 0.02): GB/s of algorithmic bytes (x and
    residual in, residual and y out).  Buffers rotate over more than L2."""
    from cuda_inference_b200 import workloads as wl
    cfg = wl.RMSNORM_WORKLOAD
    rows, hidden = cfg["rows"], cfg["hidden"]
    n = rows * hidden
    nsets = 3  # 3 x 268 MB
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    sets = [(torch.randn(n, device="cuda", generator=g).to(torch.bfloat16), torch.randn(n, device="cuda", generator=g).to(torch.bfloat16),
             torch.empty(n, device="cuda", dtype=torch.bfloat16), torch.empty(n, device="cuda", dtype=torch.bfloat16)) for _ in range(nsets)]
    gamma = (1.0 + 0.02 * torch.randn(hidden, device="cuda", generator=g)).float()
    stream = torch.cuda.Stream()

    def launch(i):
        x, r, y, ro = sets[i % nsets]
        pkg.rmsnorm_forward(rows, hidden, cfg["eps"], 2, x.data_ptr(), gamma.data_ptr(), y.data_ptr(), r.data_ptr(), ro.data_ptr(),
                            stream.cuda_stream, gamma_fp32=True)

    with torch.cuda.stream(stream):
        for i in range(max(3, warmup)):
            launch(i)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        s.record(stream)
        for i in range(steps):
            launch(i)
        e.record(stream)
        torch.cuda.synchronize()
    us = s.elapsed_time(e) * 1e3 / steps
    bytes_ = 4 * n * 2 + hidden * 4
    return {"us": us, "gbs": bytes_ / (us * 1e-6) / 1e9, "bytes": bytes_, "launches": steps}


def time_chain(torch, pkg, ranks, steps, warmup, global_batch=256, layout="nchw", tune=False):
    """ResNet-50-shaped FP16 chain, one CUDA graph per replica, batch sharded contiguously over the ranks.
    layout "nchw": the reference API's contract layer by layer; "nhwc": channel-contiguous tensors, prepacked weights and
    the residual adds fused into the convolution epilogues."""
    from cuda_inference_b200.chain import ConvChain, shard_batch
    _, count = shard_batch(global_batch, ranks.world, ranks.rank)
    chain = ConvChain(max(count, 1), 1, 224, seed=0, layout=layout, tune=tune)
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + ranks.rank)
    chain.input.copy_(torch.randn(chain.input.numel(), device="cuda", generator=g).to(torch.float16))
    stream = torch.cuda.Stream()
    chain.capture(stream)
    with torch.cuda.stream(stream):
        for _ in range(max(3, warmup)):
            chain.replay()
        stream.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ranks.barrier()
        torch.cuda.synchronize()
        s.record(stream)
        for _ in range(steps):
            chain.replay()
        e.record(stream)
        torch.cuda.synchronize()
        ranks.barrier()
    ms = ranks.max(s.elapsed_time(e))
    assert chain.device_status() == 0
    finite = bool(torch.isfinite(chain.output.float()).all().item())
    per_pass_ms = ms / steps
    return {"images_per_s": global_batch / (per_pass_ms * 1e-3), "ms_per_pass": per_pass_ms, "global_batch": global_batch,
            "images_per_rank": count, "tflops": (chain.flops / max(count, 1)) * global_batch / (per_pass_ms * 1e-3) / 1e12,
            "launches_per_pass": chain.launches, "graph": "one CUDA graph per replica", "output_finite": finite, "steps": steps,
            "layout": layout, "tuned": bool(tune)}


# ------------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------------
def make_conv_sets(torch, pkg, shape, nsets, seed):
    """Device-resident synthetic inputs with the benchmark's distributions: x ~ U[-1,1], w ~ Kaiming-uniform
    (bound sqrt(6/fan_in)), bias ~ U[-0.1,0.1], seeded.  `nsets` independent buffer sets so that consecutive steps
    touch different memory (the rotation is larger than L2)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    dt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[shape.precision]
    fan_in = shape.in_channels * shape.kernel * shape.kernel
    bound = (6.0 / fan_in) ** 0.5
    sets = []
    for _ in range(nsets):
        x = (torch.rand(shape.x_elems, device="cuda", generator=g) * 2 - 1).to(dt)
        w = ((torch.rand(shape.w_elems, device="cuda", generator=g) * 2 - 1) * bound).to(dt)
        b = ((torch.rand(shape.out_channels, device="cuda", generator=g) * 2 - 1) * 0.1).to(dt)
        y = torch.empty(shape.y_elems, device="cuda", dtype=dt)
        sets.append((x, w, b, y))
    return sets


def conv_problem(pkg, shape, flags=0):
    return pkg.ConvProblem(shape.batch, shape.in_channels, shape.in_h, shape.in_w, shape.out_channels, shape.kernel,
                           shape.kernel, shape.stride, shape.stride, shape.pad, shape.pad, 1, 1, 1, shape.precision, True, True,
                           flags)


def aligned_ws(torch, nbytes):
    t = torch.empty(max(int(nbytes), 256) + 256, dtype=torch.uint8, device="cuda")
    return t, (t.data_ptr() + 255) // 256 * 256


def time_conv(torch, pkg, shape, steps, warmup, world, barrier, max_over_ranks, cfg=None):
    """Times exactly `steps` forward calls on rotating buffer sets; replays a CUDA graph of one rotation so the host
    does not bound the measurement.  Returns a dict of raw measurements."""
    plan = pkg.ConvPlan(conv_problem(pkg, shape), cfg)
    per_set = (shape.x_elems + shape.w_elems + shape.y_elems) * shape.elem_size + plan.workspace_bytes
    nsets = max(2, min(64, int(160e6 // per_set) + 1))      # rotation > 126 MB of L2
    sets = make_conv_sets(torch, pkg, shape, nsets, seed=1234)
    wss = [aligned_ws(torch, plan.workspace_bytes) for _ in range(nsets)]
    stream = torch.cuda.Stream()

    def launch(i, st):
        x, w, b, y = sets[i % nsets]
        plan.launch(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), wss[i % nsets][1], plan.workspace_bytes, st)

    with torch.cuda.stream(stream):
        for i in range(min(warmup, nsets)):
            launch(i, stream.cuda_stream)
        stream.synchronize()
        group = min(nsets, steps)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(group):
                launch(i, torch.cuda.current_stream().cuda_stream)
        for _ in range(max(0, (warmup - min(warmup, nsets) + group - 1) // group)):
            graph.replay()
        stream.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        torch.cuda.synchronize()
        start.record(stream)
        for _ in range(steps // group):
            graph.replay()
        for i in range(steps % group):
            launch(i, stream.cuda_stream)
        end.record(stream)
        torch.cuda.synchronize()
        barrier()
        ms = max_over_ranks(start.elapsed_time(end))
        # per-stage device time (CUDA events between the stages, on the launching stream)
        x, w, b, y = sets[0]
        stage_ms = plan.time_stages(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), wss[0][1], plan.workspace_bytes,
                                    stream.cuda_stream, iters=min(200, max(20, steps)))
    assert plan.device_status() == 0, "a bounded device-side wait expired during the benchmark"
    return dict(plan=plan, ms=ms, stage_ms=stage_ms, nsets=nsets, sets=sets, wss=wss, launches=steps * plan.info.launches,
                rotation_bytes=per_set * nsets)


E2E_BUFFER_SETS = 3


class _Cudart:
    """The few CUDA runtime calls of the end-to-end loop, bound with ctypes: an asynchronous copy or an event call costs
    about a microsecond of host time this way, several through torch's tensor API, and at ~100 us per step the host must
    not be what the pipeline waits for."""

    def __init__(self):
        import ctypes as C
        self.C = C
        L = None
        for name in ("libcudart.so.12", "libcudart.so"):
            try:
                L = C.CDLL(name)
                break
            except OSError:
                continue
        if L is None:
            raise RuntimeError("the CUDA runtime library (libcudart) could not be loaded")
        L.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        L.cudaEventRecord.argtypes = [C.c_void_p, C.c_void_p]
        L.cudaStreamWaitEvent.argtypes = [C.c_void_p, C.c_void_p, C.c_uint]
        self.L = L

    def check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUDA error {rc}")

    def copy(self, dst, src, nbytes, kind, stream):
        self.check(self.L.cudaMemcpyAsync(dst, src, nbytes, kind, stream), "cudaMemcpyAsync")

    def record(self, event, stream):
        self.check(self.L.cudaEventRecord(event, stream), "cudaEventRecord")

    def wait(self, stream, event):
        self.check(self.L.cudaStreamWaitEvent(stream, event, 0), "cudaStreamWaitEvent")


def time_conv_e2e(torch, pkg, shape, plan, steps):
    """Same metric end to end through the public call with HOST buffers: every step copies x, w and bias from pinned
    host memory (one packed buffer, one copy), runs the forward call, and copies y back to pinned host memory.  Steps
    are pipelined the way a serving loop would run them: one stream each for host->device copies, the forward calls and
    device->host copies, E2E_BUFFER_SETS device/host buffer sets, events between the three (a step's copy-in overlaps
    the previous step's compute and the copy-out of the one before)."""
    import numpy as np
    rt = _Cudart()
    rng = np.random.default_rng(7)
    npdt = np.float32 if shape.precision == 0 else np.float16
    tdt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[shape.precision]
    es = shape.elem_size
    fan_in = shape.in_channels * shape.kernel * shape.kernel
    hx = torch.from_numpy(rng.uniform(-1, 1, shape.x_elems).astype(npdt)).to(tdt)
    hw = torch.from_numpy((rng.uniform(-1, 1, shape.w_elems) * (6.0 / fan_in) ** 0.5).astype(npdt)).to(tdt)
    hb = torch.from_numpy(rng.uniform(-0.1, 0.1, shape.out_channels).astype(npdt)).to(tdt)
    # x | w | bias packed at 256-byte aligned offsets of one pinned buffer
    al = lambda n: (n + 255) // 256 * 256
    off_w = al(shape.x_elems * es)
    off_b = off_w + al(shape.w_elems * es)
    in_bytes = off_b + al(shape.out_channels * es)
    hin = torch.zeros(in_bytes, dtype=torch.uint8).pin_memory()
    hin[:shape.x_elems * es] = hx.view(torch.uint8)
    hin[off_w:off_w + shape.w_elems * es] = hw.view(torch.uint8)
    hin[off_b:off_b + shape.out_channels * es] = hb.view(torch.uint8)
    nb = E2E_BUFFER_SETS
    hy = [torch.empty(shape.y_elems, dtype=tdt).pin_memory() for _ in range(nb)]
    din = [torch.empty(in_bytes, dtype=torch.uint8, device="cuda") for _ in range(nb)]
    dy = [torch.empty(shape.y_elems, dtype=tdt, device="cuda") for _ in range(nb)]
    y_bytes = shape.y_elems * es
    wst, wsp = aligned_ws(torch, plan.workspace_bytes)
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    q_in, q_run, q_out = s_in.cuda_stream, s_run.cuda_stream, s_out.cuda_stream
    events = [[torch.cuda.Event() for _ in range(nb)] for _ in range(3)]
    for row, st in zip(events, (s_in, s_run, s_out)):
        for ev in row:
            ev.record(st)          # creates the underlying CUDA event
    ev_in, ev_run, ev_out = ([ev.cuda_event for ev in row] for row in events)
    H2D, D2H = 1, 2

    def step(i):
        k = i % nb
        base = din[k].data_ptr()
        if i >= nb:
            rt.wait(q_in, ev_run[k])      # the forward call that read this input set has finished
        rt.copy(base, hin.data_ptr(), in_bytes, H2D, q_in)
        rt.record(ev_in[k], q_in)
        rt.wait(q_run, ev_in[k])
        if i >= nb:
            rt.wait(q_run, ev_out[k])     # the copy-out that read this output buffer has finished
        plan.launch(base, base + off_w, base + off_b, dy[k].data_ptr(), wsp, plan.workspace_bytes, q_run)
        rt.record(ev_run[k], q_run)
        rt.wait(q_out, ev_run[k])
        rt.copy(hy[k].data_ptr(), dy[k].data_ptr(), y_bytes, D2H, q_out)
        rt.record(ev_out[k], q_out)

    for i in range(2 * nb):
        step(i)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(s_in)
    for i in range(steps):
        step(i + 2 * nb)
    s_out.wait_stream(s_in)
    s_out.wait_stream(s_run)
    e.record(s_out)
    torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    h2d = in_bytes      # the packed buffer as copied (x, w, bias and their alignment padding)
    d2h = y_bytes
    return ms, h2d, d2h, (hx, hw, hb, hy[(steps + 2 * nb - 1) % nb])


def cpu_reference_runner():
    """Returns (orc, oracle, conv(problem, x, w, b) -> y, kind, threads) for the CPU baseline: the reference's own CPU
    code when oracle/_ref exists, else the C restatement.  Both use every host core the process may run on, whatever
    OMP_NUM_THREADS a launcher exported: the reference's convolution is a scalar function, so whole images are dealt
    to a pool of threads (ctypes calls release the GIL); the restatement is OpenMP code."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    orc = entry.load_oracle()
    o = orc.Oracle()
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    if orc.Reference.available():
        r = orc.Reference()
        pool = ThreadPoolExecutor(max_workers=threads)

        def conv(p, x, w, b):
            parts = min(threads, p.batch)
            if parts <= 1:
                return r.conv2d(p, x, w, b)[0]
            bounds = [p.batch * i // parts for i in range(parts + 1)]

            def one(i):
                lo, hi = bounds[i], bounds[i + 1]
                sub = orc.Problem.P(hi - lo, p.in_channels, p.in_h, p.in_w, p.out_channels, p.kernel_h, p.kernel_w, p.stride_h,
                                    p.stride_w, p.pad_h, p.pad_w, p.precision, p.has_bias, p.relu)
                return r.conv2d(sub, np.ascontiguousarray(x[lo:hi]), w, b)[0]

            return np.concatenate(list(pool.map(one, range(parts))), axis=0)

        return orc, o, conv, "reference", threads
    o.set_num_threads(threads)
    return orc, o, (lambda p, x, w, b: o.conv2d(p, x, w, b, want_scale=False)[0]), "port", o.num_threads()


def cpu_baseline_leg(torch, shape, host_inputs, gpu_y, budget_s=12.0):
    """Times the CPU convolution on a bounded sample (whole images of the workload) and checks the GPU result for
    those images against it.  host_inputs = (x, w, b) torch host tensors in the storage type."""
    import numpy as np
    orc, o, conv, kind, threads = cpu_reference_runner()
    hx, hw, hb = (t.float().numpy() for t in host_inputs)
    per_img = shape.in_channels * shape.in_h * shape.in_w
    n_img, reps, elapsed = 1, 0, 0.0
    check = None
    t_first = None
    while True:
        p = orc.Problem.P(n_img, shape.in_channels, shape.in_h, shape.in_w, shape.out_channels, shape.kernel, shape.kernel,
                          shape.stride, shape.stride, shape.pad, shape.pad, shape.precision, True, True)
        t0 = time.perf_counter()
        y = conv(p, hx[:n_img * per_img].reshape(p.x_shape), hw.reshape(p.w_shape), hb)
        dt = time.perf_counter() - t0
        if t_first is None:  # first call sizes the sample: as many images as fit ~1/3 of the budget per repetition
            t_first = dt
            if gpu_y is not None:
                got = gpu_y.float().numpy()[:y.size].reshape(y.shape)
                err = np.abs(got - y)
                tol = (5e-3 + 1e-2 * np.abs(y)) if shape.precision == 1 else ((2e-2 + 3e-2 * np.abs(y)) if shape.precision == 2
                                                                             else 1e-5 * np.maximum(np.abs(y), np.sqrt(np.mean(y * y))))
                check = bool(np.all(err <= tol))
            n_img = int(max(1, min(shape.batch, (budget_s / 3) // max(dt, 1e-6))))
            continue
        reps += 1
        elapsed += dt
        if elapsed >= budget_s or reps >= 50:
            break
    flops = 2 * n_img * shape.out_h * shape.out_w * shape.out_channels * shape.in_channels * shape.kernel * shape.kernel
    return {"value": flops * reps / elapsed / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": f"{n_img} of {shape.batch} images of the workload, all output channels, {reps} repetitions, {elapsed:.1f} s",
            "gpu_matches_cpu_on_sample": check}


def run_ours(args):
    import torch

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    entry.load_package()
    from cuda_inference_b200.dist import Ranks
    ranks = Ranks("nccl")
    barrier, max_over_ranks = ranks.barrier, ranks.max

    pkg = entry.load_package()
    from cuda_inference_b200 import workloads as wl
    peaks, peak_kind = load_peaks()
    if args.workload == "chain":
        return run_chain_primary(args, torch, pkg, ranks, peaks, peak_kind, local_rank)
    shape, bound = wl.CONV_WORKLOADS[args.workload]
    sampler = ClockSampler(local_rank)
    sampler.start()
    res = time_conv(torch, pkg, shape, args.steps, args.warmup, world, barrier, max_over_ranks)
    clocks = sampler.stop()
    plan = res["plan"]
    ms = res["ms"]
    value = world * args.steps * shape.flops / (ms * 1e-3) / 1e12

    conv_ms = res["stage_ms"][1]
    if bound == "hbm":
        achieved = shape.algorithmic_bytes / (conv_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"]}
    else:
        achieved = shape.flops / (conv_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"]}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get(args.workload), "kernel": "conv_tc_kernel" if shape.precision else "conv_fp32_kernel",
                 "kernel_us": conv_ms * 1e3, "repack_us": res["stage_ms"][0] * 1e3, "splitk_reduce_us": res["stage_ms"][2] * 1e3,
                 "peak_source": f"{peak_kind} (cuBLAS bf16 burst / STREAM copy)",
                 "algorithmic_per_launch": shape.flops if bound != "hbm" else shape.algorithmic_bytes})
    if plan.info.cfg.reduce != 1 and res["stage_ms"][2] > 0 and conv_ms > res["stage_ms"][2]:
        # Without a reduction launch the third stage is an empty event pair: what it measures is the cost of the event
        # records themselves, which every stage time above contains.  `achieved` / `frac` keep the raw stage time.
        net_ms = conv_ms - res["stage_ms"][2]
        net = (shape.algorithmic_bytes / (net_ms * 1e-3) / 1e9) if bound == "hbm" else (shape.flops / (net_ms * 1e-3) / 1e12)
        roof.update({"event_pair_overhead_us": res["stage_ms"][2] * 1e3, "achieved_net_of_event_overhead": net,
                     "frac_net_of_event_overhead": net / roof["peak"]})

    e2e_steps = min(args.steps, 1000)
    e2e_ms, h2d, d2h, host = time_conv_e2e(torch, pkg, shape, plan, e2e_steps)
    e2e_ms = max_over_ranks(e2e_ms)
    e2e = {"value": world * e2e_steps * shape.flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "steps": e2e_steps,
           "pipeline": f"copy-in (x, w, bias packed: one copy), forward and copy-out streams over {E2E_BUFFER_SETS} buffer sets; all copies from/to pinned host memory inside the timed region"}

    out = {
        "metric": "FP16 conv TFLOP/s (effective, 2*N*K*P*Q*C*R*S / time, repack + prepack + conv per step)",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {0: "fp32", 1: "fp16", 2: "bf16"}[shape.precision] + " (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={shape.batch} C={shape.in_channels} {shape.in_h}x{shape.in_w} K={shape.out_channels} "
                               f"{shape.kernel}x{shape.kernel}/s{shape.stride} p{shape.pad} NCHW, fused bias+ReLU",
                   "tile": {"tile_m": plan.info.cfg.tile_m, "tile_n": plan.info.cfg.tile_n, "tile_k": plan.info.cfg.tile_k, "stages": plan.info.cfg.stages,
                            "split_k": plan.info.cfg.split_k,
                            "reduce": {0: "none", 1: "workspace + reduction launch", 2: "cluster (distributed shared memory)"}[plan.info.cfg.reduce]},
                   "cold_cache": f"inputs larger than L2: {res['nsets']} rotating buffer sets, {res['rotation_bytes'] / 1e6:.0f} MB",
                   "launch": "CUDA graph of one buffer rotation, replayed", "replicas": world},
        "roofline": roof, "e2e": e2e, "gpu_launches": res["launches"], "clocks": clocks,
    }
    # Secondary measurements (not the headline): the other benchmark shapes on one GPU, and the conv chain on all ranks.
    if not args.no_secondary:
        sec = {}
        if world == 1:
            for name in ("c1", "c3_fp16", "c3_bf16", "c4a", "c4b"):
                if name == args.workload:
                    continue
                sh, bd = wl.CONV_WORKLOADS[name]
                r2 = time_conv(torch, pkg, sh, min(args.steps, 2000), 20, 1, lambda: None, float)
                k_us = r2["stage_ms"][1] * 1e3
                entry_ = {"us_per_step": r2["ms"] * 1e3 / min(args.steps, 2000), "tflops": sh.flops * min(args.steps, 2000) / (r2["ms"] * 1e-3) / 1e12,
                          "kernel_us": k_us, "repack_us": r2["stage_ms"][0] * 1e3, "bound": bd,
                          "tile": [r2["plan"].info.cfg.tile_m, r2["plan"].info.cfg.tile_n, r2["plan"].info.cfg.tile_k, r2["plan"].info.cfg.stages,
                                   r2["plan"].info.cfg.split_k]}
                if bd == "hbm":
                    entry_["pipeline_gbs"] = sh.algorithmic_bytes / (entry_["us_per_step"] * 1e-6) / 1e9
                    entry_["frac_of_hbm"] = entry_["pipeline_gbs"] / peaks["hbm_gbs"]
                elif bd == "tensor":
                    entry_["frac_of_tensor"] = entry_["tflops"] / peaks["bf16_tflops"]
                sec[name] = entry_
                del r2
                torch.cuda.empty_cache()
            rms = time_rmsnorm(torch, pkg, min(args.steps, 300), 10)
            rms["frac_of_hbm"] = rms["gbs"] / peaks["hbm_gbs"]
            sec["rmsnorm_bf16_8192x4096_residual"] = rms
            torch.cuda.empty_cache()
        ch = time_chain(torch, pkg, ranks, steps=max(3, min(args.steps, 10)), warmup=3)
        ch["frac_of_tensor"] = ch["tflops"] / world / peaks["bf16_tflops"]
        sec["chain_resnet50_fp16_batch256"] = ch
        del ch
        torch.cuda.empty_cache()
        ch2 = time_chain(torch, pkg, ranks, steps=max(3, min(args.steps, 10)), warmup=3, layout="nhwc", tune=True)
        ch2["frac_of_tensor"] = ch2["tflops"] / world / peaks["bf16_tflops"]
        sec["chain_resnet50_fp16_batch256_channel_contiguous_fused_residual_tuned"] = ch2
        out["secondary"] = sec
    if world == 1 and rank == 0 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline_leg(torch, shape, host[:3], host[3])
    if rank == 0:
        print(json.dumps(out))
    ranks.close()


def run_chain_primary(args, torch, pkg, ranks, peaks, peak_kind, local_rank):
    """`--workload chain`: the conv chain as the headline (images/s, batch 256 sharded over the ranks: strong scaling)."""
    sampler = ClockSampler(local_rank)
    sampler.start()
    ch = time_chain(torch, pkg, ranks, steps=args.steps, warmup=args.warmup, layout=args.layout, tune=args.tune)
    clocks = sampler.stop()
    # a timed region of seconds runs under the power cap: compare it with the sustained GEMM peak, a short one with the burst
    timed_s = ch["ms_per_pass"] * args.steps * 1e-3
    sustained = timed_s > 2.0 and "bf16_tflops_sustained" in peaks
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    peak_kind = f"{peak_kind} ({'sustained' if sustained else 'burst'} cuBLAS bf16; the timed region lasted {timed_s:.1f} s)"
    out = {"metric": "conv-chain images/s (ResNet-50-shaped FP16 inference chain, batch 256)", "value": ch["images_per_s"], "unit": "images/s",
           "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ch["ms_per_pass"], "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)", "data": "synthetic",
           "config": {"workload": "c5: 53-conv ResNet-50-shaped chain, 224x224x3 input N(0,1), batch 256 sharded contiguously over the ranks, "
                                  "replicated random weights, one CUDA graph per replica", "cold_cache": "activations per pass exceed L2 (5.6 GB)"},
           "roofline": {"bound": "tensor", "achieved": ch["tflops"] / ranks.world, "peak": peak, "unit": "TFLOP/s",
                        "frac": ch["tflops"] / ranks.world / peak, "traffic": None, "kernel": "whole chain (per GPU)",
                        "peak_source": peak_kind},
           "gpu_launches": ch["launches_per_pass"] * args.steps, "clocks": clocks, "chain": ch}
    if ranks.rank == 0:
        print(json.dumps(out))
    ranks.close()


# ------------------------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU convolution on the host cores
# ------------------------------------------------------------------------------------------------------------------
def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    import numpy as np
    entry.load_package()
    from cuda_inference_b200 import workloads as wl
    shape, _ = wl.CONV_WORKLOADS[args.workload]
    orc, o, conv, kind, threads = cpu_reference_runner()
    full = orc.Problem.P(shape.batch, shape.in_channels, shape.in_h, shape.in_w, shape.out_channels, shape.kernel, shape.kernel,
                         shape.stride, shape.stride, shape.pad, shape.pad, shape.precision, True, True)
    x, w, b = o.make_baseline_data(full, 0)

    def problem(n_img, n_out):
        return orc.Problem.P(n_img, shape.in_channels, shape.in_h, shape.in_w, n_out, shape.kernel, shape.kernel, shape.stride,
                             shape.stride, shape.pad, shape.pad, shape.precision, True, True)

    # size the per-step sample so that steps + warmup end within ~2 minutes
    t0 = time.perf_counter()
    conv(problem(1, shape.out_channels), x[:1], w, b)
    t_img = time.perf_counter() - t0
    budget = 110.0 / max(1, args.steps + args.warmup)
    n_img, n_out = 1, shape.out_channels
    if t_img <= budget:
        n_img = int(min(shape.batch, max(1, budget // t_img)))
    else:
        n_out = int(max(1, min(shape.out_channels, shape.out_channels * budget / t_img)))
    p = problem(n_img, n_out)
    xs, ws, bs = x[:n_img], w[:n_out], b[:n_out]
    for _ in range(args.warmup):
        conv(p, xs, ws, bs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        conv(p, xs, ws, bs)
    el = time.perf_counter() - t0
    value = p.flops * args.steps / el / 1e12
    sample = f"{n_img} of {shape.batch} images x {n_out} of {shape.out_channels} output channels per step"
    print(json.dumps({
        "impl": "reference", "metric": "FP16 conv TFLOP/s (effective, 2*N*K*P*Q*C*R*S / time)", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": el * 1e3 / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64 accumulate over storage-rounded inputs", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={shape.batch} C={shape.in_channels} {shape.in_h}x{shape.in_w} K={shape.out_channels} "
                               f"{shape.kernel}x{shape.kernel}/s{shape.stride} p{shape.pad} NCHW, fused bias+ReLU", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--workload", default="c2", help="c1 | c2 | c3_fp16 | c3_bf16 | c4a | c4b | chain")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layout", default="nchw", choices=["nchw", "nhwc"], help="--workload chain: tensor layout between layers")
    ap.add_argument("--tune", action="store_true", help="--workload chain: measure candidate configurations per layer first")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (other shapes, RMSNorm, conv chain)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
