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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu capture of that launch per
# workload (None where no capture exists).
NCU_TRAFFIC_BYTES = {"c2": 4470272, "c3_fp16": 52158976, "c4a": 5205760, "c4b": 13514752, "c1": 985856}

# The metric both arms report (the same string, so that the two lines can be compared): one step = one forward call =
# layout repack + weight prepack + convolution with fused bias + ReLU.
CONV_METRIC = "FP16 conv TFLOP/s (effective, 2*N*K*P*Q*C*R*S / time)"

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


def share_tuned_configs(ranks):
    """Every replica runs the configurations rank 0 measured (replicas that tune on their own may pick different
    kernels for the same layer)."""
    from cuda_inference_b200 import chain as chain_mod
    if not ranks.active:
        return
    box = [chain_mod.tuned_configs() if ranks.rank == 0 else None]
    ranks.dist.broadcast_object_list(box, src=0)
    if ranks.rank != 0:
        chain_mod.set_tuned_configs(box[0])


def time_chain(torch, pkg, ranks, steps, warmup, global_batch=256, layout="nchw", tune=False, world=None, keep=False, protocol=True):
    """ResNet-50-shaped FP16 chain, one CUDA graph per replica, batch sharded contiguously over the ranks.
    layout "nchw": the reference API's contract layer by layer; "nchw_fused": the same NCHW tensors with each block's residual
    add + ReLU inside the epilogue of its last convolution; "nhwc": channel-contiguous tensors, prepacked weights and
    the residual adds fused into the convolution epilogues.  world = 1 makes every rank run the WHOLE batch (the one-GPU
    point of the scaling curve, measured in the same run).  Times exactly `steps` passes between one event pair (max
    over ranks) and, beside it, the 30-sample protocol."""
    from cuda_inference_b200.chain import ConvChain, shard_batch
    w = ranks.world if world is None else world
    r = ranks.rank if world is None else 0
    _, count = shard_batch(global_batch, w, r)
    fuse = layout == "nchw_fused"   # NCHW tensors, residual add + ReLU inside the epilogue of each block's last convolution
    tensor_layout = "nchw" if fuse else layout
    if tune:
        if ranks.rank == 0:
            ConvChain(max(count, 1), 1, 224, seed=0, layout=tensor_layout, tune=True, fuse_residual=fuse)  # measures; the table stays in the process
        share_tuned_configs(ranks)
    chain = ConvChain(max(count, 1), 1, 224, seed=0, layout=tensor_layout, tune=tune, fuse_residual=fuse)
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + r)
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
    if protocol:
        proto = protocol_samples(torch, stream, chain.replay, 1, samples=30, min_ms=1.0, warmups=2)
        for k in ("median_us", "p10_us", "p90_us"):
            proto[k] = ranks.max(proto[k])
    else:  # a short run for a profiler
        proto = {"median_us": ms * 1e3 / steps, "p10_us": ms * 1e3 / steps, "p90_us": ms * 1e3 / steps, "samples": 0}
    assert chain.device_status() == 0
    finite = bool(torch.isfinite(chain.output.float()).all().item())
    per_pass_ms = ms / steps
    out = {"images_per_s": global_batch / (per_pass_ms * 1e-3), "ms_per_pass": per_pass_ms, "global_batch": global_batch,
           "images_per_rank": count, "gpus": w, "tflops": (chain.flops / max(count, 1)) * global_batch / (per_pass_ms * 1e-3) / 1e12,
           "launches_per_pass": chain.launches, "graph": "one CUDA graph per replica", "output_finite": finite, "steps": steps,
           "layout": layout, "tuned": bool(tune),
           "protocol": {"images_per_s": global_batch / (proto["median_us"] * 1e-6), "ms_per_pass_median": proto["median_us"] * 1e-3,
                        "ms_per_pass_p10": proto["p10_us"] * 1e-3, "ms_per_pass_p90": proto["p90_us"] * 1e-3, "samples": proto["samples"]}}
    if keep:
        out["_chain"] = chain
    return out


def chain_cpu_leg(torch, chain, n_img=2):
    """The CPU baseline of the conv chain on a stated sub-batch, and the end-to-end parity of those images: the first
    `n_img` images of this replica go through the reference's CPU convolution layer by layer (activations rounded to FP16
    between layers, as the tensors the GPU chain stores are; max-pool and residual add from their definitions), timed on
    all host cores, and the GPU chain's final output for the same images is compared with the result.  Images are
    independent, so the sub-batch is a sample of the workload.  Tolerance of the end-to-end comparison (accumulated over
    53 layers of FP16 storage rounding and FP32-vs-double accumulation): |err| <= 0.02 * max|ref| + 0.05 * |ref|."""
    import numpy as np
    orc, o, conv, kind, threads = cpu_reference_runner()
    prec = chain.precision
    n_img = min(n_img, chain.batch)
    slots = {}
    c0, h0, w0 = chain.slot_shapes[0]
    x = chain.input.view(chain.batch, -1)[:n_img].float().cpu().numpy().reshape(n_img, c0, h0, w0)
    slots[0] = x
    weights = {op.layer: (wsrc.float().cpu().numpy(), b.float().cpu().numpy()) for (op, _, _, b), wsrc in zip(chain.convs, chain.oihw_weights)}
    t0 = time.perf_counter()
    for op in chain.base_ops:
        if op.kind == "conv":
            sh = op.shape
            p = orc.Problem.P(n_img, sh.in_channels, sh.in_h, sh.in_w, sh.out_channels, sh.kernel, sh.kernel, sh.stride, sh.stride,
                              sh.pad, sh.pad, prec, True, op.relu)
            wv, bv = weights[op.layer]
            y = conv(p, slots[op.src], wv.reshape(p.w_shape), bv)
            slots[op.dst] = o.quantize(prec, y).reshape(p.y_shape)
        elif op.kind == "maxpool":
            _, _, _, k, st, pad = op.pool
            slots[op.dst] = o.maxpool2d(slots[op.src], k, st, pad)
        else:
            a, b2 = slots[op.src], slots[op.other]
            slots[op.dst] = o.add_relu(prec, a.ravel(), b2.ravel(), op.relu).reshape(a.shape)
    cpu_s = time.perf_counter() - t0
    last = len(chain.slot_shapes) - 1
    ref = slots[last].astype(np.float64)
    c, h, w = chain.slot_shapes[last]
    got = chain.output.view(chain.batch, -1)[:n_img].float().cpu().numpy()
    got = got.reshape(n_img, h, w, c).transpose(0, 3, 1, 2) if chain.layout == "nhwc" else got.reshape(n_img, c, h, w)
    err = np.abs(got.astype(np.float64) - ref)
    tol = 0.02 * np.abs(ref).max() + 0.05 * np.abs(ref)
    return {"value": n_img / cpu_s, "unit": "images/s", "cores": threads, "kind": kind,
            "sample": f"{n_img} of {chain.batch} images of this replica through all 53 convolutions, max-pool and 16 residual adds, once, {cpu_s:.1f} s",
            "gpu_matches_cpu_on_sample": bool(np.all(err <= tol)), "max_err_over_max_ref": float(err.max() / max(np.abs(ref).max(), 1e-30)),
            "tolerance": "|err| <= 0.02 * max|ref| + 0.05 * |ref| on the chain's final tensor"}


# ------------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------------
def make_conv_sets(torch, pkg, shape, nsets, seed):
    """Device-resident synthetic inputs with the benchmark's distributions: x ~ U[-1,1], w ~ Kaiming-uniform
    (bound sqrt(6/fan_in)), bias ~ U[-0.1,0.1], seeded.  `nsets` independent buffer sets so that consecutive steps
    touch different memory (the rotation is larger than L2)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    fp8 = shape.precision == 4   # FP8 E4M3 x and w (bit patterns as bytes), float bias, FP16 y
    dt = torch.float16 if fp8 else {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[shape.precision]
    fan_in = shape.in_channels * shape.kernel * shape.kernel
    bound = (6.0 / fan_in) ** 0.5
    sets = []
    for _ in range(nsets):
        x = torch.rand(shape.x_elems, device="cuda", generator=g) * 2 - 1
        w = (torch.rand(shape.w_elems, device="cuda", generator=g) * 2 - 1) * bound
        b = (torch.rand(shape.out_channels, device="cuda", generator=g) * 2 - 1) * 0.1
        if fp8:
            x, w = x.to(torch.float8_e4m3fn).view(torch.uint8), w.to(torch.float8_e4m3fn).view(torch.uint8)
        else:
            x, w, b = x.to(dt), w.to(dt), b.to(dt)
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


def percentile(sorted_vals, q):
    if not sorted_vals:
        return None
    i = min(len(sorted_vals) - 1, max(0, int(round(q * (len(sorted_vals) - 1)))))
    return sorted_vals[i]


def protocol_samples(torch, stream, run, units_per_run, samples=30, min_ms=1.0, warmups=5):
    """The reference's timing protocol (src/runtime/timing.cpp:42-83): `warmups` untimed runs, then `samples` samples, each
    one event pair around enough back-to-back runs to last at least `min_ms`; returns per-unit microseconds (median, p10,
    p90).  `run()` enqueues `units_per_run` units of work on `stream` (a graph replay)."""
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(warmups):
            run()
        s.record(stream)
        run()
        e.record(stream)
        e.synchronize()
        est = max(s.elapsed_time(e), 1e-3)
        reps = max(1, int(-(-min_ms // est)))
        vals = []
        for _ in range(samples):
            s.record(stream)
            for _ in range(reps):
                run()
            e.record(stream)
            e.synchronize()
            vals.append(s.elapsed_time(e) * 1e3 / (reps * units_per_run))
    vals.sort()
    return {"median_us": percentile(vals, 0.5), "p10_us": percentile(vals, 0.1), "p90_us": percentile(vals, 0.9), "samples": samples,
            "units_per_sample": reps * units_per_run}


def time_conv(torch, pkg, shape, steps, warmup, world, barrier, max_over_ranks, cfg=None, stage_times=True, protocol=True):
    """Times forward calls on rotating buffer sets (the rotation is larger than L2), always as replays of CUDA graphs so
    that the host never bounds the measurement.  Two measurements:
      * the K-step region: exactly `steps` steps between one event pair, bracketed by barriers and synchronisation;
      * the protocol: 30 samples of at least 1 ms each (median, p10, p90) -- the number of record, because a region of a
        few hundred microseconds (small K) is dominated by its first launches.
    With stage_times, the layout-repack launch and the convolution kernel are also timed alone, back to back in graphs of
    single-stage calls over the same rotation (the workspaces hold the repacked tensors of the full calls before)."""
    plan = pkg.ConvPlan(conv_problem(pkg, shape), cfg)
    per_set = (shape.x_elems + shape.w_elems + shape.y_elems) * shape.elem_size + plan.workspace_bytes
    nsets = max(2, min(64, int(160e6 // per_set) + 1))      # rotation > 126 MB of L2
    sets = make_conv_sets(torch, pkg, shape, nsets, seed=1234)
    wss = [aligned_ws(torch, plan.workspace_bytes) for _ in range(nsets)]
    stream = torch.cuda.Stream()

    def launch(i, st, mask=7):
        x, w, b, y = sets[i % nsets]
        if mask == 7:
            plan.launch(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), wss[i % nsets][1], plan.workspace_bytes, st)
        else:
            plan.launch_stages(mask, x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), wss[i % nsets][1], plan.workspace_bytes, st)

    def capture(count, mask=7):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(count):
                launch(i, torch.cuda.current_stream().cuda_stream, mask)
        return g

    with torch.cuda.stream(stream):
        for i in range(nsets):   # eager once per set: every workspace holds its repacked tensors afterwards
            launch(i, stream.cuda_stream)
        stream.synchronize()
        group = min(nsets, steps)
        graph = capture(group)
        tail = capture(steps % group) if steps % group else None
        for _ in range(max(1, -(-warmup // group))):
            graph.replay()
        stream.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        torch.cuda.synchronize()
        start.record(stream)
        for _ in range(steps // group):
            graph.replay()
        if tail is not None:
            tail.replay()
        end.record(stream)
        torch.cuda.synchronize()
        barrier()
        ms = max_over_ranks(start.elapsed_time(end))
    if not protocol:  # a short run for a profiler: the K-step region only
        us = ms * 1e3 / steps
        return dict(plan=plan, ms=ms, proto={"median_us": us, "p10_us": us, "p90_us": us, "samples": 0, "units_per_sample": steps},
                    kernel={"median_us": us, "p10_us": us, "p90_us": us}, nsets=nsets, sets=sets, wss=wss,
                    launches=steps * plan.info.launches, rotation_bytes=per_set * nsets)
    full = capture(nsets) if group != nsets else graph
    proto = protocol_samples(torch, stream, full.replay, nsets)
    for k in ("median_us", "p10_us", "p90_us"):
        proto[k] = max_over_ranks(proto[k])
    out = dict(plan=plan, ms=ms, proto=proto, nsets=nsets, sets=sets, wss=wss, launches=steps * plan.info.launches,
               rotation_bytes=per_set * nsets)
    if stage_times:
        has_repack = plan.info.launches > 1 + (1 if plan.info.cfg.reduce == 1 else 0)
        gk = capture(nsets, 2 | 4)  # the convolution kernel (and the reduction launch of a workspace split-K)
        out["kernel"] = protocol_samples(torch, stream, gk.replay, nsets)
        if has_repack:
            gr = capture(nsets, 1)
            out["repack"] = protocol_samples(torch, stream, gr.replay, nsets)
    assert plan.device_status() == 0, "a bounded device-side wait expired during the benchmark"
    return out


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
    code when oracle/_ref exists, else the C restatement.  Both are OpenMP loops over the outputs
    (src/cpu/cpu_reference.cpp:23 of the reference); the thread count is set to every host core the process may run on,
    whatever OMP_NUM_THREADS a launcher exported, and nothing else is threaded on top of it."""
    orc = entry.load_oracle()
    o = orc.Oracle()
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    if orc.Reference.available():
        r = orc.Reference()
        r.set_num_threads(threads)
        return orc, o, (lambda p, x, w, b: r.conv2d(p, x, w, b)[0]), "reference", r.num_threads()
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


def chain_block(torch, pkg, ranks, peaks, steps, do_cpu):
    """The conv chain (batch 256 sharded over the ranks, strong scaling) in both layouts: images/s over at least 50 passes,
    and for N > 1 the one-GPU point measured in the same run (every rank runs the whole batch) with the efficiency
    against it.  On one GPU, rank 0 also runs the CPU baseline of the chain on a sub-batch and checks the GPU output."""
    out = {}
    passes = max(50, min(steps, 200))
    for key, layout, tune in (("nchw", "nchw", False), ("nchw_fused", "nchw_fused", False), ("nhwc_fused_tuned", "nhwc", True)):
        ch = time_chain(torch, pkg, ranks, steps=passes, warmup=3, layout=layout, tune=tune, keep=True)
        chain = ch.pop("_chain")
        ch["frac_of_tensor"] = ch["tflops"] / ranks.world / peaks["bf16_tflops"]
        if do_cpu and layout == "nchw":
            ch["cpu_baseline"] = chain_cpu_leg(torch, chain, n_img=2)
        del chain
        torch.cuda.empty_cache()
        if ranks.world > 1:
            one = time_chain(torch, pkg, ranks, steps=max(10, passes // 4), warmup=3, layout=layout, tune=tune, world=1)
            ch["one_gpu_images_per_s_same_run"] = one["images_per_s"]
            ch["efficiency_vs_one_gpu"] = ch["images_per_s"] / (ranks.world * one["images_per_s"])
            torch.cuda.empty_cache()
        out[key] = ch
    return out


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
    if shape.precision == wl.FP8_E4M3 and not args.profile_run:
        raise SystemExit("c2_fp8 (an extension without a CPU-reference arm) is measured in the secondary block of the default run; "
                         "--profile-run runs it alone for a profiler")
    sampler = ClockSampler(local_rank)
    sampler.start()
    cfg = None
    if args.cfg:  # an explicit point of the kernel family instead of the heuristic's choice, e.g. --cfg split_k=4,reduce=1
        cfg = pkg.make_cfg(**{k: int(v) for k, v in (kv.split("=") for kv in args.cfg.split(","))})
    res = time_conv(torch, pkg, shape, args.steps, args.warmup, world, barrier, max_over_ranks, cfg=cfg, protocol=not args.profile_run)
    clocks = sampler.stop()
    if args.profile_run:  # for ncu: warm-up and the K-step region only (the numbers of such a run are not measurements)
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload, "us_per_step_k_region": res["ms"] * 1e3 / args.steps,
                              "launches_per_step": res["plan"].info.launches}))
        ranks.close()
        return
    plan = res["plan"]
    proto = res["proto"]
    step_us = proto["median_us"]                      # the number of record: median of 30 samples of >= 1 ms
    value = world * shape.flops / (step_us * 1e-6) / 1e12
    region_us = res["ms"] * 1e3 / args.steps          # the plain K-step region, for comparison

    kernel_us = res["kernel"]["median_us"]
    if bound == "hbm":
        achieved = shape.algorithmic_bytes / (kernel_us * 1e-6) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"]}
    else:
        achieved = shape.flops / (kernel_us * 1e-6) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"]}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get(args.workload), "kernel": "conv_tc_kernel" if shape.precision else "conv_fp32_kernel",
                 "kernel_us": kernel_us, "kernel_us_p10_p90": [res["kernel"]["p10_us"], res["kernel"]["p90_us"]],
                 "repack_us": res["repack"]["median_us"] if "repack" in res else 0.0,
                 "how": "average launch duration over CUDA-graph replays of that kernel alone, back to back over the rotating "
                        "buffer sets (30 samples of >= 1 ms, median); the workspaces hold the repacked tensors",
                 "peak_source": f"{peak_kind} (cuBLAS bf16 burst / STREAM copy)",
                 "algorithmic_per_launch": shape.flops if bound != "hbm" else shape.algorithmic_bytes})

    e2e_steps = max(200, min(args.steps, 1000))
    e2e_ms, h2d, d2h, host = time_conv_e2e(torch, pkg, shape, plan, e2e_steps)
    e2e_ms = max_over_ranks(e2e_ms)
    e2e = {"value": world * e2e_steps * shape.flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "steps": e2e_steps,
           "pipeline": f"copy-in (x, w, bias packed: one copy), forward and copy-out streams over {E2E_BUFFER_SETS} buffer sets; all copies from/to pinned host memory inside the timed region"}

    out = {
        "metric": CONV_METRIC,
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_us * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {0: "fp32", 1: "fp16", 2: "bf16"}[shape.precision] + " (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={shape.batch} C={shape.in_channels} {shape.in_h}x{shape.in_w} K={shape.out_channels} "
                               f"{shape.kernel}x{shape.kernel}/s{shape.stride} p{shape.pad} NCHW, fused bias+ReLU",
                   "step": "one forward call = layout repack + weight prepack + convolution with fused bias + ReLU",
                   "tile": {"tile_m": plan.info.cfg.tile_m, "tile_n": plan.info.cfg.tile_n, "tile_k": plan.info.cfg.tile_k, "stages": plan.info.cfg.stages,
                            "split_k": plan.info.cfg.split_k, "cta_pair": plan.info.cfg.cta_pair == 2,
                            "reduce": {0: "none", 1: "workspace + reduction launch", 2: "cluster (distributed shared memory)"}[plan.info.cfg.reduce]},
                   "cold_cache": f"inputs larger than L2: {res['nsets']} rotating buffer sets, {res['rotation_bytes'] / 1e6:.0f} MB",
                   "launch": "CUDA graphs of one buffer rotation, replayed", "replicas": world,
                   "fp32_tolerance": "relative error <= 1e-5 with the denominator floored at rms(ref) (this build's reading of the bound)"},
        "timing": {"protocol": "5 warm-up replays, then 30 samples, each one CUDA-event pair around >= 1 ms of graph replays; value = median",
                   "step_us_median": step_us, "step_us_p10": proto["p10_us"], "step_us_p90": proto["p90_us"],
                   "steps_per_sample": proto["units_per_sample"],
                   "k_step_region": {"steps": args.steps, "us_per_step": region_us,
                                     "note": "exactly K steps between one event pair after W warm-up steps (barrier and synchronise on both sides)"}},
        "roofline": roof, "e2e": e2e, "gpu_launches": res["launches"], "clocks": clocks,
    }
    del res
    torch.cuda.empty_cache()
    do_cpu = world == 1 and rank == 0 and not args.no_cpu
    if not args.no_secondary:
        # the workload the multi-GPU runs exist for: a first-class block, not part of "secondary"
        out["chain"] = chain_block(torch, pkg, ranks, peaks, args.steps, do_cpu)
        if world == 1:
            sec = {}
            for name in ("c1", "c3_fp16", "c3_bf16", "c4a", "c4b", "c2_fp8"):
                if name == args.workload:
                    continue
                sh, bd = wl.CONV_WORKLOADS[name]
                r2 = time_conv(torch, pkg, sh, 200, 20, 1, lambda: None, float)
                us = r2["proto"]["median_us"]
                cfg2 = r2["plan"].info.cfg
                entry_ = {"us_per_step": us, "us_per_step_p10_p90": [r2["proto"]["p10_us"], r2["proto"]["p90_us"]],
                          "tflops": sh.flops / (us * 1e-6) / 1e12, "kernel_us": r2["kernel"]["median_us"],
                          "repack_us": r2["repack"]["median_us"] if "repack" in r2 else 0.0, "bound": bd,
                          "tile": [cfg2.tile_m, cfg2.tile_n, cfg2.tile_k, cfg2.stages, cfg2.split_k], "cta_pair": cfg2.cta_pair == 2}
                if bd == "hbm":
                    entry_["pipeline_gbs"] = sh.algorithmic_bytes / (us * 1e-6) / 1e9
                    entry_["frac_of_hbm"] = entry_["pipeline_gbs"] / peaks["hbm_gbs"]
                    entry_["kernel_frac_of_hbm"] = sh.algorithmic_bytes / (entry_["kernel_us"] * 1e-6) / 1e9 / peaks["hbm_gbs"]
                elif bd == "tensor":
                    entry_["frac_of_tensor"] = entry_["tflops"] / peaks["bf16_tflops"]
                    entry_["kernel_frac_of_tensor"] = sh.flops / (entry_["kernel_us"] * 1e-6) / 1e12 / peaks["bf16_tflops"]
                sec[name] = entry_
                del r2
                torch.cuda.empty_cache()
            rms = time_rmsnorm(torch, pkg, 300, 10)
            rms["frac_of_hbm"] = rms["gbs"] / peaks["hbm_gbs"]
            sec["rmsnorm_bf16_8192x4096_residual"] = rms
            torch.cuda.empty_cache()
            out["secondary"] = sec
    if do_cpu:
        out["cpu_baseline"] = cpu_baseline_leg(torch, shape, host[:3], host[3])
    if rank == 0:
        print(json.dumps(out))
    ranks.close()


def run_chain_primary(args, torch, pkg, ranks, peaks, peak_kind, local_rank):
    """`--workload chain`: the conv chain as the headline (images/s, batch 256 sharded over the ranks: strong scaling)."""
    sampler = ClockSampler(local_rank)
    sampler.start()
    ch = time_chain(torch, pkg, ranks, steps=args.steps, warmup=args.warmup, global_batch=args.chain_batch, layout=args.layout, tune=args.tune,
                    protocol=not args.profile_run)
    clocks = sampler.stop()
    # a timed region of seconds runs under the power cap: compare it with the sustained GEMM peak, a short one with the burst
    timed_s = ch["ms_per_pass"] * args.steps * 1e-3
    sustained = timed_s > 2.0 and "bf16_tflops_sustained" in peaks
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    peak_kind = f"{peak_kind} ({'sustained' if sustained else 'burst'} cuBLAS bf16; the timed region lasted {timed_s:.1f} s)"
    out = {"metric": f"conv-chain images/s (ResNet-50-shaped FP16 inference chain, batch {args.chain_batch})", "value": ch["images_per_s"], "unit": "images/s",
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
        "impl": "reference", "metric": CONV_METRIC, "value": value, "unit": "TFLOP/s",
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
    ap.add_argument("--workload", default="c2", help="c1 | c2 | c3_fp16 | c3_bf16 | c4a | c4b | stem | chain (c2_fp8 with --profile-run only)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layout", default="nchw", choices=["nchw", "nchw_fused", "nhwc"], help="--workload chain: tensor layout between layers")
    ap.add_argument("--chain-batch", type=int, default=256, help="--workload chain: global batch (256 is the benchmark's; 32 is one replica's share on 8 GPUs)")
    ap.add_argument("--tune", action="store_true", help="--workload chain: measure candidate configurations per layer first")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cfg", default="", help="explicit configuration, comma-separated key=value of tile_m, tile_n, tile_k, stages, split_k, variant, reduce, cta_pair")
    ap.add_argument("--profile-run", action="store_true", help="warm-up and the K-step region only, nothing else (for a run under a profiler)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (other shapes, RMSNorm, conv chain)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
