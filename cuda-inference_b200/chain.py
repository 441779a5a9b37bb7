"""The ResNet-50-shaped convolution chain as a sequence of C-ABI launches (convolutions with fused bias + ReLU, one
max-pool, residual adds), enqueued on a caller's stream and capturable as ONE CUDA graph.

Device buffers come from torch (plumbing only); every kernel that runs is this library's.  One ``ConvChain`` lives on
one GPU; multi-GPU runs are independent replicas over a batch shard (no collective, no peer access)."""
from __future__ import annotations

import math

from . import (ConvPlan, ConvProblem, GieError, add_relu, make_cfg, maxpool2d, maxpool2d_nhwc, FLAG_INPUT_NHWC, FLAG_OUTPUT_NHWC,
               FLAG_RESIDUAL, FLAG_WEIGHTS_PREPACKED)
from .workloads import FP16, BF16, chain_flops, fuse_residuals, resnet50_chain


def _torch():
    import torch
    return torch


def shard_batch(global_batch: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous batch shard of `rank`: (first image, image count).  Earlier ranks take the remainder."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, rem = divmod(global_batch, world)
    count = base + (1 if rank < rem else 0)
    first = rank * base + min(rank, rem)
    return first, count


def layer_weight_bound(shape, relu: bool) -> float:
    """Kaiming-uniform bound for a layer followed by ReLU (gain sqrt 2); layers without ReLU (block outputs and
    projection shortcuts, i.e. where a folded batch-norm would sit) use gain 1 / 0.5 so activations stay in FP16
    range through 16 residual blocks."""
    fan_in = shape.in_channels * shape.kernel * shape.kernel
    return math.sqrt(6.0 / fan_in) if relu else 0.5 * math.sqrt(3.0 / fan_in)


def candidate_cfgs(out_channels: int):
    """Configuration points tried per layer when a chain is built with tune=True: the heuristic's own pick (None) plus
    tile shapes and ring depths around it.  Unsupported points are skipped by plan creation."""
    cfgs = [None]
    for tile_m in (128, 256):
        for tile_n in (64, 128, 256):
            if tile_n > 64 and tile_n // 2 >= out_channels:
                continue
            for stages in (2, 3, 4, 6):
                cfgs.append(dict(tile_m=tile_m, tile_n=tile_n, stages=stages, cta_pair=1))
    for tile_n in (128, 256):  # 256-pixel tiles computed by CTA pairs (the ring takes what shared memory is left)
        if tile_n // 2 < out_channels:
            cfgs.append(dict(tile_n=tile_n, cta_pair=2))
    return cfgs


_TUNED: dict = {}  # (problem fields, flags) -> best cfg kwargs (or None), per process


def tuned_configs() -> dict:
    """The configurations measured so far in this process (picklable: send it to the other replicas)."""
    return dict(_TUNED)


def set_tuned_configs(table: dict) -> None:
    """Adopts configurations measured elsewhere (rank 0 of a multi-GPU run), so that every replica runs the same kernels."""
    _TUNED.update(table)


class ConvChain:
    def __init__(self, batch: int, precision: int = FP16, image: int = 224, seed: int = 0, weights=None, device=None,
                 layout: str = "nchw", tune: bool = False, fuse_residual: bool | None = None):
        """weights: optional list of (w, b) host numpy arrays in storage bit patterns per convolution, in the order of
        resnet50_chain (tests); when None, weights are generated on the device from `seed` + layer index with the
        benchmark distributions.
        layout "nchw": every tensor NCHW (the reference API's tensor contract, layer by layer); the weights, which the chain
        owns, are converted once at construction, so a layer's repack launch rearranges activations only.
        layout "nhwc": the input image stays NCHW; every later tensor is channel-contiguous, weights are prepacked once
        at construction, and each block's residual add + ReLU runs inside the epilogue of its last convolution
        (no repack launches, no add launches).
        fuse_residual: each block's residual add + ReLU inside the epilogue of its last convolution (always in the nhwc
        layout; in the nchw layout an option, default off: the unfused chain is the reference API's operator set layer by
        layer, the fused one needs the residual operand this library adds to it).
        tune: time candidate_cfgs() for every distinct layer on this GPU (a few launches each, on scratch buffers of the
        chain) and build each plan with the fastest; the choice is remembered per process."""
        torch = _torch()
        self.torch = torch
        if layout not in ("nchw", "nhwc"):
            raise ValueError("layout must be 'nchw' or 'nhwc'")
        self.layout = layout
        self.batch, self.precision, self.image = batch, precision, image
        self.dtype = torch.float16 if precision == FP16 else torch.bfloat16
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        base_ops, self.slot_shapes = resnet50_chain(batch, precision, image)
        nhwc = layout == "nhwc"
        self.base_ops = base_ops  # the unfused layer list (convolutions, max-pool, residual adds)
        self.oihw_weights = []    # OIHW weights per entry of self.convs, as generated (the nhwc layout launches converted copies)
        base_relu = {op.layer: op.relu for op in base_ops if op.kind == "conv"}
        self.fused = True if nhwc else bool(fuse_residual)
        self.ops = fuse_residuals(base_ops) if self.fused else base_ops
        self.flops = chain_flops(self.ops)
        self.slots = {i: torch.empty(batch * c * h * w, dtype=self.dtype, device=self.device) for i, (c, h, w) in self.slot_shapes.items()}
        self.convs = []  # (op, plan, w, b) in launch order; w is prepacked in the nhwc layout
        ws_bytes = 256
        for op in self.ops:
            if op.kind != "conv":
                continue
            s = op.shape
            li = op.layer
            # the chain owns its weights: they are converted once, here, to the layout each plan's kernel reads
            flags = FLAG_WEIGHTS_PREPACKED | (FLAG_RESIDUAL if (self.fused and op.other >= 0) else 0)
            if nhwc:
                flags = FLAG_OUTPUT_NHWC | FLAG_WEIGHTS_PREPACKED
                if op.src != 0:
                    flags |= FLAG_INPUT_NHWC  # the image itself (3 channels) stays NCHW and is repacked by the stem
                if op.other >= 0:
                    flags |= FLAG_RESIDUAL
            problem = ConvProblem(s.batch, s.in_channels, s.in_h, s.in_w, s.out_channels, s.kernel, s.kernel, s.stride, s.stride,
                                  s.pad, s.pad, 1, 1, 1, precision, True, op.relu, flags)
            plan = self._tuned_plan(problem, op) if tune else ConvPlan(problem)
            if weights is not None:
                import numpy as np
                w = torch.from_numpy(weights[li][0].view(np.int16)).to(self.device).view(self.dtype)
                b = torch.from_numpy(weights[li][1].view(np.int16)).to(self.device).view(self.dtype)
            else:
                g = torch.Generator(device=self.device)
                g.manual_seed(seed + li)
                # a layer followed by ReLU (directly, or through the block's residual add) draws with gain sqrt(2)
                bound = layer_weight_bound(s, base_relu[li])
                w = ((torch.rand(s.w_elems, device=self.device, generator=g) * 2 - 1) * bound).to(self.dtype)
                b = ((torch.rand(s.out_channels, device=self.device, generator=g) * 2 - 1) * 0.1).to(self.dtype)
            self.oihw_weights.append(w)
            wp = torch.empty(plan.prepacked_weight_bytes // 2, dtype=self.dtype, device=self.device)
            plan.prepack_weights(w.data_ptr(), wp.data_ptr(), torch.cuda.current_stream().cuda_stream)
            w = wp
            self.convs.append((op, plan, w, b))
            ws_bytes = max(ws_bytes, plan.workspace_bytes)
        torch.cuda.current_stream().synchronize()
        self._ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=self.device)
        self.ws_ptr = (self._ws.data_ptr() + 255) // 256 * 256
        self.ws_bytes = ws_bytes
        self.launches = sum(p.info.launches for _, p, _, _ in self.convs) + sum(1 for op in self.ops if op.kind != "conv")
        self.graph = None

    def _tuned_plan(self, problem: ConvProblem, op) -> ConvPlan:
        """The fastest of candidate_cfgs() for this layer, measured with CUDA events on the chain's own buffers."""
        torch = self.torch
        key = (problem.batch, problem.in_channels, problem.in_h, problem.in_w, problem.out_channels, problem.kernel_h, problem.stride_h,
               problem.precision, problem.relu, problem.flags)
        if key in _TUNED:
            kw = _TUNED[key]
            return ConvPlan(problem, make_cfg(**kw) if kw else None)
        s = op.shape
        x, y = self.slots[op.src], self.slots[op.dst]
        res = self.slots[op.other] if op.other >= 0 else y
        w = torch.zeros(s.w_elems * 4 + 4096, dtype=self.dtype, device=self.device)  # room for any padded layout
        b = torch.zeros(s.out_channels, dtype=self.dtype, device=self.device)
        stream = torch.cuda.current_stream().cuda_stream
        best, best_kw, best_ms = None, None, float("inf")
        for kw in candidate_cfgs(s.out_channels):
            try:
                plan = ConvPlan(problem, make_cfg(**kw) if kw else None)
            except GieError:
                continue
            ws = torch.empty(plan.workspace_bytes + 256, dtype=torch.uint8, device=self.device)
            wsp = (ws.data_ptr() + 255) // 256 * 256

            def go():
                if problem.flags & FLAG_RESIDUAL:
                    plan.launch_fused(x.data_ptr(), w.data_ptr(), b.data_ptr(), res.data_ptr(), y.data_ptr(), wsp, plan.workspace_bytes, stream)
                else:
                    plan.launch(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), wsp, plan.workspace_bytes, stream)

            go()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                go()
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            if plan.device_status() == 0 and ms < best_ms:
                best, best_kw, best_ms = plan, kw, ms
            del ws
        if best is None:
            raise RuntimeError("no configuration could run this layer")
        _TUNED[key] = best_kw
        return best

    @property
    def input(self):
        return self.slots[0]

    @property
    def output(self):
        return self.slots[len(self.slots) - 1]

    def enqueue(self, stream: int) -> None:
        """All launches of one forward pass on `stream` (capture-safe: no allocation, no synchronisation)."""
        ci = 0
        for op in self.ops:
            if op.kind == "conv":
                _, plan, w, b = self.convs[ci]
                ci += 1
                if op.other >= 0 and self.fused:
                    plan.launch_fused(self.slots[op.src].data_ptr(), w.data_ptr(), b.data_ptr(), self.slots[op.other].data_ptr(),
                                      self.slots[op.dst].data_ptr(), self.ws_ptr, self.ws_bytes, stream)
                else:
                    plan.launch(self.slots[op.src].data_ptr(), w.data_ptr(), b.data_ptr(), self.slots[op.dst].data_ptr(), self.ws_ptr,
                                self.ws_bytes, stream)
            elif op.kind == "maxpool":
                c, h, w, k, s, p = op.pool
                pool = maxpool2d_nhwc if self.layout == "nhwc" else maxpool2d
                pool(self.precision, self.batch, c, h, w, k, s, p, self.slots[op.src].data_ptr(), self.slots[op.dst].data_ptr(), stream)
            else:
                n = self.slots[op.dst].numel()
                add_relu(self.precision, op.relu, self.slots[op.src].data_ptr(), self.slots[op.other].data_ptr(),
                         self.slots[op.dst].data_ptr(), n, stream)

    def capture(self, stream) -> None:
        """Runs the chain once eagerly on `stream` (a torch.cuda.Stream), then captures it as one CUDA graph."""
        torch = self.torch
        with torch.cuda.stream(stream):
            self.enqueue(stream.cuda_stream)
            stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                self.enqueue(torch.cuda.current_stream().cuda_stream)

    def replay(self) -> None:
        self.graph.replay()

    def device_status(self) -> int:
        st = 0
        for _, plan, _, _ in self.convs:
            st |= plan.device_status()
        return st
