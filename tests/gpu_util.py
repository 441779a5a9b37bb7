"""Helpers for the GPU parity tests: device buffers via torch (plumbing only), launches through the C ABI."""
from __future__ import annotations

import numpy as np

GUARD = 128  # guard-band elements on both sides of every output buffer


def torch_mod():
    import torch
    return torch


def to_device_storage(o, precision, host_f32, offset_elems=0):
    """Uploads host float values as the raw storage array (fp32, or 16-bit patterns).  With offset_elems the returned
    pointer is offset by that many elements inside a larger allocation (mis-alignment tests)."""
    torch = torch_mod()
    raw = o.to_storage(precision, np.ascontiguousarray(host_f32).ravel())
    if raw.dtype == np.uint16:
        raw = raw.view(np.int16)
    t = torch.empty(raw.size + offset_elems + 8, dtype=torch.from_numpy(raw[:1]).dtype, device="cuda")
    t[offset_elems:offset_elems + raw.size] = torch.from_numpy(raw).cuda()
    return t, t.data_ptr() + offset_elems * t.element_size()


class OutBuf:
    """Output buffer poisoned with 0xFF bytes (a NaN pattern in every supported type) and fenced by guard bands."""

    def __init__(self, precision, numel, offset_elems=0):
        torch = torch_mod()
        self.precision = precision
        self.numel = numel
        self.dtype = torch.float32 if precision in (0, 3) else torch.int16
        self.off = GUARD + offset_elems
        self.t = torch.empty(numel + 2 * GUARD + offset_elems + 8, dtype=self.dtype, device="cuda")
        self.t.view(torch.uint8).fill_(0xFF)
        self.ptr = self.t.data_ptr() + self.off * self.t.element_size()

    def read(self, o) -> np.ndarray:
        raw = self.t.cpu().numpy()
        body = raw[self.off:self.off + self.numel]
        lo, hi = raw[:self.off], raw[self.off + self.numel:]
        assert np.all(lo.view(np.uint8) == 0xFF) and np.all(hi.view(np.uint8) == 0xFF), "guard band overwritten"
        if body.dtype == np.int16:
            return o.from_bits16(self.precision, body.view(np.uint16))
        return body.astype(np.float32, copy=True)

    def raw_bits(self) -> np.ndarray:
        return self.t.cpu().numpy()[self.off:self.off + self.numel].copy()


class Workspace:
    def __init__(self, nbytes):
        torch = torch_mod()
        self.nbytes = int(nbytes)
        self.t = torch.empty(self.nbytes + 512 + 256, dtype=torch.uint8, device="cuda")
        self.t.fill_(0xFF)
        base = self.t.data_ptr()
        self.ptr = (base + 255) // 256 * 256
        self.lead = self.ptr - base

    def check_guard(self):
        raw = self.t.cpu().numpy()
        assert np.all(raw[:self.lead] == 0xFF) and np.all(raw[self.lead + self.nbytes:] == 0xFF), "workspace overrun"


def pkg_problem(pkg, p, flags=0):
    return pkg.ConvProblem(p.batch, p.in_channels, p.in_h, p.in_w, p.out_channels, p.kernel_h, p.kernel_w, p.stride_h,
                           p.stride_w, p.pad_h, p.pad_w, p.dilation_h, p.dilation_w, p.groups, p.precision, p.has_bias,
                           p.relu, flags)


def run_conv(pkg, o, p, x, w, b, cfg=None, flags=0, offsets=(0, 0, 0), repeats=1, plan=None):
    """One forward through gieb_conv_launch; returns (output as float32 array of p.y_shape, plan)."""
    torch = torch_mod()
    stream = torch.cuda.current_stream().cuda_stream
    own = plan is None
    if plan is None:
        plan = pkg.ConvPlan(pkg_problem(pkg, p, flags), cfg)
    bias_prec = 0 if (flags & pkg.FLAG_BIAS_FP32) else p.precision
    tx, px = to_device_storage(o, p.precision, x, offsets[0])
    tw, pw = to_device_storage(o, p.precision, w, offsets[1])
    tb, pb = to_device_storage(o, bias_prec, b if b is not None else np.zeros(p.out_channels, np.float32))
    out = OutBuf(p.precision, int(np.prod(p.y_shape)), offsets[2])
    ws = Workspace(plan.workspace_bytes)
    for _ in range(repeats):
        plan.launch(px, pw, pb if p.has_bias else None, out.ptr, ws.ptr if plan.workspace_bytes else None,
                    plan.workspace_bytes, stream)
    torch.cuda.synchronize()
    assert plan.device_status() == 0, "a bounded device-side wait expired"
    ws.check_guard()
    y = out.read(o).reshape(p.y_shape)
    del tx, tw, tb
    return y, plan, out


def describe_mismatch(p, got, ref, scale, tolfn):
    """Short diagnostic: where the worst elements are (helps telling layout bugs from rounding)."""
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    bad = np.argwhere(~(err <= tolfn(ref, scale)) | ~np.isfinite(got))
    lines = [f"{len(bad)} bad of {got.size}; first: "]
    for idx in bad[:12]:
        idx = tuple(idx)
        lines.append(f"  y{idx}: got {got[idx]!r} ref {ref[idx]!r}")
    if len(bad):
        for ax, name in enumerate("bohw"):
            vals = np.unique(bad[:, ax])
            lines.append(f"  bad {name}: {vals[:24].tolist()}{'...' if len(vals) > 24 else ''} ({len(vals)} distinct)")
    return "\n".join(lines)
