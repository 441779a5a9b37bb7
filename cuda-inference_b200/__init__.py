"""Python host-side mirror of the C ABI in ``include/gie_b200.h`` (ctypes; no torch types cross the boundary).

The native library ``libgie_b200.so`` is built in-tree by ``build.py``.  Importing this package never falls back to
any other implementation: if the library is missing, loading raises.  Device memory and streams come from the caller
(raw integer device pointers and a ``cudaStream_t`` value), exactly as in the reference's operator API.

Because the directory name contains a hyphen, load the package with ``importlib`` under the module name
``cuda_inference_b200`` (see ``__graft_entry__.load_package``).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgie_b200.so")

# gie::StatusCode values (include/gpu_inference/error.h:16-26 of the reference)
OK, INVALID_ARGUMENT, UNSUPPORTED, WORKSPACE_TOO_SMALL, CUDA_ERROR, INTERNAL = 0, 1, 2, 3, 4, 7
STATUS_NAMES = {0: "ok", 1: "invalid_argument", 2: "unsupported", 3: "workspace_too_small", 4: "cuda_error", 7: "internal"}
# gie::Precision order
FP32, FP16, BF16, TF32 = 0, 1, 2, 3
FP8_E4M3 = 4  # an extension of this library: FP8 E4M3 x and w, float bias, FP16 y (see include/gie_b200.h)
FLAG_BIAS_FP32, FLAG_WEIGHTS_PREPACKED = 1, 2
FLAG_INPUT_NHWC, FLAG_OUTPUT_NHWC, FLAG_RESIDUAL = 4, 8, 16


class GieError(RuntimeError):
    """Mirror of gie::Error: carries the status code of the failed call."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "in_channels", "in_h", "in_w", "out_channels", "kernel_h", "kernel_w", "stride_h", "stride_w",
        "pad_h", "pad_w", "dilation_h", "dilation_w", "groups", "precision", "has_bias", "relu")] + [("flags", C.c_uint32)]


class ConvCfg(C.Structure):
    _fields_ = [("tile_n", C.c_int32), ("tile_k", C.c_int32), ("stages", C.c_int32), ("split_k", C.c_int32),
                ("variant", C.c_int32), ("tile_m", C.c_int32), ("reduce", C.c_int32), ("cta_pair", C.c_int32)]


class ConvInfo(C.Structure):
    _fields_ = [("supported", C.c_int32), ("variant", C.c_int32), ("cfg", ConvCfg), ("workspace_bytes", C.c_uint64),
                ("persistent_bytes", C.c_uint64), ("dynamic_smem_bytes", C.c_uint32), ("threads_per_block", C.c_uint32),
                ("num_blocks", C.c_int64), ("launches", C.c_int32), ("padded_channels", C.c_int32), ("reason", C.c_char * 256)]


class RmsNormDesc(C.Structure):
    _fields_ = [("rows", C.c_int32), ("hidden", C.c_int32), ("eps", C.c_float), ("dtype", C.c_int32), ("flags", C.c_uint32)]


_lib = None


def lib() -> C.CDLL:
    """Loads the native library once; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python {os.path.join(HERE, 'build.py')}` (needs nvcc, no GPU)")
        L = C.CDLL(LIB_PATH)
        vp, i32, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
        L.gieb_last_error.restype = C.c_char_p
        L.gieb_version.restype = i32
        L.gieb_conv_validate.argtypes = [C.POINTER(ConvDesc)]
        L.gieb_conv_query.argtypes = [C.POINTER(ConvDesc), C.POINTER(ConvCfg), i32, C.POINTER(ConvInfo)]
        L.gieb_padded_channels.argtypes = [C.POINTER(ConvDesc), C.POINTER(ConvCfg)]
        L.gieb_conv_plan_create.argtypes = [C.POINTER(ConvDesc), C.POINTER(ConvCfg), i32, C.POINTER(vp)]
        L.gieb_conv_plan_destroy.argtypes = [vp]
        L.gieb_conv_plan_destroy.restype = None
        L.gieb_conv_plan_info.argtypes = [vp, C.POINTER(ConvInfo)]
        L.gieb_conv_launch.argtypes = [vp, vp, vp, vp, vp, vp, sz, vp]
        L.gieb_conv_plan_prepacked_weight_bytes.argtypes = [vp, C.POINTER(C.c_uint64)]
        L.gieb_conv_plan_prepack_weights.argtypes = [vp, vp, vp, vp]
        L.gieb_conv_launch_fused.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, vp]
        L.gieb_conv_launch_stages.argtypes = [vp, C.c_uint, vp, vp, vp, vp, vp, sz, vp]
        L.gieb_conv_time_stages.argtypes = [vp, vp, vp, vp, vp, vp, sz, vp, i32, C.POINTER(C.c_float)]
        L.gieb_conv_forward_static.argtypes = [C.POINTER(ConvDesc), C.POINTER(ConvCfg), vp, vp, vp, vp, vp]
        L.gieb_conv_plan_device_status.argtypes = [vp, C.POINTER(C.c_uint32)]
        L.gieb_conv_static_status.argtypes = [C.POINTER(C.c_uint32), vp]
        L.gieb_conv_plan_inject_stall.argtypes = [vp, C.c_uint32, C.c_uint64]
        L.gieb_repack_nchw_to_nhwc.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        L.gieb_prepack_weights.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        L.gieb_rmsnorm_launch.argtypes = [C.POINTER(RmsNormDesc), vp, vp, vp, vp, vp, vp]
        L.gieb_bias_act_launch.argtypes = [i32, i32, i32, i32, vp, i32, vp, vp]
        L.gieb_maxpool2d_launch.argtypes = [i32] * 8 + [vp, vp, vp]
        L.gieb_maxpool2d_nhwc_launch.argtypes = [i32] * 8 + [vp, vp, vp]
        L.gieb_add_relu_launch.argtypes = [i32, i32, vp, vp, vp, i64, vp]
        _lib = L
    return _lib


def last_error() -> str:
    return lib().gieb_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    if status != OK:
        raise GieError(status, last_error())


@dataclass
class ConvProblem:
    """Mirror of gie::ConvProblem (geometry + precision + fused epilogue), plus the extension flags."""

    batch: int = 1
    in_channels: int = 1
    in_h: int = 1
    in_w: int = 1
    out_channels: int = 1
    kernel_h: int = 1
    kernel_w: int = 1
    stride_h: int = 1
    stride_w: int = 1
    pad_h: int = 0
    pad_w: int = 0
    dilation_h: int = 1
    dilation_w: int = 1
    groups: int = 1
    precision: int = FP32
    has_bias: bool = False
    relu: bool = False
    flags: int = 0

    def desc(self) -> ConvDesc:
        return ConvDesc(self.batch, self.in_channels, self.in_h, self.in_w, self.out_channels, self.kernel_h, self.kernel_w,
                        self.stride_h, self.stride_w, self.pad_h, self.pad_w, self.dilation_h, self.dilation_w, self.groups,
                        int(self.precision), int(self.has_bias), int(self.relu), int(self.flags))

    @property
    def out_h(self) -> int:
        return (self.in_h + 2 * self.pad_h - self.dilation_h * (self.kernel_h - 1) - 1) // self.stride_h + 1

    @property
    def out_w(self) -> int:
        return (self.in_w + 2 * self.pad_w - self.dilation_w * (self.kernel_w - 1) - 1) // self.stride_w + 1

    @property
    def flops(self) -> int:
        return 2 * self.out_channels * self.batch * self.out_h * self.out_w * self.in_channels * self.kernel_h * self.kernel_w


def make_cfg(tile_n=0, tile_k=0, stages=0, split_k=0, variant=0, tile_m=0, reduce=0, cta_pair=0) -> ConvCfg:
    return ConvCfg(tile_n, tile_k, stages, split_k, variant, tile_m, reduce, cta_pair)


def validate_problem(p: ConvProblem) -> None:
    """gie::validate_problem: raises GieError(INVALID_ARGUMENT / UNSUPPORTED)."""
    check(lib().gieb_conv_validate(C.byref(p.desc())))


def query(p: ConvProblem, cfg: ConvCfg | None = None, device: int = -1) -> ConvInfo:
    info = ConvInfo()
    check(lib().gieb_conv_query(C.byref(p.desc()), C.byref(cfg) if cfg is not None else None, device, C.byref(info)))
    return info


class ConvPlan:
    """Mirror of gie::ExecutionPlan for the one sm_100a kernel family: create once, launch many times."""

    def __init__(self, problem: ConvProblem, cfg: ConvCfg | None = None, device: int = -1):
        self.problem = problem
        self._h = C.c_void_p()
        check(lib().gieb_conv_plan_create(C.byref(problem.desc()), C.byref(cfg) if cfg is not None else None, device,
                                          C.byref(self._h)))
        self.info = ConvInfo()
        check(lib().gieb_conv_plan_info(self._h, C.byref(self.info)))

    @property
    def workspace_bytes(self) -> int:
        return int(self.info.workspace_bytes)

    def launch(self, x: int, w: int, bias: int | None, y: int, workspace: int | None, workspace_bytes: int, stream: int = 0) -> None:
        """execute_unchecked: raw device pointers, asynchronous on `stream`."""
        check(lib().gieb_conv_launch(self._h, x, w, bias, y, workspace, workspace_bytes, stream))

    @property
    def prepacked_weight_bytes(self) -> int:
        v = C.c_uint64()
        check(lib().gieb_conv_plan_prepacked_weight_bytes(self._h, C.byref(v)))
        return int(v.value)

    def prepack_weights(self, w: int, dst: int, stream: int = 0) -> None:
        """OIHW weights -> the layout this plan's kernel reads (for problems with FLAG_WEIGHTS_PREPACKED)."""
        check(lib().gieb_conv_plan_prepack_weights(self._h, w, dst, stream))

    def launch_fused(self, x: int, w: int, bias: int | None, residual: int, y: int, workspace: int | None, workspace_bytes: int,
                     stream: int = 0) -> None:
        """launch() with a residual tensor (shape, layout and type of y) added before the activation; for plans whose
        problem carries FLAG_RESIDUAL."""
        check(lib().gieb_conv_launch_fused(self._h, x, w, bias, residual, y, workspace, workspace_bytes, stream))

    def launch_stages(self, stage_mask: int, x: int, w: int, bias: int | None, y: int, workspace: int | None, workspace_bytes: int,
                      stream: int = 0) -> None:
        """launch() restricted to some stages (bit 0 repack + prepack, bit 1 convolution kernel, bit 2 split-K reduction);
        without bit 0 the workspace must hold the repacked tensors of an earlier full launch.  For measurements."""
        check(lib().gieb_conv_launch_stages(self._h, stage_mask, x, w, bias, y, workspace, workspace_bytes, stream))

    def time_stages(self, x, w, bias, y, workspace, workspace_bytes, stream=0, iters=100):
        """Average milliseconds per call of (repack + prepack, convolution kernel, split-K reduction)."""
        ms = (C.c_float * 3)()
        check(lib().gieb_conv_time_stages(self._h, x, w, bias, y, workspace, workspace_bytes, stream, iters, ms))
        return float(ms[0]), float(ms[1]), float(ms[2])

    def device_status(self) -> int:
        v = C.c_uint32()
        check(lib().gieb_conv_plan_device_status(self._h, C.byref(v)))
        return int(v.value)

    def inject_stall(self, roles: int, wait_limit_cycles: int) -> None:
        """Test hook: later launches skip the given roles (bit 0 producers, bit 1 MMA issuer) and every device-side wait
        gives up after `wait_limit_cycles` SM cycles; roles = 0 restores normal behaviour."""
        check(lib().gieb_conv_plan_inject_stall(self._h, roles, wait_limit_cycles))

    def close(self) -> None:
        if self._h:
            lib().gieb_conv_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def conv_forward_static(problem: ConvProblem, x: int, w: int, bias: int | None, y: int, stream: int = 0,
                        cfg: ConvCfg | None = None) -> None:
    """Forward call for callers that must not allocate device memory: uses the 8 MiB scratch built into the library
    instead of a plan and a workspace.  Calls that overlap on the GPU race on that scratch; larger problems raise
    GieError(WORKSPACE_TOO_SMALL)."""
    check(lib().gieb_conv_forward_static(C.byref(problem.desc()), C.byref(cfg) if cfg is not None else None, x, w, bias, y, stream))


def conv_static_status(stream: int = 0) -> int:
    """Status word of the last conv_forward_static call on the current device (waits for `stream`): 0 = every bounded
    device-side wait was satisfied, so y is complete.  Allocates nothing."""
    v = C.c_uint32()
    check(lib().gieb_conv_static_status(C.byref(v), stream))
    return int(v.value)


def repack_nchw_to_nhwc(src: int, dst: int, batch: int, channels: int, hw: int, c_padded: int, stream: int = 0) -> None:
    check(lib().gieb_repack_nchw_to_nhwc(src, dst, batch, channels, hw, c_padded, stream))


def prepack_weights(src: int, dst: int, out_channels: int, channels: int, rs: int, c_padded: int, stream: int = 0) -> None:
    check(lib().gieb_prepack_weights(src, dst, out_channels, channels, rs, c_padded, stream))


def rmsnorm_forward(rows: int, hidden: int, eps: float, dtype: int, x: int, gamma: int, y: int, residual_in: int | None = None,
                    residual_out: int | None = None, stream: int = 0, gamma_fp32: bool = False) -> None:
    """gie::rmsnorm_forward on raw device pointers; dtype uses gie::DataType order (0 fp32, 1 fp16, 2 bf16)."""
    d = RmsNormDesc(rows, hidden, eps, dtype, 1 if gamma_fp32 else 0)
    check(lib().gieb_rmsnorm_launch(C.byref(d), x, gamma, y, residual_in, residual_out, stream))


def bias_act(precision: int, batch: int, channels: int, hw: int, bias: int | None, relu: bool, y: int, stream: int = 0) -> None:
    check(lib().gieb_bias_act_launch(precision, batch, channels, hw, bias, int(relu), y, stream))


def maxpool2d(precision: int, batch: int, channels: int, h: int, w: int, kernel: int, stride: int, pad: int, x: int, y: int,
              stream: int = 0) -> None:
    check(lib().gieb_maxpool2d_launch(precision, batch, channels, h, w, kernel, stride, pad, x, y, stream))


def maxpool2d_nhwc(precision: int, batch: int, channels: int, h: int, w: int, kernel: int, stride: int, pad: int, x: int, y: int,
                   stream: int = 0) -> None:
    """maxpool2d on channel-contiguous [B][H][W][C] tensors (fp16 / bf16, C % 8 == 0)."""
    check(lib().gieb_maxpool2d_nhwc_launch(precision, batch, channels, h, w, kernel, stride, pad, x, y, stream))


def add_relu(precision: int, relu: bool, a: int, b: int, y: int, n: int, stream: int = 0) -> None:
    check(lib().gieb_add_relu_launch(precision, int(relu), a, b, y, n, stream))
