"""ctypes bindings for the TEST oracle (never imported by the product).

Two libraries live beside this file:
  * ``libgie_oracle.so``      -- the C restatement in ``gie_oracle.c`` (always available; ``make -C oracle``)
  * ``_ref/libgie_ref.so``    -- the reference library's own oracle sources compiled unmodified
                                 (``make -C oracle ref``; only buildable where the reference checkout exists)

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libgie_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libgie_ref.so")

FP32, FP16, BF16, TF32 = 0, 1, 2, 3
PRECISION_NAMES = {FP32: "fp32", FP16: "fp16", BF16: "bf16", TF32: "tf32"}
DIST_UNIFORM, DIST_NORMAL, DIST_SPARSE, DIST_POSITIVE = 0, 1, 2, 3

OK, INVALID_ARGUMENT, UNSUPPORTED, WORKSPACE_TOO_SMALL, CUDA_ERROR = 0, 1, 2, 3, 4


class ConvDesc(C.Structure):
    """Field order shared by gie_oracle.c (orc_conv_desc) and ref_shim.cpp (Desc)."""

    _fields_ = [(n, C.c_int32) for n in (
        "batch", "in_channels", "in_h", "in_w", "out_channels", "kernel_h", "kernel_w",
        "stride_h", "stride_w", "pad_h", "pad_w", "dilation_h", "dilation_w", "groups",
        "precision", "has_bias", "relu")]


@dataclass
class Problem:
    """One convolution problem: geometry + storage precision + fused epilogue."""

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

    @staticmethod
    def P(B, Cin, H, W, O, Kh, Kw, Sh, Sw, Ph, Pw, precision=FP32, bias=False, relu=False) -> "Problem":
        """Same positional order as the reference tests' shape helper (tests/shapes.h:18-24)."""
        return Problem(B, Cin, H, W, O, Kh, Kw, Sh, Sw, Ph, Pw, 1, 1, 1, precision, bias, relu)

    def desc(self) -> ConvDesc:
        return ConvDesc(self.batch, self.in_channels, self.in_h, self.in_w, self.out_channels, self.kernel_h,
                        self.kernel_w, self.stride_h, self.stride_w, self.pad_h, self.pad_w, self.dilation_h,
                        self.dilation_w, self.groups, int(self.precision), int(self.has_bias), int(self.relu))

    @staticmethod
    def _cdiv(a: int, b: int) -> int:
        """C integer division (truncation toward zero), as in the reference's int arithmetic."""
        q = abs(a) // abs(b)
        return q if (a >= 0) == (b >= 0) else -q

    @property
    def out_h(self) -> int:
        return self._cdiv(self.in_h + 2 * self.pad_h - self.dilation_h * (self.kernel_h - 1) - 1, self.stride_h) + 1

    @property
    def out_w(self) -> int:
        return self._cdiv(self.in_w + 2 * self.pad_w - self.dilation_w * (self.kernel_w - 1) - 1, self.stride_w) + 1

    @property
    def x_shape(self):
        return (self.batch, self.in_channels, self.in_h, self.in_w)

    @property
    def w_shape(self):
        return (self.out_channels, self.in_channels, self.kernel_h, self.kernel_w)

    @property
    def y_shape(self):
        return (self.batch, self.out_channels, self.out_h, self.out_w)

    @property
    def gemm_k(self) -> int:
        return self.in_channels * self.kernel_h * self.kernel_w

    @property
    def flops(self) -> int:
        return 2 * self.out_channels * self.batch * self.out_h * self.out_w * self.gemm_k

    @property
    def elem_size(self) -> int:
        return 2 if self.precision in (FP16, BF16) else 4

    def algorithmic_bytes(self) -> int:
        """X + W + Y + bias, each once, in the storage type."""
        n = int(np.prod(self.x_shape)) + int(np.prod(self.w_shape)) + int(np.prod(self.y_shape))
        if self.has_bias:
            n += self.out_channels
        return n * self.elem_size


class Tolerance(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("c_acc", "c_out", "c_inter", "c_in", "u_in", "u_acc", "u_out", "abs_floor")] + [
        ("k", C.c_int64)]


class Metrics(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("n", "over_tol", "nan_count", "inf_count")] + [
        (n, C.c_double) for n in ("max_abs", "mean_abs", "rms", "max_rel", "frac_over_tol", "worst_tol_ratio")]

    def passed(self) -> bool:
        return self.n > 0 and self.nan_count == 0 and self.inf_count == 0 and self.over_tol == 0

    def summary(self) -> str:
        return (f"max_abs={self.max_abs:.3e} rms={self.rms:.3e} max_rel={self.max_rel:.3e} over_tol={self.over_tol}/{self.n} "
                f"worst_tol_ratio={self.worst_tol_ratio:.3f} nan={self.nan_count} inf={self.inf_count}")


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: np.ndarray | None, ty=C.c_float):
    return None if a is None else a.ctypes.data_as(C.POINTER(ty))


def e4m3_quantize(a) -> np.ndarray:
    """Values rounded to FP8 E4M3 (the 8-bit format of the OCP 8-bit floating point specification: 1 sign, 4 exponent bits
    with bias 7, 3 mantissa bits, no infinities, largest finite value 448): round to nearest even, saturating at +-448.  The
    reference has no FP8 path; this grid is what the FP8 extension of the library under test stores, and every value
    on it is also an FP16 value, so the FP16 oracle applies to tensors quantized with it."""
    x = np.asarray(a, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    _, e = np.frexp(mag)                       # mag = m * 2**e with m in [0.5, 1)
    exp = np.clip(e - 1, -6, 8)                # exponent of the leading bit; subnormals share the step of 2**-6
    step = np.ldexp(1.0, exp - 3)
    q = np.minimum(np.rint(mag / step) * step, 448.0)
    return np.copysign(q, x).astype(np.float32)


def e4m3_bits(q) -> np.ndarray:
    """Bit patterns (uint8) of values that already lie on the E4M3 grid."""
    x = np.asarray(q, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    _, e = np.frexp(mag)
    exp = np.clip(e - 1, -6, 8)
    normal = mag >= 2.0 ** -6
    mant = np.where(normal, mag / np.ldexp(1.0, exp) * 8.0 - 8.0, mag / 2.0 ** -9)
    biased = np.where(normal, exp + 7, 0)
    bits = (np.signbit(x).astype(np.uint8) << 7) | (biased.astype(np.uint8) << 3) | np.rint(mant).astype(np.uint8)
    return bits.astype(np.uint8)


def build(ref: bool = True, quiet: bool = True) -> None:
    """Compile the C restatement and, where the reference checkout exists, the reference's own oracle."""
    out = subprocess.DEVNULL if quiet else None
    subprocess.check_call(["make", "-C", HERE], stdout=out)
    if ref and os.path.isdir(os.environ.get("GIE_REFERENCE_DIR", "/root/reference")):
        subprocess.check_call(["make", "-C", HERE, "ref", "REF=" + os.environ.get("GIE_REFERENCE_DIR", "/root/reference")],
                              stdout=out)


class Oracle:
    """The C restatement (gie_oracle.c)."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build(ref=False)
        self.lib = C.CDLL(path)
        L = self.lib
        L.orc_validate.argtypes = [C.POINTER(ConvDesc)]
        L.orc_conv2d.argtypes = [C.POINTER(ConvDesc)] + [C.POINTER(C.c_float)] * 5
        L.orc_flops.argtypes = [C.POINTER(ConvDesc)]
        L.orc_flops.restype = C.c_int64
        L.orc_out_h.argtypes = [C.POINTER(ConvDesc)]
        L.orc_out_w.argtypes = [C.POINTER(ConvDesc)]
        L.orc_rng_next_u64.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_next_u64.restype = C.c_uint64
        L.orc_fill_dist.argtypes = [C.POINTER(C.c_uint64), C.c_int, C.c_float, C.POINTER(C.c_float), C.c_int64]
        L.orc_fill_uniform.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_float, C.POINTER(C.c_float), C.c_int64]
        L.orc_quantize.argtypes = [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int64]
        L.orc_to_bits16.argtypes = [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_uint16), C.c_int64]
        L.orc_from_bits16.argtypes = [C.c_int, C.POINTER(C.c_uint16), C.POINTER(C.c_float), C.c_int64]
        L.orc_tolerance_for.argtypes = [C.POINTER(ConvDesc), C.c_int, C.POINTER(Tolerance)]
        L.orc_compare.argtypes = [C.POINTER(C.c_float)] * 3 + [C.c_int64, C.POINTER(Tolerance), C.POINTER(Metrics)]
        L.orc_rmsnorm.argtypes = [C.c_int64, C.c_int64, C.c_double, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float),
                                  C.POINTER(C.c_float), C.POINTER(C.c_double), C.POINTER(C.c_float)]
        L.orc_maxpool2d.argtypes = [C.c_int] * 10 + [C.POINTER(C.c_float)] * 2
        L.orc_add_relu.argtypes = [C.c_int, C.c_int] + [C.POINTER(C.c_float)] * 3 + [C.c_int64]
        L.orc_set_num_threads.argtypes = [C.c_int]

    # -- problem helpers -------------------------------------------------------------------------
    def validate(self, p: Problem) -> int:
        return self.lib.orc_validate(C.byref(p.desc()))

    def num_threads(self) -> int:
        return self.lib.orc_num_threads()

    def set_num_threads(self, n: int) -> None:
        self.lib.orc_set_num_threads(n)

    # -- convolution -----------------------------------------------------------------------------
    def conv2d(self, p: Problem, x, w, bias=None, want_scale=True):
        d = p.desc()
        st = self.lib.orc_validate(C.byref(d))
        if st != OK:
            raise ValueError(f"oracle rejected problem with status {st}")
        x, w = _f32(x), _f32(w)
        b = _f32(bias) if (bias is not None and p.has_bias) else None
        y = np.empty(p.y_shape, np.float32)
        sc = np.empty(p.y_shape, np.float32) if want_scale else None
        st = self.lib.orc_conv2d(C.byref(d), _ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(sc))
        assert st == OK
        return y, sc

    # -- random data -----------------------------------------------------------------------------
    class Rng:
        def __init__(self, lib, seed: int):
            self.lib = lib
            self.state = C.c_uint64(seed)

        def next_u64(self) -> int:
            return self.lib.orc_rng_next_u64(C.byref(self.state))

        def draw(self, dist: int, n: int, mul: float = 1.0) -> np.ndarray:
            out = np.empty(n, np.float32)
            self.lib.orc_fill_dist(C.byref(self.state), dist, C.c_float(mul), _ptr(out), n)
            return out

        def uniform(self, lo: float, hi: float, n: int) -> np.ndarray:
            out = np.empty(n, np.float32)
            self.lib.orc_fill_uniform(C.byref(self.state), C.c_float(lo), C.c_float(hi), _ptr(out), n)
            return out

    def rng(self, seed: int) -> "Oracle.Rng":
        return Oracle.Rng(self.lib, seed)

    def quantize(self, precision: int, a) -> np.ndarray:
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.orc_quantize(precision, _ptr(a), _ptr(out), a.size)
        return out

    def to_bits16(self, precision: int, a) -> np.ndarray:
        a = _f32(a)
        out = np.empty(a.shape, np.uint16)
        self.lib.orc_to_bits16(precision, _ptr(a), _ptr(out, C.c_uint16), a.size)
        return out

    def from_bits16(self, precision: int, a) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.uint16)
        out = np.empty(a.shape, np.float32)
        self.lib.orc_from_bits16(precision, _ptr(a, C.c_uint16), _ptr(out), a.size)
        return out

    def to_storage(self, precision: int, a) -> np.ndarray:
        """Host float values -> the raw array a device tensor of this precision holds."""
        return _f32(a) if precision in (FP32, TF32) else self.to_bits16(precision, a)

    def from_storage(self, precision: int, a) -> np.ndarray:
        return _f32(a) if precision in (FP32, TF32) else self.from_bits16(precision, a)

    def make_conv_data(self, p: Problem, seed: int, dist: int = DIST_UNIFORM):
        """The reference generator (src/runtime/testing.cu:75-99): x, then w*sqrt(3/K), then bias U(-1,1),
        all rounded to the storage precision (bias only for 16-bit storage)."""
        r = self.rng(seed)
        nx, nw = int(np.prod(p.x_shape)), int(np.prod(p.w_shape))
        x = r.draw(dist, nx)
        wscale = np.sqrt(np.float32(3.0) / np.float32(p.gemm_k), dtype=np.float32)
        w = r.draw(dist, nw, float(wscale))
        b = r.uniform(-1.0, 1.0, p.out_channels)
        x = self.quantize(p.precision, x).reshape(p.x_shape)
        w = self.quantize(p.precision, w).reshape(p.w_shape)
        if p.precision in (FP16, BF16):
            b = self.quantize(p.precision, b)
        return x, w, b

    def make_baseline_data(self, p: Problem, seed: int = 0, normal_input: bool = False):
        """The benchmark configurations' distributions: x ~ U[-1,1] (or N(0,1)), w ~ Kaiming-uniform with
        bound sqrt(6/fan_in), bias ~ U[-0.1,0.1]; one SplitMix64 stream, order x -> w -> bias; rounded to storage."""
        r = self.rng(seed)
        nx, nw = int(np.prod(p.x_shape)), int(np.prod(p.w_shape))
        x = r.draw(DIST_NORMAL if normal_input else DIST_UNIFORM, nx)
        bound = np.sqrt(np.float32(6.0) / np.float32(p.gemm_k), dtype=np.float32)
        w = r.draw(DIST_UNIFORM, nw, float(bound))
        b = r.uniform(-0.1, 0.1, p.out_channels)
        x = self.quantize(p.precision, x).reshape(p.x_shape)
        w = self.quantize(p.precision, w).reshape(p.w_shape)
        b = self.quantize(p.precision, b)
        return x, w, b

    # -- comparison ------------------------------------------------------------------------------
    def tolerance(self, p: Problem, intermediate_rounding: bool = False) -> Tolerance:
        t = Tolerance()
        self.lib.orc_tolerance_for(C.byref(p.desc()), int(intermediate_rounding), C.byref(t))
        return t

    def compare(self, p: Problem, test, ref, scale, intermediate_rounding: bool = False) -> Metrics:
        test, ref, scale = _f32(test).ravel(), _f32(ref).ravel(), _f32(scale).ravel()
        t = self.tolerance(p, intermediate_rounding)
        m = Metrics()
        self.lib.orc_compare(_ptr(test), _ptr(ref), _ptr(scale), test.size, C.byref(t), C.byref(m))
        return m

    # -- other operators -------------------------------------------------------------------------
    def rmsnorm(self, x, gamma, eps: float, precision: int, res_in=None):
        x, gamma = _f32(x), _f32(gamma)
        rows, hidden = x.shape
        r = _f32(res_in) if res_in is not None else None
        y = np.empty((rows, hidden), np.float64)
        ro = np.empty((rows, hidden), np.float32) if r is not None else None
        self.lib.orc_rmsnorm(rows, hidden, eps, precision, _ptr(x), _ptr(gamma), _ptr(r), _ptr(y, C.c_double), _ptr(ro))
        return y, ro

    def maxpool2d(self, x, k=3, s=2, pad=1) -> np.ndarray:
        x = _f32(x)
        b, c, h, w = x.shape
        oh, ow = (h + 2 * pad - k) // s + 1, (w + 2 * pad - k) // s + 1
        y = np.empty((b, c, oh, ow), np.float32)
        self.lib.orc_maxpool2d(b, c, h, w, k, k, s, s, pad, pad, _ptr(x), _ptr(y))
        return y

    def add_relu(self, precision: int, a, b, relu=True) -> np.ndarray:
        a, b = _f32(a), _f32(b)
        y = np.empty_like(a)
        self.lib.orc_add_relu(precision, int(relu), _ptr(a), _ptr(b), _ptr(y), a.size)
        return y


class Reference:
    """The reference library's own oracle (compiled unmodified); exists only where ``make -C oracle ref`` ran."""

    def __init__(self, path: str = REF_SO):
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_validate.argtypes = [C.POINTER(ConvDesc)]
        L.ref_conv2d.argtypes = [C.POINTER(ConvDesc)] + [C.POINTER(C.c_float)] * 5
        L.ref_gpu_conv2d.argtypes = [C.POINTER(ConvDesc)] + [C.c_void_p] * 6
        L.ref_out_hw.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int64)]
        L.ref_rng_u64.argtypes = [C.c_uint64, C.c_int64, C.POINTER(C.c_uint64)]
        L.ref_rng_draw.argtypes = [C.c_uint64, C.c_int, C.c_int64, C.POINTER(C.c_float)]
        L.ref_make_conv_host.argtypes = [C.POINTER(ConvDesc), C.c_uint64, C.c_int] + [C.POINTER(C.c_float)] * 3
        L.ref_quantize.argtypes = [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int64]
        L.ref_compare.argtypes = [C.POINTER(ConvDesc), C.c_int] + [C.POINTER(C.c_float)] * 3 + [C.c_int64, C.POINTER(C.c_double)]
        L.ref_tol.argtypes = [C.POINTER(ConvDesc), C.c_int, C.c_double, C.c_double]
        L.ref_tol.restype = C.c_double
        L.ref_set_num_threads.argtypes = [C.c_int]

    def set_num_threads(self, n: int) -> None:
        """OpenMP threads of the reference's CPU convolution (an OpenMP loop over the outputs)."""
        self.lib.ref_set_num_threads(n)

    def num_threads(self) -> int:
        return self.lib.ref_num_threads()

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def validate(self, p: Problem) -> int:
        return self.lib.ref_validate(C.byref(p.desc()))

    def out_hw_flops(self, p: Problem):
        oh, ow, fl = C.c_int(), C.c_int(), C.c_int64()
        self.lib.ref_out_hw(C.byref(p.desc()), C.byref(oh), C.byref(ow), C.byref(fl))
        return oh.value, ow.value, fl.value

    def conv2d(self, p: Problem, x, w, bias=None):
        x, w = _f32(x), _f32(w)
        b = _f32(bias) if (bias is not None and p.has_bias) else None
        y = np.empty(p.y_shape, np.float32)
        sc = np.empty(p.y_shape, np.float32)
        st = self.lib.ref_conv2d(C.byref(p.desc()), _ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(sc))
        if st != OK:
            raise ValueError(f"reference rejected problem with status {st}")
        return y, sc

    def gpu_conv2d(self, p: Problem, x_dev: int, w_dev: int, bias_dev: int | None, y_dev: int, scale_dev: int, stream: int = 0) -> int:
        """The reference's double-precision GPU convolution on raw device pointers (asynchronous)."""
        return self.lib.ref_gpu_conv2d(C.byref(p.desc()), x_dev, w_dev, bias_dev, y_dev, scale_dev, stream)

    def rng_u64(self, seed: int, n: int) -> np.ndarray:
        out = np.empty(n, np.uint64)
        self.lib.ref_rng_u64(seed, n, _ptr(out, C.c_uint64))
        return out

    def rng_draw(self, seed: int, dist: int, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        self.lib.ref_rng_draw(seed, dist, n, _ptr(out))
        return out

    def make_conv_data(self, p: Problem, seed: int, dist: int = DIST_UNIFORM):
        x = np.empty(p.x_shape, np.float32)
        w = np.empty(p.w_shape, np.float32)
        b = np.empty(p.out_channels, np.float32)
        self.lib.ref_make_conv_host(C.byref(p.desc()), seed, dist, _ptr(x), _ptr(w), _ptr(b))
        return x, w, b

    def quantize(self, precision: int, a) -> np.ndarray:
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.ref_quantize(precision, _ptr(a), _ptr(out), a.size)
        return out

    def compare(self, p: Problem, test, ref, scale, intermediate_rounding=False) -> dict:
        test, ref, scale = _f32(test).ravel(), _f32(ref).ravel(), _f32(scale).ravel()
        out = np.zeros(10, np.float64)
        self.lib.ref_compare(C.byref(p.desc()), int(intermediate_rounding), _ptr(test), _ptr(ref), _ptr(scale), test.size,
                             _ptr(out, C.c_double))
        keys = ("n", "over_tol", "nan_count", "inf_count", "max_abs", "mean_abs", "rms", "max_rel", "frac_over_tol",
                "worst_tol_ratio")
        return dict(zip(keys, out.tolist()))

    def tol(self, p: Problem, ref: float, scale: float, intermediate_rounding=False) -> float:
        return self.lib.ref_tol(C.byref(p.desc()), int(intermediate_rounding), ref, scale)


# The 26 correctness shapes of the reference test-suite (tests/shapes.h:27-56): name -> P(...) arguments.
CORRECTNESS_SHAPES = {
    "tiny_1ch_5x5_k3": (1, 1, 5, 5, 1, 3, 3, 1, 1, 0, 0),
    "scalar_1x1_k1": (1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0),
    "rgb_8x8_k3p1": (1, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1),
    "rgb_32x32_k3p1_b2": (2, 3, 32, 32, 16, 3, 3, 1, 1, 1, 1),
    "odd_unequal_k5s2": (1, 3, 33, 31, 8, 5, 5, 2, 2, 2, 2),
    "pointwise_odd_b2": (2, 16, 15, 17, 24, 1, 1, 1, 1, 0, 0),
    "resnet_14x14_b8_k3": (8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1),
    "resnet_56x56_1x1": (1, 64, 56, 56, 64, 1, 1, 1, 1, 0, 0),
    "resnet_down_28_s2_b2": (2, 64, 28, 28, 128, 3, 3, 2, 2, 1, 1),
    "k7_b16_c32": (16, 32, 20, 20, 48, 7, 7, 1, 1, 3, 3),
    "deep_512ch_7x7": (1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1),
    "b32_c16_16x16": (32, 16, 16, 16, 32, 3, 3, 1, 1, 1, 1),
    "irregular_c7_o9_s2": (2, 7, 11, 13, 9, 3, 3, 2, 2, 0, 0),
    "kernel_eq_map_7x7": (1, 3, 7, 7, 5, 7, 7, 1, 1, 3, 3),
    "c130_o130_9x9": (2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1),
    "o255_pointwise_13": (1, 64, 13, 13, 255, 1, 1, 1, 1, 0, 0),
    "k5_b4_c96_27": (4, 96, 27, 27, 192, 5, 5, 1, 1, 2, 2),
    "stem_7x7_s2_64": (2, 3, 64, 64, 64, 7, 7, 2, 2, 3, 3),
    "down_14_s2_c256": (1, 256, 14, 14, 256, 3, 3, 2, 2, 1, 1),
    "small_b8_4x4": (8, 8, 4, 4, 8, 3, 3, 1, 1, 1, 1),
    "boundary_pad2_3x3": (1, 2, 3, 3, 3, 3, 3, 1, 1, 2, 2),
    "boundary_pad4_k5": (1, 16, 10, 10, 16, 5, 5, 1, 1, 4, 4),
    "aniso_k3x5_s2x1": (2, 8, 17, 23, 12, 3, 5, 2, 1, 1, 2),
    "k1x3": (1, 4, 12, 12, 6, 1, 3, 1, 1, 0, 1),
    "k3x1": (1, 4, 12, 12, 6, 3, 1, 1, 1, 1, 0),
    "wide_1x1_b32": (32, 24, 7, 7, 40, 1, 1, 1, 1, 0, 0),
}

# The benchmark configurations (all seeded, see make_baseline_data).
BASELINE_CONFIGS = {
    "c1": Problem.P(1, 64, 56, 56, 64, 3, 3, 1, 1, 1, 1, FP32, True, True),
    "c2": Problem.P(32, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1, FP16, True, True),
    "c3_fp16": Problem.P(64, 512, 28, 28, 128, 1, 1, 1, 1, 0, 0, FP16, True, True),
    "c3_bf16": Problem.P(64, 512, 28, 28, 128, 1, 1, 1, 1, 0, 0, BF16, True, True),
    "c4a": Problem.P(8, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1, FP16, True, True),
    "c4b": Problem.P(16, 128, 56, 56, 256, 3, 3, 2, 2, 1, 1, FP16, True, True),
}
