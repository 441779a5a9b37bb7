"""GPU parity tests of the convolution path, through the C ABI, against the CPU oracle on identical seeded inputs.

Mirrors the reference's tests/test_tensor_core.cpp, test_implicit_gemm.cpp, test_fusion.cpp and the run_suite protocol
(tests/conv_test_common.h:84-127): the 26 correctness shapes x precisions x cycling epilogue mode x four data
distributions, output poisoned with NaN bytes first, reference tolerance policy (no element over tolerance)."""
import numpy as np
import pytest

import gpu_util as gu

pytestmark = pytest.mark.gpu


def _tolfn(o, p):
    t = o.tolerance(p)
    k = float(t.k)
    return lambda ref, scale: (t.c_acc * t.u_acc * np.sqrt(k) * scale + t.c_out * t.u_out * np.abs(ref) + t.abs_floor)


def _check(o, p, got, ref, scale, what):
    m = o.compare(p, got, ref, scale)
    assert m.passed(), f"{what}: {m.summary()}\n" + gu.describe_mismatch(p, got, ref, scale, _tolfn(o, p))
    return m


def _suite_cases(orc):
    cases = []
    cell = 0
    for name, args in orc.CORRECTNESS_SHAPES.items():
        for prec in (orc.FP32, orc.FP16, orc.BF16, orc.TF32):
            mode = cell % 3
            cell += 1
            cases.append((name, args, prec, mode, cell % 4, 0xC0FFEE + cell))
    return cases


@pytest.mark.parametrize("prec_name", ["fp32", "fp16", "bf16", "tf32"])
def test_correctness_shape_suite(pkg, orc, oracle, prec_name):
    prec = {"fp32": orc.FP32, "fp16": orc.FP16, "bf16": orc.BF16, "tf32": orc.TF32}[prec_name]
    ran = 0
    for name, args, pr, mode, dist, seed in _suite_cases(orc):
        if pr != prec:
            continue
        p = orc.Problem.P(*args, precision=pr, bias=mode >= 1, relu=mode == 2)
        x, w, b = oracle.make_conv_data(p, seed, dist)
        ref, scale = oracle.conv2d(p, x, w, b if p.has_bias else None)
        got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b if p.has_bias else None)
        _check(oracle, p, got, ref, scale, f"{name} {prec_name} mode={mode} dist={dist} cfg=({plan.info.cfg.tile_n},"
                                           f"{plan.info.cfg.tile_k},{plan.info.cfg.stages},{plan.info.cfg.split_k})")
        ran += 1
    assert ran == len(orc.CORRECTNESS_SHAPES)


TILE_CASES = [
    # (shape args, cfg kwargs)
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=32, tile_k=16, stages=2)),
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=64, tile_k=32, stages=3)),
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=64, tile_k=64, stages=4, split_k=3)),
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=6, split_k=2)),
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=32, stages=2)),
    ((2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=16, stages=5, split_k=4)),
    ((2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=64, stages=3)),
    ((1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=6, split_k=8)),
    ((1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=64, stages=4, split_k=16)),
    ((2, 64, 28, 28, 128, 3, 3, 2, 2, 1, 1), dict(tile_n=128, tile_k=64, stages=4)),
    ((2, 8, 17, 23, 12, 3, 5, 2, 1, 1, 2), dict(tile_n=32, tile_k=16, stages=3, split_k=5)),
    ((4, 96, 27, 27, 192, 5, 5, 1, 1, 2, 2), dict(tile_n=64, tile_k=32, stages=8, split_k=2)),
    # split-K summed inside the kernel: the slices of a tile form a cluster and exchange partials through distributed shared memory
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=64, tile_k=64, stages=3, split_k=2, reduce=2)),
    ((8, 64, 14, 14, 128, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=32, stages=4, split_k=4, reduce=2)),
    ((2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=3, split_k=2, reduce=2)),
    ((1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=64, stages=4, split_k=8, reduce=2)),
    ((32, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=4, split_k=2, reduce=2)),
    ((3, 200, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(tile_n=256, tile_k=32, stages=3, split_k=2, reduce=2, variant=4)),
    # CTAs that own their SM drain the accumulators with 16 epilogue warps (640 threads): deep rings, partial channel chunks
    ((2, 64, 12, 12, 100, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=6)),                 # one tile per CTA, last chunk 4 channels wide
    ((4, 64, 14, 14, 200, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=64, stages=4)),                 # 256-column tile, channels end inside chunk 6
    ((40, 32, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=32, stages=8)),                # several tiles per persistent CTA
    ((2, 64, 16, 16, 72, 1, 1, 1, 1, 0, 0), dict(tile_n=128, tile_k=64, stages=6, variant=2)),       # direct-NCHW route
    # 256-pixel tiles: two accumulators per CTA share each weight tile
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=64, tile_k=64, stages=3)),
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=256, tile_k=64, stages=3, split_k=2)),
    ((3, 64, 14, 14, 130, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=128, tile_k=32, stages=2)),   # 588 px: last tile owns one half
    ((2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=32, tile_k=16, stages=4, split_k=3)),
    ((2, 64, 28, 28, 128, 3, 3, 2, 2, 1, 1), dict(tile_m=256, tile_n=128, tile_k=64, stages=2)),
    ((1, 16, 5, 5, 8, 1, 1, 1, 1, 0, 0), dict(tile_m=256, tile_n=32, tile_k=16, stages=2)),         # 25 px: one half, mostly empty
]


@pytest.mark.parametrize("case", range(len(TILE_CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_explicit_tile_configurations(pkg, orc, oracle, case, prec_name):
    """Every tile/stage/split-K point of the kernel family must give the same answer (tcmma config sweep analogue,
    tests/test_tensor_core.cpp:72-98)."""
    args, kw = TILE_CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=(case % 2 == 0))
    x, w, b = oracle.make_conv_data(p, 1000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b)
    cfg = pkg.make_cfg(**kw)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b, cfg=cfg)
    for k, v in kw.items():
        assert getattr(plan.info.cfg, k) == v or k == "split_k"
    _check(oracle, p, got, ref, scale, f"case {case} {kw} {prec_name}")


PAIR_CASES = [
    # 256-pixel tiles computed by pairs of CTAs (tcgen05.mma.cta_group::2): each CTA loads its own 128 pixels and half of
    # the weight rows; the leader issues the MMAs for both.  (shape args, cfg kwargs)
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=64, tile_k=64, stages=3)),        # 1568 px: 7 pair tiles, the last one half empty
    ((8, 64, 14, 14, 128, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=128, tile_k=32, stages=4)),
    ((8, 64, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=256, tile_k=64, stages=6)),
    ((2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=256, tile_k=16, stages=5)),       # 162 px: the peer owns 34; channel tails
    ((1, 16, 5, 5, 8, 1, 1, 1, 1, 0, 0), dict(cta_pair=2, tile_n=64, tile_k=16, stages=2)),           # 25 px: the peer owns nothing
    ((2, 64, 28, 28, 128, 3, 3, 2, 2, 1, 1), dict(cta_pair=2, tile_n=128, tile_k=64, stages=2)),      # stride 2
    ((4, 96, 27, 27, 192, 5, 5, 1, 1, 2, 2), dict(cta_pair=2, tile_n=128, tile_k=32, stages=8)),      # 5x5, 2916 px, channel tile tail
    ((1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=256, tile_k=64, stages=6, split_k=4)),   # split-K through the workspace
    ((8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=64, tile_k=32, stages=4, split_k=3)),
    ((96, 64, 28, 28, 64, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=64, tile_k=64, stages=4)),       # 294 pair tiles: several per pair (persistent walk)
    ((40, 32, 14, 14, 512, 3, 3, 1, 1, 1, 1), dict(cta_pair=2, tile_n=256, tile_k=32, stages=6)),     # 62 tiles, double-buffered accumulators
    ((3, 200, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(cta_pair=2, variant=4, tile_n=256, tile_k=32, stages=3)),  # tiled activation loads
    ((2, 512, 28, 28, 128, 1, 1, 1, 1, 0, 0), dict(cta_pair=2, variant=2, tile_n=128, tile_k=64, stages=4)),  # direct NCHW (pixel-major operand)
    ((3, 70, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(cta_pair=2, variant=2, tile_n=256, tile_k=32, stages=3)),
    ((2, 3, 37, 29, 64, 7, 7, 2, 2, 3, 3), dict(cta_pair=2, variant=5, tile_n=64)),                   # row-gather route
]


@pytest.mark.parametrize("case", range(len(PAIR_CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_cta_pair_tiles(pkg, orc, oracle, case, prec_name):
    args, kw = PAIR_CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=(case % 2 == 0))
    x, w, b = oracle.make_conv_data(p, 7000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b, cfg=pkg.make_cfg(**kw), repeats=2)
    assert plan.info.cfg.cta_pair == 2 and plan.info.cfg.tile_m == 256
    assert plan.info.num_blocks % 2 == 0
    _check(oracle, p, got, ref, scale, f"pair case {case} {kw} {prec_name}")


SWAP_CASES = [
    # NCHW output whose planes are 16-byte multiples, on 128- or 256-channel tiles: the accumulator is kept transposed
    # (lane = output channel) and the epilogue writes 32-channel x 32-pixel boxes with TMA stores.  (shape, cfg, y offset in elements)
    ((4, 64, 16, 16, 128, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=4), 0),               # 256 px per image: units never leave an image
    ((3, 64, 12, 14, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=32, stages=3), 0),               # 168 px per image: units cross images; channel tail of 2
    ((3, 64, 12, 14, 200, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=16, stages=4), 0),               # two channel halves, the second one partial
    ((5, 32, 12, 14, 256, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=256, tile_k=32, stages=3), 0),   # 256 x 256 tile, 840 px: last tile owns one half
    ((2, 64, 28, 28, 128, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=128, tile_k=64, stages=2), 0),
    ((40, 32, 8, 8, 128, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=32, stages=2), 0),                # 20 tiles; several per CTA with two CTAs per SM
    ((64, 64, 24, 24, 256, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=64, stages=3), 0),              # 288 tiles on 148 persistent CTAs
    ((3, 64, 12, 14, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=3), 1),               # y off by 2 bytes: no TMA, single-element stores
    ((3, 64, 12, 14, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=3), 2),               # y 4-byte aligned: pairs of pixels
    ((3, 64, 12, 14, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=64, stages=3), 4),               # y 8-byte aligned: runs of four pixels
    ((2, 96, 16, 24, 192, 1, 1, 1, 1, 0, 0), dict(variant=4, tile_n=128, tile_k=32, stages=4), 0),    # tiled activation loads
    ((2, 512, 28, 28, 128, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=128, tile_k=64, stages=4), 0),   # direct NCHW in (pixel-major operand), NCHW out
    ((3, 70, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=256, tile_k=32, stages=3), 0),    # 200 px = 3 boxes of 64 + 8: the map clips the tail
    ((5, 256, 28, 28, 96, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_m=256, tile_n=128, tile_k=64), 0),
    ((2, 64, 56, 56, 128, 3, 3, 2, 2, 1, 1), dict(tile_n=128, tile_k=64, stages=4), 0),               # stride 2 -> 28 x 28
]


@pytest.mark.parametrize("case", range(len(SWAP_CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_transposed_accumulator_nchw_stores(pkg, orc, oracle, case, prec_name, monkeypatch):
    monkeypatch.setenv("GIEB_TRANSPOSED_ACC", "2")  # this form wherever the problem allows it, whatever the cost model prefers
    args, kw, yoff = SWAP_CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    p = orc.Problem.P(*args, precision=prec, bias=(case % 3 != 1), relu=(case % 2 == 0))
    x, w, b = oracle.make_conv_data(p, 8000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b if p.has_bias else None)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b if p.has_bias else None, cfg=pkg.make_cfg(**kw), offsets=(0, 0, yoff), repeats=2)
    assert plan.info.cfg.split_k == 1 and plan.info.cfg.tile_n == kw["tile_n"] and plan.info.threads_per_block == 384
    _check(oracle, p, got, ref, scale, f"transposed-accumulator case {case} {kw} yoff={yoff} {prec_name}")


@pytest.mark.parametrize("case", [0, 1, 2, 3, 9, 11, 12])
@pytest.mark.parametrize("res_off", [0, 1])
def test_transposed_accumulator_fused_residual(pkg, orc, oracle, case, res_off, monkeypatch):
    """y = act(conv + bias + residual) with one rounding on the NCHW TMA-store kernels: every lane reads the residual's 32
    pixels of its own channel (16-byte vectors, or element by element when the residual pointer is off by 2 bytes); units
    that cross into the next image, channel tails and clipped pixel tails included."""
    import torch
    monkeypatch.setenv("GIEB_TRANSPOSED_ACC", "2")
    args, kw, yoff = SWAP_CASES[case]
    prec = orc.FP16 if case % 2 == 0 else orc.BF16
    relu = case % 3 != 0
    p_lin = orc.Problem.P(*args, precision=prec, bias=True, relu=False)
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=relu)
    x, w, b = oracle.make_conv_data(p, 8100 + case, case % 4)
    lin, scale = oracle.conv2d(p_lin, x, w, b)
    res = oracle.quantize(prec, oracle.rng(8200 + case).uniform(-1, 1, lin.size)).reshape(lin.shape)
    ref = lin.astype(np.float64) + res.astype(np.float64)
    ref = (np.maximum(ref, 0.0) if relu else ref).astype(np.float32)
    scale = (scale.astype(np.float64) + np.abs(res)).astype(np.float32)
    plan = pkg.ConvPlan(gu.pkg_problem(pkg, p, pkg.FLAG_RESIDUAL), pkg.make_cfg(**kw))
    assert plan.info.threads_per_block == 384 and plan.info.cfg.split_k == 1
    stream = torch.cuda.current_stream().cuda_stream
    tx, px = gu.to_device_storage(oracle, prec, x)
    tw, pw = gu.to_device_storage(oracle, prec, w)
    tb, pb = gu.to_device_storage(oracle, prec, b)
    tr, pr = gu.to_device_storage(oracle, prec, res, res_off)
    out = gu.OutBuf(prec, int(np.prod(p.y_shape)), yoff)
    ws = gu.Workspace(plan.workspace_bytes)
    for _ in range(2):
        plan.launch_fused(px, pw, pb, pr, out.ptr, ws.ptr if plan.workspace_bytes else None, plan.workspace_bytes, stream)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    ws.check_guard()
    _check(oracle, p, out.read(oracle).reshape(p.y_shape), ref, scale, f"transposed accumulator + residual, case {case} res_off={res_off}")


STRIDED_1X1_CASES = [
    # 1x1 kernels with stride > 1 and no padding over NCHW input: the repack copies only the pixels the convolution reads and
    # the kernel runs a stride-1 1x1 over the copy (tiled loads); variant 1 keeps the im2col route over the whole tensor
    ((2, 64, 9, 11, 32, 1, 1, 2, 3, 0, 0), dict()),                       # asymmetric strides, odd extents
    ((3, 96, 14, 14, 160, 1, 1, 2, 2, 0, 0), dict()),
    ((2, 40, 7, 7, 50, 1, 1, 3, 3, 0, 0), dict(tile_k=16)),                # channel tails, 3 x 3 output
    ((4, 256, 28, 28, 512, 1, 1, 2, 2, 0, 0), dict()),                     # a projection shortcut
    ((4, 256, 28, 28, 512, 1, 1, 2, 2, 0, 0), dict(variant=1)),            # the same through im2col loads
    ((1, 128, 5, 5, 64, 1, 1, 4, 4, 0, 0), dict(tile_k=32, split_k=2, reduce=1)),
]


@pytest.mark.parametrize("case", range(len(STRIDED_1X1_CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_strided_pointwise_reads_a_subsampled_copy(pkg, orc, oracle, case, prec_name):
    args, kw = STRIDED_1X1_CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    p = orc.Problem.P(*args, precision=prec, bias=(case % 2 == 0), relu=(case % 3 != 0))
    x, w, b = oracle.make_conv_data(p, 8400 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b if p.has_bias else None)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b if p.has_bias else None, cfg=pkg.make_cfg(**kw), repeats=2)
    want_variant = kw.get("variant", 4)
    assert plan.info.cfg.variant == want_variant
    if want_variant == 4:  # the copy holds out_h * out_w pixels per image, not in_h * in_w
        al = lambda n: (n + 255) // 256 * 256
        cp, sk = plan.info.padded_channels, plan.info.cfg.split_k
        y_elems = int(np.prod(p.y_shape))
        expect = al(p.batch * p.out_h * p.out_w * cp * 2) + al(p.out_channels * cp * 2) + (al(sk * ((y_elems + 3) // 4 * 4) * 4) if sk > 1 else 0)
        assert plan.workspace_bytes == expect
    _check(oracle, p, got, ref, scale, f"strided 1x1 case {case} {kw} {prec_name}")


FP8_CASES = [
    # FP8 E4M3 x and w (1 byte per element), float bias, FP16 y: kind::f8f6f4 MMAs over the same byte layouts as the 16-bit path
    ((2, 64, 12, 12, 64, 3, 3, 1, 1, 1, 1), dict()),
    ((1, 128, 10, 9, 96, 3, 3, 1, 1, 1, 1), dict(tile_k=128, tile_n=32, stages=2)),
    ((3, 40, 9, 11, 50, 3, 3, 2, 2, 1, 1), dict(tile_k=32)),                           # channel tails on both sides (40 -> 64, 50)
    ((2, 96, 8, 8, 128, 1, 1, 1, 1, 0, 0), dict(variant=4)),                           # tiled loads
    ((2, 256, 7, 7, 64, 1, 1, 1, 1, 0, 0), dict(variant=1, tile_k=64)),
    ((1, 192, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=128, stages=3)),
    ((4, 64, 16, 16, 64, 5, 5, 1, 1, 2, 2), dict(tile_k=64, split_k=4, reduce=1)),       # workspace reduction
    ((2, 512, 6, 6, 128, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=128, split_k=2, reduce=2, stages=4)),  # cluster reduction
    ((8, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict(tile_m=256, tile_n=128, tile_k=128)),  # 256-pixel tiles, several tiles per CTA
    ((1, 3, 20, 20, 16, 7, 7, 2, 2, 3, 3), dict()),                                     # 3 channels padded to 32
    ((6, 128, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=128, cta_pair=2)),  # CTA pairs (cta_group::2 kind::f8f6f4), 1176 px: the last pair's peer is half empty
    ((3, 64, 12, 14, 200, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=64, cta_pair=2, stages=3)),
]


@pytest.mark.parametrize("case", range(len(FP8_CASES)))
def test_fp8_e4m3_extension(pkg, orc, oracle, case):
    """Inputs on the E4M3 grid are exact FP16 values and their products are exact in FP32, so the FP16 oracle (double
    accumulation, FP16 output tolerance) is the oracle of the FP8 path on the same values."""
    import torch
    from oracle import oracle as orc_mod
    args, kw = FP8_CASES[case]
    relu, bias = case % 2 == 0, case % 3 != 1
    p = orc.Problem.P(*args, precision=orc.FP16, bias=bias, relu=relu)
    x, w, b = oracle.make_conv_data(p, 8300 + case, case % 4)
    x, w = orc_mod.e4m3_quantize(x), orc_mod.e4m3_quantize(w)
    ref, scale = oracle.conv2d(p, x, w, b if bias else None)
    prob = pkg.ConvProblem(p.batch, p.in_channels, p.in_h, p.in_w, p.out_channels, p.kernel_h, p.kernel_w, p.stride_h, p.stride_w, p.pad_h,
                           p.pad_w, 1, 1, 1, pkg.FP8_E4M3, bias, relu, 0)
    plan = pkg.ConvPlan(prob, pkg.make_cfg(**kw))
    for k, v in kw.items():
        if k in ("tile_k", "tile_n", "split_k"):
            assert getattr(plan.info.cfg, k) == v
    stream = torch.cuda.current_stream().cuda_stream
    tx = torch.from_numpy(orc_mod.e4m3_bits(x).ravel()).cuda()
    tw = torch.from_numpy(orc_mod.e4m3_bits(w).ravel()).cuda()
    tb = torch.from_numpy(np.ascontiguousarray(b, dtype=np.float32)).cuda()
    out = gu.OutBuf(orc.FP16, int(np.prod(p.y_shape)))
    ws = gu.Workspace(plan.workspace_bytes)
    for _ in range(2):
        plan.launch(tx.data_ptr(), tw.data_ptr(), tb.data_ptr() if bias else None, out.ptr, ws.ptr if plan.workspace_bytes else None,
                    plan.workspace_bytes, stream)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    ws.check_guard()
    _check(oracle, p, out.read(oracle).reshape(p.y_shape), ref, scale, f"FP8 case {case} {kw}")


def test_fp8_refuses_what_it_does_not_offer(pkg):
    for flags in (pkg.FLAG_INPUT_NHWC, pkg.FLAG_OUTPUT_NHWC, pkg.FLAG_RESIDUAL, pkg.FLAG_WEIGHTS_PREPACKED):
        with pytest.raises(pkg.GieError) as e:
            pkg.ConvPlan(pkg.ConvProblem(1, 64, 8, 8, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1, pkg.FP8_E4M3, True, True, flags))
        assert e.value.code == pkg.UNSUPPORTED
    for kw in (dict(variant=2), dict(tile_k=16), dict(split_k=2, reduce=2, cta_pair=2)):
        with pytest.raises(pkg.GieError) as e:
            pkg.ConvPlan(pkg.ConvProblem(1, 64, 8, 8, 64, 1, 1, 1, 1, 0, 0, 1, 1, 1, pkg.FP8_E4M3, True, True, 0), pkg.make_cfg(**kw))
        assert e.value.code == pkg.UNSUPPORTED


DIRECT_CASES = [
    # 1x1 / stride 1 / pad 0 with H*W % 8 == 0: activations are read straight from NCHW (pixel-major operand)
    ((2, 64, 8, 8, 64, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=64, tile_k=64, stages=2), 0),
    ((1, 64, 56, 56, 64, 1, 1, 1, 1, 0, 0), dict(variant=2), 0),
    ((3, 70, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=256, tile_k=32, stages=3), 0),     # C tail, 200 px = 3 boxes + 8
    ((2, 512, 28, 28, 128, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_m=256, tile_n=128, tile_k=64, stages=2), 0),
    ((2, 96, 4, 6, 40, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_k=16, tile_n=64, split_k=3, stages=2), 0),  # 24 px per image
    ((5, 256, 28, 28, 96, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_m=256, tile_n=128, split_k=2, tile_k=64), 0),
    ((2, 64, 16, 16, 48, 1, 1, 1, 1, 0, 0), dict(variant=2), 1),                                         # x off by 2 bytes: repack route
    ((2, 64, 16, 16, 48, 1, 1, 1, 1, 0, 0), dict(variant=4), 0),
    ((2, 64, 16, 16, 48, 1, 1, 1, 1, 0, 0), dict(variant=1), 0),
    ((2, 512, 8, 8, 256, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=256, tile_k=64, stages=4), 0),       # one image per 64-pixel box
    ((2, 512, 8, 8, 256, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=128, tile_k=64, stages=4), 0),
    ((4, 512, 8, 8, 256, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=256, tile_k=64, stages=3), 0),
    # cluster reduction on the direct route: rows are numbered in 64-pixel boxes, 16 or 24 of them real pixels
    ((2, 1024, 4, 4, 256, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=256, tile_k=64, stages=4, split_k=4, reduce=2), 0),
    ((3, 256, 4, 6, 200, 1, 1, 1, 1, 0, 0), dict(variant=2, tile_n=128, tile_k=64, stages=2, split_k=2, reduce=2), 0),
]


TF32_CASES = [
    # FP32 storage on the tensor cores (kind::tf32): inputs rounded to TF32 (ties away) by the repack, FP32 accumulate and output
    ((2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict()),
    ((2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=128, tile_k=32, stages=3, split_k=2, reduce=1)),
    ((2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), dict(tile_n=64, tile_k=16, stages=4, split_k=2, reduce=2)),
    ((2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1), dict(tile_n=256, tile_k=8, stages=3)),
    ((3, 70, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(variant=4, tile_n=128, tile_k=32)),
    ((3, 70, 10, 20, 255, 1, 1, 1, 1, 0, 0), dict(variant=1)),
    ((1, 3, 33, 31, 20, 7, 7, 2, 2, 3, 3), dict()),
    ((2, 64, 28, 28, 128, 3, 3, 2, 2, 1, 1), dict(tile_m=256, tile_n=128, tile_k=32, stages=2)),
    ((8, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1), dict()),
]


@pytest.mark.parametrize("case", range(len(TF32_CASES)))
def test_tf32_tensor_path(pkg, orc, oracle, case):
    args, kw = TF32_CASES[case]
    p = orc.Problem.P(*args, precision=orc.TF32, bias=(case % 3 != 0), relu=(case % 2 == 0))
    x, w, b = oracle.make_conv_data(p, 6000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b if p.has_bias else None)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b if p.has_bias else None, cfg=pkg.make_cfg(**kw))
    assert plan.info.variant in (1, 4)
    _check(oracle, p, got, ref, scale, f"tf32 case {case} {kw}")


GATHER_CASES = [
    # few input channels: the S taps of a filter row become channels (variant 5)
    ((2, 3, 32, 32, 64, 7, 7, 2, 2, 3, 3), dict()),                      # the stem geometry: picked automatically
    ((2, 3, 37, 29, 64, 7, 7, 2, 2, 3, 3), dict(variant=5)),             # odd extents: partial last tile, padded columns
    ((3, 1, 20, 24, 40, 3, 3, 1, 1, 1, 1), dict(variant=5)),             # one channel, 3 taps -> 16 gathered channels
    ((2, 4, 18, 18, 48, 5, 5, 1, 1, 2, 2), dict(variant=5, tile_n=64)),  # 5 x 4 = 20 -> 32
    ((2, 8, 16, 20, 96, 3, 5, 2, 1, 1, 2), dict(variant=5, tile_k=16, split_k=2)),   # 5 x 8 = 40 -> 48: three 16-channel slabs per row
    ((1, 3, 64, 64, 32, 7, 7, 2, 2, 3, 3), dict(variant=5, tile_m=256, tile_n=32)),
    ((2, 3, 30, 40, 64, 7, 7, 2, 2, 3, 3), dict(variant=5)),             # whole-row gather, rows not a multiple of four
    ((3, 4, 9, 16, 32, 5, 5, 1, 1, 2, 2), dict(variant=5)),              # whole-row gather, stride 1, 20 -> 32 channels
    # stride_w = 2 with at most 4 channels: column pairs stored once, overlapping windows (the layout the stem takes)
    ((2, 4, 20, 22, 16, 3, 3, 2, 2, 1, 1), dict(variant=5)),             # two positions per window (16 values)
    ((2, 1, 18, 26, 32, 7, 7, 2, 2, 3, 3), dict(variant=5)),             # one channel
    ((1, 3, 33, 48, 64, 7, 7, 1, 2, 3, 2), dict(variant=5)),             # pad_w = 2: the window starts on a pair, stride_h = 1
    ((3, 2, 12, 8, 24, 7, 7, 2, 2, 3, 3), dict(variant=5, tile_k=16)),   # four output columns, windows mostly padding
]


@pytest.mark.parametrize("case", range(len(GATHER_CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_row_gather_route(pkg, orc, oracle, case, prec_name):
    args, kw = GATHER_CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=(case % 2 == 0))
    x, w, b = oracle.make_conv_data(p, 5000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b, cfg=pkg.make_cfg(**kw))
    assert plan.info.variant == 5
    _check(oracle, p, got, ref, scale, f"gather case {case} {kw} {prec_name}")
    if p.stride_w == 2 and p.in_channels <= 4:  # x off by one element: the gather reads columns one by one
        got, _, _ = gu.run_conv(pkg, oracle, p, x, w, b, cfg=pkg.make_cfg(**kw), offsets=(1, 0, 0))
        _check(oracle, p, got, ref, scale, f"gather case {case} {kw} {prec_name}, x misaligned")


@pytest.mark.parametrize("case", range(len(DIRECT_CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_pointwise_routes(pkg, orc, oracle, case, prec_name):
    args, kw, xoff = DIRECT_CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=(case % 2 == 1))
    x, w, b = oracle.make_conv_data(p, 2000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, w, b)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b, cfg=pkg.make_cfg(**kw), offsets=(xoff, 0, 0))
    assert plan.info.variant == kw["variant"]
    _check(oracle, p, got, ref, scale, f"pointwise case {case} {kw} {prec_name}")


def test_baseline_configurations_full_size(pkg, orc, oracle):
    """The benchmark shapes at full size with the benchmark distributions, checked with BOTH tolerances: the
    reference's scale-aware policy and the benchmark's |err| <= a + b*|ref| bounds."""
    bounds = {orc.FP16: (5e-3, 1e-2), orc.BF16: (2e-2, 3e-2)}
    for name, p in orc.BASELINE_CONFIGS.items():
        x, w, b = oracle.make_baseline_data(p, 0)
        ref, scale = oracle.conv2d(p, x, w, b)
        got, plan, _ = gu.run_conv(pkg, oracle, p, x, w, b)
        _check(oracle, p, got, ref, scale, name)
        err = np.abs(got.astype(np.float64) - ref)
        if p.precision == orc.FP32:
            # FP32 bound of the benchmark: relative error <= 1e-5.  An element-wise ratio is meaningless where the
            # sum cancels (|ref| far below the magnitude of its terms), so the denominator is floored at rms(ref);
            # the norm-wise relative error is checked as well.
            rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
            rel = err / np.maximum(np.abs(ref), rms)
            assert rel.max() <= 1e-5, f"{name}: fp32 relative error {rel.max():.3e}"
            assert np.sqrt(np.sum(err ** 2)) / np.sqrt(np.sum(ref.astype(np.float64) ** 2)) <= 1e-5
        else:
            a, r = bounds[p.precision]
            assert np.all(err <= a + r * np.abs(ref)), f"{name}: max err {err.max():.3e}"


def test_fp32_bias_option_matches_storage_bias(pkg, orc, oracle):
    """GIEB_FLAG_BIAS_FP32: an FP32 bias vector holding the storage-rounded values gives bit-identical output."""
    p = orc.Problem.P(4, 32, 12, 12, 48, 3, 3, 1, 1, 1, 1, orc.FP16, True, True)
    x, w, b = oracle.make_conv_data(p, 77)
    y0, _, o0 = gu.run_conv(pkg, oracle, p, x, w, b)
    y1, _, o1 = gu.run_conv(pkg, oracle, p, x, w, b, flags=pkg.FLAG_BIAS_FP32)
    assert np.array_equal(o0.raw_bits(), o1.raw_bits())


def test_prepacked_weights_option(pkg, orc, oracle):
    """GIEB_FLAG_WEIGHTS_PREPACKED: prepacking once with gieb_prepack_weights gives bit-identical output."""
    import torch
    p = orc.Problem.P(4, 24, 12, 12, 40, 3, 3, 1, 1, 1, 1, orc.BF16, True, False)
    x, w, b = oracle.make_conv_data(p, 78)
    y0, plan0, o0 = gu.run_conv(pkg, oracle, p, x, w, b)
    cp = gu.pkg_problem(pkg, p, pkg.FLAG_WEIGHTS_PREPACKED)
    plan = pkg.ConvPlan(cp)
    cpad = plan.info.padded_channels
    assert plan.workspace_bytes < plan0.workspace_bytes
    tw, pw = gu.to_device_storage(oracle, p.precision, w)
    wk = torch.empty(p.out_channels * 9 * cpad, dtype=torch.int16, device="cuda")
    pkg.prepack_weights(pw, wk.data_ptr(), p.out_channels, p.in_channels, 9, cpad, torch.cuda.current_stream().cuda_stream)
    tx, px = gu.to_device_storage(oracle, p.precision, x)
    tb, pb = gu.to_device_storage(oracle, p.precision, b)
    out = gu.OutBuf(p.precision, int(np.prod(p.y_shape)))
    ws = gu.Workspace(plan.workspace_bytes)
    plan.launch(px, wk.data_ptr(), pb, out.ptr, ws.ptr, plan.workspace_bytes, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(out.raw_bits(), o0.raw_bits())


def test_misaligned_tensor_pointers(pkg, orc, oracle):
    """X, W and Y offset by one element (2 bytes) must work (tests/test_tensor_core.cpp:38-57,
    tests/test_runtime_concurrency.cu:190-216)."""
    for prec in (orc.FP16, orc.BF16, orc.FP32):
        p = orc.Problem.P(2, 16, 9, 11, 24, 3, 3, 1, 1, 1, 1, prec, True, True)
        x, w, b = oracle.make_conv_data(p, 5)
        ref, scale = oracle.conv2d(p, x, w, b)
        got, _, _ = gu.run_conv(pkg, oracle, p, x, w, b, offsets=(1, 1, 1))
        _check(oracle, p, got, ref, scale, f"misaligned prec={prec}")


@pytest.mark.parametrize("woff", [0, 1, 8])
def test_pointwise_weights_in_place_and_fallback(pkg, orc, oracle, woff):
    """1x1 filters over unpadded channels are read where the caller keeps them when the pointer is 16-byte aligned
    (one launch); a pointer that is not takes the prepack launch.  Both must give the oracle's values, on the
    direct-NCHW route and with a channel-contiguous input."""
    for flags_name in ("nchw", "nhwc_in"):
        p = orc.Problem.P(3, 64, 8, 16, 96, 1, 1, 1, 1, 0, 0, orc.FP16, True, True)
        x, w, b = oracle.make_conv_data(p, 77 + woff)
        ref, scale = oracle.conv2d(p, x, w, b)
        flags = 0
        xin = x
        if flags_name == "nhwc_in":
            flags = pkg.FLAG_INPUT_NHWC
            xin = np.ascontiguousarray(x.reshape(3, 64, 8 * 16).transpose(0, 2, 1))
        got, plan, _ = gu.run_conv(pkg, oracle, p, xin, w, b, flags=flags, offsets=(0, woff, 0))
        assert plan.info.launches == 1   # the plan counts on aligned weights
        _check(oracle, p, got, ref, scale, f"1x1 weights offset {woff} elements, {flags_name}")


def test_relu_gives_exact_zeros_and_runs_are_deterministic(pkg, orc, oracle):
    """ReLU outputs are exactly zero where the reference is zero-clamped well below zero (tests/test_fusion.cpp:15-30);
    two launches give identical bits."""
    p = orc.Problem.P(2, 32, 10, 10, 32, 3, 3, 1, 1, 1, 1, orc.FP16, True, True)
    x, w, b = oracle.make_conv_data(p, 9, orc.DIST_NORMAL)
    p_lin = orc.Problem.P(2, 32, 10, 10, 32, 3, 3, 1, 1, 1, 1, orc.FP16, True, False)
    lin, _ = oracle.conv2d(p_lin, x, w, b)
    y0, plan, o0 = gu.run_conv(pkg, oracle, p, x, w, b)
    y1, _, o1 = gu.run_conv(pkg, oracle, p, x, w, b, plan=plan)
    assert np.array_equal(o0.raw_bits(), o1.raw_bits())
    assert np.all(y0[lin < -1e-2] == 0.0)
    assert np.all(y0 >= 0.0)


def test_launch_argument_checks(pkg, orc, oracle):
    """Status codes of the launch-time checks (tests/test_validation.cpp:23-95 subset that lives below the C ABI)."""
    import torch
    p = orc.Problem.P(2, 8, 10, 10, 8, 3, 3, 1, 1, 1, 1, orc.FP16, True, False)
    plan = pkg.ConvPlan(gu.pkg_problem(pkg, p))
    assert plan.workspace_bytes > 0
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    base = (buf.data_ptr() + 255) // 256 * 256
    st = torch.cuda.current_stream().cuda_stream
    with pytest.raises(pkg.GieError) as e:
        plan.launch(None, base, base, base, base, plan.workspace_bytes, st)
    assert e.value.code == pkg.INVALID_ARGUMENT
    with pytest.raises(pkg.GieError) as e:
        plan.launch(base, base, None, base, base, plan.workspace_bytes, st)
    assert e.value.code == pkg.INVALID_ARGUMENT
    with pytest.raises(pkg.GieError) as e:
        plan.launch(base, base, base, base, None, 0, st)
    assert e.value.code == pkg.WORKSPACE_TOO_SMALL
    with pytest.raises(pkg.GieError) as e:
        plan.launch(base, base, base, base, base, plan.workspace_bytes - 1, st)
    assert e.value.code == pkg.WORKSPACE_TOO_SMALL
    with pytest.raises(pkg.GieError) as e:
        plan.launch(base, base, base, base, base + 16, plan.workspace_bytes, st)
    assert e.value.code == pkg.INVALID_ARGUMENT
    torch.cuda.synchronize()


def test_cuda_graph_capture_matches_eager(pkg, orc, oracle):
    """A captured launch replays bit-identically, also after the inputs change (tests/test_cuda_graph.cu:42-70)."""
    import torch
    p = orc.Problem.P(4, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, orc.FP16, True, True)
    plan = pkg.ConvPlan(gu.pkg_problem(pkg, p))
    x, w, b = oracle.make_conv_data(p, 21)
    tx, px = gu.to_device_storage(oracle, p.precision, x)
    tw, pw = gu.to_device_storage(oracle, p.precision, w)
    tb, pb = gu.to_device_storage(oracle, p.precision, b)
    out = gu.OutBuf(p.precision, int(np.prod(p.y_shape)))
    ws = gu.Workspace(plan.workspace_bytes)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        plan.launch(px, pw, pb, out.ptr, ws.ptr, plan.workspace_bytes, s.cuda_stream)  # warm-up outside capture
        s.synchronize()
        eager = out.raw_bits()
        out.t.view(torch.uint8).fill_(0xFF)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            plan.launch(px, pw, pb, out.ptr, ws.ptr, plan.workspace_bytes, torch.cuda.current_stream().cuda_stream)
        g.replay()
        torch.cuda.synchronize()
        assert np.array_equal(out.raw_bits(), eager)
        # new inputs in the same buffers
        x2, w2, b2 = oracle.make_conv_data(p, 22)
        raw = oracle.to_storage(p.precision, x2.ravel()).view(np.int16)
        tx[:raw.size] = torch.from_numpy(raw).cuda()
        raw = oracle.to_storage(p.precision, w2.ravel()).view(np.int16)
        tw[:raw.size] = torch.from_numpy(raw).cuda()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
    ref, scale = oracle.conv2d(p, x2, w2, b)
    got = oracle.from_bits16(p.precision, out.raw_bits().view(np.uint16)).reshape(p.y_shape)
    _check(oracle, p, got, ref, scale, "graph replay with new inputs")


def test_repack_is_bit_exact(pkg, orc, oracle):
    """NCHW -> channel-padded NHWC and OIHW -> [O][RS][Cp] are pure permutations of 16-bit patterns (NaNs included)."""
    import torch
    rng = np.random.default_rng(3)
    st = torch.cuda.current_stream().cuda_stream
    for (bt, c, hw, cp, off) in [(2, 64, 196, 64, 0), (3, 5, 49, 16, 1), (1, 130, 81, 160, 0), (2, 3, 4096, 16, 0), (4, 256, 784, 256, 0),
                                 (256, 256, 9, 256, 0), (64, 3, 49, 16, 1), (5, 17, 33, 32, 3), (1, 8, 1, 8, 0), (7, 70, 25, 128, 0),
                                 (2, 64, 200, 64, 4)]:
        src = rng.integers(0, 65536, size=bt * c * hw, dtype=np.uint16)
        t = torch.empty(src.size + off + 8, dtype=torch.int16, device="cuda")
        t[off:off + src.size] = torch.from_numpy(src.view(np.int16)).cuda()
        dst = torch.full((bt * hw * cp + 64,), -1, dtype=torch.int16, device="cuda")
        pkg.repack_nchw_to_nhwc(t.data_ptr() + 2 * off, dst.data_ptr(), bt, c, hw, cp, st)
        torch.cuda.synchronize()
        got = dst.cpu().numpy().view(np.uint16)
        exp = np.zeros((bt, hw, cp), np.uint16)
        exp[:, :, :c] = src.reshape(bt, c, hw).transpose(0, 2, 1)
        assert np.array_equal(got[:exp.size].reshape(exp.shape), exp), (bt, c, hw, cp, off)
        assert np.all(got[exp.size:] == 0xFFFF)


@pytest.mark.parametrize("kw", [dict(tile_n=128, tile_k=64, stages=4), dict(tile_n=64, tile_k=32, stages=3, split_k=2, reduce=2),
                                dict(cta_pair=2, tile_n=128, tile_k=64, stages=4)])
@pytest.mark.parametrize("roles,expect", [(1, 2), (2, 1 | 4)])
def test_bounded_waits_run_out_and_report(pkg, orc, oracle, kw, roles, expect):
    """A device-side wait that is never satisfied gives up after its limit, sets its bit in the plan's status word, the
    kernel ends by itself with its tensor memory freed, and the next launch of the same plan is correct again.  The stall
    is injected on the host (a role that issues nothing); nothing faults.  roles 1: the producers load nothing, so the MMA
    issuer gives up (bit 1 = value 2); roles 2: the issuer does nothing, so the producers (value 1) and the epilogue
    (value 4) give up."""
    import time
    import torch
    p = orc.Problem.P(4, 64, 14, 14, 128, 3, 3, 1, 1, 1, 1, precision=orc.FP16, bias=True, relu=True)
    x, w, b = oracle.make_conv_data(p, 31, 1)
    ref, scale = oracle.conv2d(p, x, w, b)
    plan = pkg.ConvPlan(gu.pkg_problem(pkg, p), pkg.make_cfg(**kw))
    got, _, _ = gu.run_conv(pkg, oracle, p, x, w, b, plan=plan)
    _check(oracle, p, got, ref, scale, "before the injected stall")
    plan.inject_stall(roles, 2_000_000)  # about a millisecond per wait
    tx, px = gu.to_device_storage(oracle, p.precision, x)
    tw, pw = gu.to_device_storage(oracle, p.precision, w)
    tb, pb = gu.to_device_storage(oracle, p.precision, b)
    out = gu.OutBuf(p.precision, int(np.prod(p.y_shape)))
    ws = gu.Workspace(plan.workspace_bytes)
    t0 = time.time()
    plan.launch(px, pw, pb, out.ptr, ws.ptr, plan.workspace_bytes, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()  # the kernel returns by itself
    assert time.time() - t0 < 5.0
    status = plan.device_status()
    assert status & expect == expect and status != 0, f"status word {status}, expected bits {expect}"
    out.read(oracle)  # guard bands intact
    ws.check_guard()
    plan.close()
    # the device and its tensor memory are fine: a fresh plan of the same configuration computes the right answer
    plan2 = pkg.ConvPlan(gu.pkg_problem(pkg, p), pkg.make_cfg(**kw))
    got2, _, _ = gu.run_conv(pkg, oracle, p, x, w, b, plan=plan2)
    _check(oracle, p, got2, ref, scale, "after the injected stall")
