"""GPU parity of the chain-oriented extensions of the convolution entry points: channel-contiguous input and output
tensors (read and written in place, no repack) and a residual operand fused into the epilogue.  The reference has
neither (every tensor is NCHW, include/gpu_inference/conv2d.h:66-69; its epilogue is bias + ReLU,
src/kernels/fused_epilogue.cuh:11-16), so the oracle is the reference convolution without activation, plus the
residual, plus the activation, compared under the reference's tolerance policy with the residual magnitude added to
the scale."""
import numpy as np
import pytest

import gpu_util as gu

pytestmark = pytest.mark.gpu

# (shape args, cfg kwargs, input nhwc, output nhwc, residual, prepacked weights)
CASES = [
    ((2, 64, 12, 12, 96, 3, 3, 1, 1, 1, 1), dict(), True, True, True, True),
    ((2, 64, 12, 12, 96, 3, 3, 1, 1, 1, 1), dict(), False, True, False, False),
    ((2, 64, 12, 12, 96, 3, 3, 1, 1, 1, 1), dict(), True, False, True, False),
    ((2, 64, 12, 12, 96, 3, 3, 1, 1, 1, 1), dict(), False, False, True, False),                   # NCHW residual
    ((3, 128, 10, 10, 200, 1, 1, 1, 1, 0, 0), dict(), True, True, True, True),                    # 1x1, channel tail (200)
    ((3, 128, 10, 10, 200, 1, 1, 1, 1, 0, 0), dict(variant=1), True, True, False, True),
    ((2, 256, 14, 14, 256, 3, 3, 2, 2, 1, 1), dict(tile_n=128, split_k=3, reduce=1), True, True, True, True),   # workspace reduction
    ((2, 256, 14, 14, 256, 3, 3, 2, 2, 1, 1), dict(tile_n=128, split_k=2, reduce=2), True, True, True, True),   # cluster reduction
    ((2, 256, 14, 14, 256, 3, 3, 2, 2, 1, 1), dict(tile_n=128, split_k=3, reduce=1), True, False, True, True),
    ((2, 48, 9, 11, 40, 3, 3, 1, 1, 1, 1), dict(), True, True, True, False),                      # C = 48: 16-channel slabs
    ((2, 64, 16, 16, 64, 1, 1, 1, 1, 0, 0), dict(variant=2), False, True, True, True),            # direct NCHW read, NHWC write
    ((4, 64, 28, 28, 64, 3, 3, 1, 1, 1, 1), dict(tile_m=256), True, True, True, True),
    ((1, 32, 7, 7, 30, 5, 5, 1, 1, 2, 2), dict(), True, True, True, False),                       # O = 30: one partial chunk
]


def _tolfn(o, p):
    t = o.tolerance(p)
    k = float(t.k)
    return lambda ref, scale: (t.c_acc * t.u_acc * np.sqrt(k) * scale + t.c_out * t.u_out * np.abs(ref) + t.abs_floor)


def _nhwc(a):
    return np.ascontiguousarray(a.transpose(0, 2, 3, 1))


@pytest.mark.parametrize("case", range(len(CASES)))
@pytest.mark.parametrize("prec_name", ["fp16", "bf16"])
def test_channel_contiguous_and_residual(pkg, orc, oracle, case, prec_name):
    import torch
    args, kw, in_nhwc, out_nhwc, with_res, prepacked = CASES[case]
    prec = orc.FP16 if prec_name == "fp16" else orc.BF16
    relu = case % 3 != 1
    p_lin = orc.Problem.P(*args, precision=prec, bias=True, relu=False)
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=relu)
    x, w, b = oracle.make_conv_data(p, 3000 + case, case % 4)
    lin, scale = oracle.conv2d(p_lin, x, w, b)
    res = oracle.quantize(prec, oracle.rng(4000 + case).uniform(-1, 1, lin.size)).reshape(lin.shape) if with_res else None
    ref = lin.astype(np.float64) + (res.astype(np.float64) if with_res else 0.0)
    if relu:
        ref = np.maximum(ref, 0.0)
    ref = ref.astype(np.float32)
    if with_res:
        scale = (scale.astype(np.float64) + np.abs(res)).astype(np.float32)

    flags = (pkg.FLAG_INPUT_NHWC if in_nhwc else 0) | (pkg.FLAG_OUTPUT_NHWC if out_nhwc else 0) | \
            (pkg.FLAG_RESIDUAL if with_res else 0) | (pkg.FLAG_WEIGHTS_PREPACKED if prepacked else 0)
    plan = pkg.ConvPlan(gu.pkg_problem(pkg, p, flags), pkg.make_cfg(**kw))
    stream = torch.cuda.current_stream().cuda_stream
    tx, px = gu.to_device_storage(oracle, prec, _nhwc(x) if in_nhwc else x)
    tw, pw = gu.to_device_storage(oracle, prec, w)
    if prepacked:
        cp = plan.info.padded_channels
        rs = p.kernel_h * p.kernel_w
        twp = torch.empty(p.out_channels * rs * cp + 8, dtype=torch.int16, device="cuda")
        pkg.prepack_weights(pw, twp.data_ptr(), p.out_channels, p.in_channels, rs, cp, stream)
        pw = twp.data_ptr()
    tb, pb = gu.to_device_storage(oracle, prec, b)
    out = gu.OutBuf(prec, int(np.prod(p.y_shape)))
    ws = gu.Workspace(plan.workspace_bytes)
    wsp = ws.ptr if plan.workspace_bytes else None
    if with_res:
        tr, pr = gu.to_device_storage(oracle, prec, _nhwc(res) if out_nhwc else res)
        plan.launch_fused(px, pw, pb, pr, out.ptr, wsp, plan.workspace_bytes, stream)
    else:
        plan.launch(px, pw, pb, out.ptr, wsp, plan.workspace_bytes, stream)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    ws.check_guard()
    got = out.read(oracle)
    B, O, P, Q = p.y_shape
    got = got.reshape(B, P, Q, O).transpose(0, 3, 1, 2) if out_nhwc else got.reshape(p.y_shape)
    m = oracle.compare(p, np.ascontiguousarray(got), ref, scale)
    assert m.passed(), f"case {case} {kw} {prec_name}: {m.summary()}\n" + gu.describe_mismatch(p, np.ascontiguousarray(got), ref, scale, _tolfn(oracle, p))
    if in_nhwc:
        assert plan.info.launches == (1 if prepacked else 2) + (1 if plan.info.cfg.reduce == 1 else 0)


def test_residual_argument_rules(pkg, orc, oracle):
    """A plan with a fused residual refuses the plain launch, and the other way round; a channel-contiguous input needs
    C % 16 == 0 and is not offered on the FP32 path."""
    import torch
    p = orc.Problem.P(1, 32, 8, 8, 32, 3, 3, 1, 1, 1, 1, precision=orc.FP16, bias=False, relu=True)
    t = torch.zeros(1 << 16, dtype=torch.int16, device="cuda")
    ws = gu.Workspace(1 << 20)
    fused = pkg.ConvPlan(gu.pkg_problem(pkg, p, pkg.FLAG_RESIDUAL))
    plain = pkg.ConvPlan(gu.pkg_problem(pkg, p, 0))
    with pytest.raises(pkg.GieError) as e:
        fused.launch(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), ws.ptr, 1 << 20, 0)
    assert e.value.code == pkg.INVALID_ARGUMENT
    with pytest.raises(pkg.GieError) as e:
        plain.launch_fused(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), t.data_ptr(), ws.ptr, 1 << 20, 0)
    assert e.value.code == pkg.INVALID_ARGUMENT
    odd = orc.Problem.P(1, 24, 8, 8, 32, 3, 3, 1, 1, 1, 1, precision=orc.FP16, bias=False, relu=True)
    assert not pkg.query(gu.pkg_problem(pkg, odd, pkg.FLAG_INPUT_NHWC)).supported
    f32 = orc.Problem.P(1, 32, 8, 8, 32, 3, 3, 1, 1, 1, 1, precision=orc.FP32, bias=False, relu=True)
    assert not pkg.query(gu.pkg_problem(pkg, f32, pkg.FLAG_OUTPUT_NHWC)).supported
    torch.cuda.synchronize()


def test_maxpool_channel_contiguous_matches_planar(pkg, orc, oracle):
    import torch
    for prec, dt in ((orc.FP16, torch.float16), (orc.BF16, torch.bfloat16)):
        B, C, H, W = 3, 40, 13, 17
        x = torch.randn(B, C, H, W, device="cuda").to(dt)
        y0 = torch.empty(B, C, 7, 9, device="cuda", dtype=dt)
        y1 = torch.empty(B, 7, 9, C, device="cuda", dtype=dt)
        xn = x.permute(0, 2, 3, 1).contiguous()
        st = torch.cuda.current_stream().cuda_stream
        pkg.maxpool2d(prec, B, C, H, W, 3, 2, 1, x.data_ptr(), y0.data_ptr(), st)
        pkg.maxpool2d_nhwc(prec, B, C, H, W, 3, 2, 1, xn.data_ptr(), y1.data_ptr(), st)
        torch.cuda.synchronize()
        assert torch.equal(y1.permute(0, 3, 1, 2).contiguous().view(torch.int16), y0.view(torch.int16))
