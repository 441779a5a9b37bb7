"""Randomised GPU parity: seeded random geometries, precisions, layouts and epilogues through the C ABI with whatever
configuration the plan picks, each compared with the CPU oracle under the reference's tolerance policy.  Complements
the hand-picked cases of the other files (the reference's own suite is a fixed shape list, tests/shapes.h:27-56)."""
import numpy as np
import pytest

import gpu_util as gu

pytestmark = pytest.mark.gpu

N_CASES = 72


def _draw(rng, orc):
    prec = [orc.FP16, orc.BF16, orc.TF32, orc.FP32][int(rng.integers(0, 4))]
    k = int(rng.choice([1, 1, 3, 3, 5, 7]))
    stride = int(rng.choice([1, 1, 2]))
    pad = int(rng.integers(0, min(k, 3)))
    c = int(rng.choice([3, 4, 8, 16, 24, 32, 48, 64, 96, 130, 160]))
    o = int(rng.choice([8, 16, 30, 40, 64, 100, 128, 200, 256]))
    h = int(rng.integers(max(k - 2 * pad, 4), 22))
    w = int(rng.integers(max(k - 2 * pad, 4), 22))
    b = int(rng.integers(1, 5))
    args = (b, c, h, w, o, k, k, stride, stride, pad, pad)
    sixteen = prec in (orc.FP16, orc.BF16)
    in_nhwc = sixteen and c % 16 == 0 and rng.random() < 0.4
    out_nhwc = sixteen and rng.random() < 0.4
    residual = sixteen and rng.random() < 0.4
    prepacked = sixteen and rng.random() < 0.3
    return prec, args, bool(rng.random() < 0.7), bool(rng.random() < 0.5), in_nhwc, out_nhwc, residual, prepacked


def _nhwc(a):
    return np.ascontiguousarray(a.transpose(0, 2, 3, 1))


@pytest.mark.parametrize("case", range(N_CASES))
def test_random_problem(pkg, orc, oracle, case):
    import torch
    rng = np.random.default_rng(90000 + case)
    prec, args, bias, relu, in_nhwc, out_nhwc, with_res, prepacked = _draw(rng, orc)
    p_lin = orc.Problem.P(*args, precision=prec, bias=bias, relu=False)
    p = orc.Problem.P(*args, precision=prec, bias=bias, relu=relu)
    x, w, b = oracle.make_conv_data(p, 91000 + case, case % 4)
    lin, scale = oracle.conv2d(p_lin, x, w, b if bias else None)
    res = oracle.quantize(prec, oracle.rng(92000 + case).uniform(-1, 1, lin.size)).reshape(lin.shape) if with_res else None
    ref = lin.astype(np.float64) + (res.astype(np.float64) if with_res else 0.0)
    if relu:
        ref = np.maximum(ref, 0.0)
    ref = ref.astype(np.float32)
    if with_res:
        scale = (scale.astype(np.float64) + np.abs(res)).astype(np.float32)
    flags = (pkg.FLAG_INPUT_NHWC if in_nhwc else 0) | (pkg.FLAG_OUTPUT_NHWC if out_nhwc else 0) | \
            (pkg.FLAG_RESIDUAL if with_res else 0) | (pkg.FLAG_WEIGHTS_PREPACKED if prepacked else 0)
    plan = pkg.ConvPlan(gu.pkg_problem(pkg, p, flags))
    stream = torch.cuda.current_stream().cuda_stream
    tx, px = gu.to_device_storage(oracle, prec, _nhwc(x) if in_nhwc else x)
    tw, pw = gu.to_device_storage(oracle, prec, w)
    if prepacked:
        twp = torch.empty(plan.prepacked_weight_bytes // 2 + 8, dtype=torch.int16, device="cuda")
        plan.prepack_weights(pw, twp.data_ptr(), stream)
        pw = twp.data_ptr()
    tb, pb = gu.to_device_storage(oracle, prec, b)
    out = gu.OutBuf(prec, int(np.prod(p.y_shape)))
    ws = gu.Workspace(plan.workspace_bytes)
    wsp = ws.ptr if plan.workspace_bytes else None
    if with_res:
        tr, pr = gu.to_device_storage(oracle, prec, _nhwc(res) if out_nhwc else res)
        plan.launch_fused(px, pw, pb if bias else None, pr, out.ptr, wsp, plan.workspace_bytes, stream)
    else:
        plan.launch(px, pw, pb if bias else None, out.ptr, wsp, plan.workspace_bytes, stream)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    ws.check_guard()
    got = out.read(oracle)
    B, O, P, Q = p.y_shape
    got = np.ascontiguousarray(got.reshape(B, P, Q, O).transpose(0, 3, 1, 2)) if out_nhwc else got.reshape(p.y_shape)
    m = oracle.compare(p, got, ref, scale)
    c = plan.info.cfg
    assert m.passed(), (f"case {case}: prec={prec} args={args} bias={bias} relu={relu} flags={flags} "
                        f"cfg=({c.tile_m},{c.tile_n},{c.tile_k},s{c.stages},k{c.split_k},v{c.variant},r{c.reduce}): {m.summary()}")


@pytest.mark.parametrize("case", range(N_CASES))
def test_random_configuration(pkg, orc, oracle, case):
    """The same idea over the configuration space: random tile shape, ring depth, split-K factor, reduction mode and
    CTA pairing on a random tensor-path problem.  Points the library refuses (with kUnsupported) are redrawn until one is
    accepted, so every case runs; every accepted point must be right."""
    rng = np.random.default_rng(95000 + case)
    plan = None
    for _attempt in range(200):
        prec = [orc.FP16, orc.BF16, orc.TF32][int(rng.integers(0, 3))]
        k = int(rng.choice([1, 3, 3, 5]))
        stride = int(rng.choice([1, 1, 2]))
        pad = int(rng.integers(0, min(k, 3)))
        c = int(rng.choice([16, 32, 64, 96, 128, 192]))
        o = int(rng.choice([32, 64, 96, 128, 256]))
        h, w = int(rng.integers(6, 20)), int(rng.integers(6, 20))
        args = (int(rng.integers(1, 6)), c, h, w, o, k, k, stride, stride, pad, pad)
        tile_k = int(rng.choice([16, 32, 64])) if prec != orc.TF32 else int(rng.choice([8, 16, 32]))
        kw = dict(tile_m=int(rng.choice([128, 256])), tile_n=int(rng.choice([32, 64, 128, 256])), tile_k=tile_k,
                  stages=int(rng.integers(2, 7)), split_k=int(rng.choice([1, 1, 2, 3, 4, 8])), reduce=int(rng.integers(0, 3)),
                  cta_pair=int(rng.choice([0, 1, 2])))
        p = orc.Problem.P(*args, precision=prec, bias=bool(rng.random() < 0.7), relu=bool(rng.random() < 0.5))
        try:
            plan = pkg.ConvPlan(gu.pkg_problem(pkg, p, 0), pkg.make_cfg(**kw))
            break
        except pkg.GieError as e:
            assert e.code == pkg.UNSUPPORTED, str(e)
    assert plan is not None, "no accepted configuration in 200 draws"
    x, wt, b = oracle.make_conv_data(p, 96000 + case, case % 4)
    ref, scale = oracle.conv2d(p, x, wt, b if p.has_bias else None)
    got, plan, _ = gu.run_conv(pkg, oracle, p, x, wt, b if p.has_bias else None, plan=plan)
    m = oracle.compare(p, got, ref, scale)
    assert m.passed(), f"case {case}: prec={prec} args={args} {kw}: {m.summary()}"
