"""GPU parity tests of RMSNorm and the elementwise operators, through the C ABI, against the CPU oracle.
Mirrors the reference's tests/test_rmsnorm.cpp and the FP32 fused == unfused bitwise check of tests/test_fusion.cpp."""
import numpy as np
import pytest

import gpu_util as gu

pytestmark = pytest.mark.gpu

DT = {"fp32": 0, "fp16": 1, "bf16": 2}
U_OUT = {0: 6e-8, 1: 4.9e-4, 2: 3.9e-3}


def _up(o, dt, a, off=0):
    return gu.to_device_storage(o, dt, a, off)


def _rms_case(pkg, orc, o, rows, hidden, dt, fused, seed, off=0, gamma_fp32=False, alias_res=False):
    import torch
    r = o.rng(seed)
    x = o.quantize(dt, r.draw(orc.DIST_NORMAL, rows * hidden, 3.0)).reshape(rows, hidden)
    res = o.quantize(dt, r.draw(orc.DIST_NORMAL, rows * hidden)).reshape(rows, hidden)
    g = r.uniform(0.5, 1.5, hidden)
    if not gamma_fp32:
        g = o.quantize(dt, g)
    yref, rref = o.rmsnorm(x, g, 1e-6, dt, res if fused else None)
    tx, px = _up(o, dt, x, off)
    tr, pr = _up(o, dt, res)
    tg, pg = _up(o, 0 if gamma_fp32 else dt, g)
    out = gu.OutBuf(dt, rows * hidden)
    rout = gu.OutBuf(dt, rows * hidden)
    rout_ptr = px if alias_res else rout.ptr
    pkg.rmsnorm_forward(rows, hidden, 1e-6, dt, px, pg, out.ptr, pr if fused else None, rout_ptr if fused else None,
                        torch.cuda.current_stream().cuda_stream, gamma_fp32=gamma_fp32)
    torch.cuda.synchronize()
    y = out.read(o).reshape(rows, hidden)
    # tolerance of tests/test_rmsnorm.cpp:44
    tol = (16.0 if dt == 0 else 3.0) * U_OUT[dt] * np.abs(yref) + 1e-30 + (1e-7 if dt == 1 else 0.0)
    bad = np.abs(y - yref) > tol
    assert not bad.any(), f"rows={rows} hidden={hidden} dt={dt} fused={fused}: {bad.sum()} bad, max err {np.abs(y - yref).max()}"
    if fused:
        if alias_res:
            raw = tx.cpu().numpy()[off:off + rows * hidden]
            got = o.from_storage(dt, raw.view(np.uint16) if dt else raw).reshape(rows, hidden)
        else:
            got = rout.read(o).reshape(rows, hidden)
        assert np.array_equal(got, rref), "residual stream must equal round(x + r) exactly"


@pytest.mark.parametrize("dt_name", ["fp32", "fp16", "bf16"])
def test_rmsnorm_irregular_hidden(pkg, orc, oracle, dt_name):
    dt = DT[dt_name]
    for hidden in (1, 7, 33, 64, 127, 1000, 1024, 4096, 5120, 8191):
        for fused in (False, True):
            _rms_case(pkg, orc, oracle, 5, hidden, dt, fused, seed=5 * 1315423911 + hidden)


def test_rmsnorm_long_rows_and_many_rows(pkg, orc, oracle):
    _rms_case(pkg, orc, oracle, 3, 16384, 2, True, 1)
    _rms_case(pkg, orc, oracle, 2, 65536, 1, True, 2)      # 8 vectors x 1024 threads
    _rms_case(pkg, orc, oracle, 2, 65536 + 8, 1, True, 3)  # beyond the register-resident path
    _rms_case(pkg, orc, oracle, 300, 4096, 2, True, 4)
    _rms_case(pkg, orc, oracle, 300, 4096, 2, False, 5)


def test_rmsnorm_misaligned_and_options(pkg, orc, oracle):
    _rms_case(pkg, orc, oracle, 3, 64, 0, False, 6, off=1)     # 4-byte offset: scalar path (tests/test_rmsnorm.cpp:63-73)
    _rms_case(pkg, orc, oracle, 3, 64, 1, True, 7, off=1)
    _rms_case(pkg, orc, oracle, 4, 4096, 2, True, 8, gamma_fp32=True)
    _rms_case(pkg, orc, oracle, 4, 1000, 1, True, 9, gamma_fp32=True)
    _rms_case(pkg, orc, oracle, 4, 4096, 2, True, 10, alias_res=True)  # residual_out may alias x (rmsnorm.h:26)


def test_rmsnorm_full_size_benchmark_shape(pkg, orc, oracle):
    """8192 x 4096 BF16 with residual: gamma = 1 + N(0, 0.02), activations N(0,1), eps 1e-6."""
    import torch
    rows, hidden, dt = 8192, 4096, 2
    r = oracle.rng(0)
    x = oracle.quantize(dt, r.draw(orc.DIST_NORMAL, rows * hidden)).reshape(rows, hidden)
    res = oracle.quantize(dt, r.draw(orc.DIST_NORMAL, rows * hidden)).reshape(rows, hidden)
    g = (1.0 + 0.02 * r.draw(orc.DIST_NORMAL, hidden)).astype(np.float32)
    yref, rref = oracle.rmsnorm(x, g, 1e-6, dt, res)
    tx, px = _up(oracle, dt, x)
    tr, pr = _up(oracle, dt, res)
    tg, pg = _up(oracle, 0, g)
    out, rout = gu.OutBuf(dt, rows * hidden), gu.OutBuf(dt, rows * hidden)
    pkg.rmsnorm_forward(rows, hidden, 1e-6, dt, px, pg, out.ptr, pr, rout.ptr, torch.cuda.current_stream().cuda_stream, gamma_fp32=True)
    torch.cuda.synchronize()
    y = out.read(oracle).reshape(rows, hidden)
    assert np.array_equal(rout.read(oracle).reshape(rows, hidden), rref)
    assert np.all(np.abs(y - yref) <= 3.0 * 3.9e-3 * np.abs(yref) + 1e-30)


def test_rmsnorm_rejects_bad_arguments(pkg):
    """tests/test_rmsnorm.cpp:75-83."""
    import torch
    a = torch.zeros(64, dtype=torch.uint8, device="cuda")
    b = torch.zeros(64, dtype=torch.uint8, device="cuda")
    c = torch.zeros(64, dtype=torch.uint8, device="cuda")
    for args in [(1, 4, a.data_ptr(), b.data_ptr(), a.data_ptr(), None, None),
                 (1, 4, a.data_ptr(), b.data_ptr(), c.data_ptr(), a.data_ptr(), None),
                 (1, 0, a.data_ptr(), b.data_ptr(), c.data_ptr(), None, None)]:
        rows, hidden, x, g, y, ri, ro = args
        with pytest.raises(pkg.GieError) as e:
            pkg.rmsnorm_forward(rows, hidden, 1e-6, 0, x, g, y, ri, ro, 0)
        assert e.value.code == pkg.INVALID_ARGUMENT


def test_fp32_fused_epilogue_equals_unfused_bitwise(pkg, orc, oracle):
    """conv(+bias+ReLU fused) == conv, then bias_act in place, bit for bit in FP32 (tests/test_fusion.cpp:34-58)."""
    import torch
    p_f = orc.Problem.P(2, 16, 12, 12, 24, 3, 3, 1, 1, 1, 1, orc.FP32, True, True)
    p_u = orc.Problem.P(2, 16, 12, 12, 24, 3, 3, 1, 1, 1, 1, orc.FP32, False, False)
    x, w, b = oracle.make_conv_data(p_f, 31, orc.DIST_NORMAL)
    yf, _, of = gu.run_conv(pkg, oracle, p_f, x, w, b)
    yu, _, ou = gu.run_conv(pkg, oracle, p_u, x, w, None)
    tb, pb = gu.to_device_storage(oracle, 0, b)
    pkg.bias_act(0, p_u.batch, p_u.out_channels, p_u.out_h * p_u.out_w, pb, True, ou.ptr, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(of.raw_bits().view(np.uint32), ou.raw_bits().view(np.uint32))


def test_maxpool_and_add_relu(pkg, orc, oracle):
    import torch
    st = torch.cuda.current_stream().cuda_stream
    r = oracle.rng(44)
    for dt in (1, 2):
        # (widths that are multiples of 4 with an even height take the warp-per-plane kernel: one strip, two strips, a
        #  single group; the others the per-row and the generic kernels)
        for (b, c, h, w) in [(2, 5, 13, 17), (1, 64, 112, 112), (3, 4, 8, 8), (2, 3, 10, 140), (1, 2, 6, 4), (1, 3, 224, 224), (2, 3, 10, 6), (1, 2, 14, 260), (1, 2, 58, 8), (2, 1, 224, 12)]:
            x = oracle.quantize(dt, r.draw(orc.DIST_NORMAL, b * c * h * w)).reshape(b, c, h, w)
            ref = oracle.maxpool2d(x, 3, 2, 1)
            tx, px = _up(oracle, dt, x)
            out = gu.OutBuf(dt, ref.size)
            pkg.maxpool2d(dt, b, c, h, w, 3, 2, 1, px, out.ptr, st)
            torch.cuda.synchronize()
            assert np.array_equal(out.read(oracle).reshape(ref.shape), ref)
        for n, off in [(1000, 0), (4099, 0), (4096, 1)]:
            a = oracle.quantize(dt, r.draw(orc.DIST_NORMAL, n))
            bb = oracle.quantize(dt, r.draw(orc.DIST_NORMAL, n))
            for relu in (True, False):
                ref = oracle.add_relu(dt, a, bb, relu)
                ta, pa = _up(oracle, dt, a, off)
                tb2, pb2 = _up(oracle, dt, bb)
                out = gu.OutBuf(dt, n)
                pkg.add_relu(dt, relu, pa, pb2, out.ptr, n, st)
                torch.cuda.synchronize()
                assert np.array_equal(out.read(oracle), ref)
