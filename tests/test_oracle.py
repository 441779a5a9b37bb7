"""CPU tests that PIN the oracle (oracle/gie_oracle.c): the reference's own known-answer tests restated
(tests/test_cpu_reference.cpp:20-171), the golden fixtures produced by the reference's unmodified sources
(tests/golden/, see make_golden.py), and -- where oracle/_ref exists -- a direct bit-for-bit comparison."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def P(orc, *a, **k):
    return orc.Problem.P(*a, **k)


# ---- known-answer tests (tests/test_cpu_reference.cpp) ----------------------------------------------------------
def test_output_size_formula(orc, oracle):
    assert P(orc, 1, 1, 7, 7, 1, 3, 3, 2, 2, 0, 0).out_h == 3
    assert P(orc, 1, 1, 8, 8, 1, 3, 3, 2, 2, 1, 1).out_h == 4
    p = P(orc, 1, 1, 5, 9, 1, 5, 3, 1, 3, 2, 1)
    assert (p.out_h, p.out_w) == (5, 3)
    p = P(orc, 2, 3, 224, 224, 64, 7, 7, 2, 2, 3, 3)
    assert p.out_h == 112 and p.flops == 2 * 64 * (2 * 112 * 112) * (3 * 49)
    assert oracle.lib.orc_flops(p.desc()) == p.flops and oracle.lib.orc_out_h(p.desc()) == 112


def test_known_answers(orc, oracle):
    y, _ = oracle.conv2d(P(orc, 1, 1, 3, 3, 1, 3, 3, 1, 1, 0, 0), np.ones(9), np.ones(9))
    assert y.ravel().tolist() == [9.0]                                   # ones window
    y, _ = oracle.conv2d(P(orc, 1, 1, 3, 3, 1, 2, 2, 1, 1, 0, 0), np.arange(1, 10), [1, 0, 0, -1])
    assert y.ravel().tolist() == [-4.0] * 4                              # cross-correlation, kernel not flipped
    y, _ = oracle.conv2d(P(orc, 1, 1, 2, 2, 1, 3, 3, 1, 1, 1, 1), np.ones(4), np.ones(9))
    assert y.ravel().tolist() == [4.0] * 4                               # zero padding
    y, _ = oracle.conv2d(P(orc, 1, 1, 3, 3, 1, 3, 3, 1, 1, 1, 1), np.arange(1, 10), np.ones(9))
    assert (y.ravel()[0], y.ravel()[4], y.ravel()[8]) == (12.0, 45.0, 28.0)
    y, _ = oracle.conv2d(P(orc, 1, 1, 4, 4, 1, 1, 1, 2, 2, 0, 0), np.arange(16), [1.0])
    assert y.ravel().tolist() == [0.0, 2.0, 8.0, 10.0]                   # stride


def test_known_answer_channels_batch_bias_relu_and_scale(orc, oracle):
    p = P(orc, 2, 2, 1, 1, 2, 1, 1, 1, 1, 0, 0, bias=True, relu=True)
    y, s = oracle.conv2d(p, [1, 2, -3, 4], [1, 1, -1, 0.5], [0.25, -0.5])
    assert y.ravel().tolist() == [3.25, 0.0, 1.25, 4.5]
    assert abs(s.ravel()[0] - np.sqrt(5.0 + 9.0 + 0.0625)) < 1e-6


def test_identity_kernel_and_determinism(orc, oracle):
    p = P(orc, 2, 3, 5, 6, 3, 1, 1, 1, 1, 0, 0)
    x = oracle.rng(7).uniform(-1, 1, 2 * 3 * 5 * 6)
    w = np.zeros(9, np.float32)
    w[[0, 4, 8]] = 1
    y, _ = oracle.conv2d(p, x, w)
    assert np.array_equal(y.ravel(), x)
    p = P(orc, 2, 5, 9, 7, 4, 3, 3, 2, 1, 1, 1)
    r = oracle.rng(3)
    x, w = r.uniform(-1, 1, 2 * 5 * 9 * 7), r.uniform(-1, 1, 4 * 5 * 9)
    assert np.array_equal(oracle.conv2d(p, x, w)[0], oracle.conv2d(p, x, w)[0])


def test_quantization_helpers(orc, oracle):
    q = lambda pr, v: float(oracle.quantize(pr, [v])[0])
    assert q(orc.FP32, 0.1) == np.float32(0.1) and q(orc.FP16, 1.0) == 1.0
    assert q(orc.FP16, 0.1) != np.float32(0.1) and abs(q(orc.FP16, 0.1) - 0.1) < 1e-4 and abs(q(orc.BF16, 0.1) - 0.1) < 1e-3
    assert q(orc.TF32, 1.0 + 1.0 / 2048) == 1.0 + 1.0 / 1024     # tie -> away from zero
    assert q(orc.TF32, 1.0 + 1.0 / 4096) == 1.0


def test_error_metrics_detect_nan_and_over_tolerance(orc, oracle):
    p = P(orc, 1, 4, 4, 4, 1, 1, 1, 1, 1, 0, 0)
    ref, scale, test = np.ones(8, np.float32), np.ones(8, np.float32), np.ones(8, np.float32)
    assert oracle.compare(p, test, ref, scale).passed()
    test[3] = 1 + 1e-3
    m = oracle.compare(p, test, ref, scale)
    assert not m.passed() and m.over_tol == 1
    test[3] = np.nan
    m = oracle.compare(p, test, ref, scale)
    assert m.nan_count == 1 and not m.passed()


def test_invalid_problems_are_rejected(orc, oracle):
    bad = [(0, 1, 5, 5, 1, 3, 3, 1, 1, 0, 0), (1, 1, 2, 2, 1, 5, 5, 1, 1, 0, 0), (1, 1, 5, 5, 1, 3, 3, 0, 1, 0, 0),
           (1, 1, 5, 5, 1, 3, 3, 1, 1, -1, 0), (30000, 1, 512, 512, 1, 1, 1, 1, 1, 0, 0)]
    for a in bad:
        assert oracle.validate(P(orc, *a)) == orc.INVALID_ARGUMENT, a
    d = P(orc, 1, 1, 9, 9, 1, 3, 3, 1, 1, 0, 0)
    d.dilation_h = 2
    assert oracle.validate(d) == orc.UNSUPPORTED
    g = P(orc, 1, 4, 9, 9, 4, 3, 3, 1, 1, 0, 0)
    g.groups = 2
    assert oracle.validate(g) == orc.UNSUPPORTED


# ---- golden fixtures generated from the reference's own sources ---------------------------------------------------
def test_golden_rng_streams(orc, oracle):
    g = np.load(os.path.join(GOLD, "rng.npz"))
    for seed, key in ((0, "u64_seed0"), (0xC0FFEE, "u64_seed_c0ffee")):
        r = oracle.rng(seed)
        assert [r.next_u64() for _ in range(64)] == g[key].tolist()
    for d in range(4):
        for s in (0, 12345):
            assert np.array_equal(oracle.rng(s).draw(d, 257), g[f"dist{d}_seed{s}"])


def test_golden_storage_rounding(orc, oracle):
    g = np.load(os.path.join(GOLD, "quantize.npz"))
    for name, prec in (("fp16", orc.FP16), ("bf16", orc.BF16), ("tf32", orc.TF32)):
        got = oracle.quantize(prec, g["values"])
        assert np.array_equal(got.view(np.uint32), g[name].view(np.uint32)), name
    # raw 16-bit patterns round-trip to the same floats
    for prec in (orc.FP16, orc.BF16):
        q = oracle.quantize(prec, g["values"])
        assert np.array_equal(oracle.from_bits16(prec, oracle.to_bits16(prec, g["values"])).view(np.uint32), q.view(np.uint32))
    if hasattr(np, "float16"):
        finite = np.isfinite(g["values"]) & (np.abs(g["values"]) < 65000)
        assert np.array_equal(oracle.to_bits16(orc.FP16, g["values"])[finite], g["values"][finite].astype(np.float16).view(np.uint16))


def test_golden_convolutions(orc, oracle):
    g = np.load(os.path.join(GOLD, "conv.npz"))
    keys = sorted({k.rsplit("|", 1)[0] for k in g.files})
    assert len(keys) == 36
    for key in keys:
        name, prec, mode, dist, seed = key.split("|")
        p = orc.Problem.P(*orc.CORRECTNESS_SHAPES[name], precision=int(prec), bias=int(mode) >= 1, relu=int(mode) == 2)
        x, w, b = oracle.make_conv_data(p, int(seed), int(dist))
        sums = np.array([x.astype(np.float64).sum(), w.astype(np.float64).sum(), b.astype(np.float64).sum()])
        assert np.array_equal(sums, g[key + "|xsum"]), key           # same generated data
        y, sc = oracle.conv2d(p, x, w, b if p.has_bias else None)
        assert np.array_equal(y.view(np.uint32), g[key + "|y"].view(np.uint32)), key
        assert np.array_equal(sc.view(np.uint32), g[key + "|scale"].view(np.uint32)), key


def test_golden_tolerance_model(orc, oracle):
    g = np.load(os.path.join(GOLD, "tolerance.npz"))
    import ctypes as C
    for prec in (orc.FP32, orc.FP16, orc.BF16, orc.TF32):
        p = orc.Problem.P(1, 64, 8, 8, 8, 3, 3, 1, 1, 1, 1, precision=prec)
        got = []
        for r in (0.0, 0.5, -3.0):
            for s in (0.1, 2.0):
                for ir in (False, True):
                    t = oracle.tolerance(p, ir)
                    got.append(t.c_acc * t.u_acc * np.sqrt(float(t.k)) * s + t.c_out * t.u_out * abs(r) + t.c_inter * t.u_out * s +
                               t.c_in * t.u_in * s + t.abs_floor)
        assert np.allclose(got, g[str(prec)], rtol=1e-15, atol=0)


# ---- direct comparison with the compiled reference, where it exists (this container; not the GPU box necessarily) ----
def test_restatement_equals_compiled_reference(orc, oracle):
    if not orc.Reference.available():
        pytest.skip("oracle/_ref was not built on this machine (needs the reference checkout)")
    ref = orc.Reference()
    cell = 0
    for name, args in orc.CORRECTNESS_SHAPES.items():
        for prec in (orc.FP32, orc.FP16, orc.BF16):
            cell += 1
            p = orc.Problem.P(*args, precision=prec, bias=cell % 3 >= 1, relu=cell % 3 == 2)
            if p.flops > 2e8:
                continue
            x, w, b = ref.make_conv_data(p, 99 + cell, cell % 4)
            x2, w2, b2 = oracle.make_conv_data(p, 99 + cell, cell % 4)
            assert np.array_equal(x, x2) and np.array_equal(w, w2) and np.array_equal(b, b2)
            yr, sr = ref.conv2d(p, x, w, b if p.has_bias else None)
            yo, so = oracle.conv2d(p, x, w, b if p.has_bias else None)
            assert np.array_equal(yr, yo) and np.array_equal(sr, so), name
            noisy = yo + np.float32(1e-3) * oracle.rng(cell).draw(1, yo.size).reshape(yo.shape)
            mo, mr = oracle.compare(p, noisy, yo, so), ref.compare(p, noisy, yo, so)
            assert mo.over_tol == mr["over_tol"] and abs(mo.worst_tol_ratio - mr["worst_tol_ratio"]) <= 1e-9 * mr["worst_tol_ratio"]
            assert oracle.validate(p) == ref.validate(p) == 0


def test_rmsnorm_oracle_properties(orc, oracle):
    """No reference library code exists for the RMSNorm oracle (it is inline in tests/test_rmsnorm.cpp:31-48):
    check the restatement against an independent numpy formula."""
    r = oracle.rng(1)
    x = r.draw(orc.DIST_NORMAL, 6 * 100).reshape(6, 100)
    res = r.draw(orc.DIST_NORMAL, 6 * 100).reshape(6, 100)
    g = r.uniform(0.5, 1.5, 100)
    y, ro = oracle.rmsnorm(x, g, 1e-6, orc.BF16, res)
    s = oracle.quantize(orc.BF16, (x.astype(np.float64) + res.astype(np.float64)).astype(np.float32)).astype(np.float64)
    assert np.array_equal(ro, s.astype(np.float32))
    exp = s / np.sqrt((s * s).mean(axis=1, keepdims=True) + 1e-6) * g
    assert np.allclose(y, exp, rtol=1e-12, atol=0)
    y2, _ = oracle.rmsnorm(x, g, 1e-6, orc.FP32)
    xd = x.astype(np.float64)
    assert np.allclose(y2, xd / np.sqrt((xd * xd).mean(axis=1, keepdims=True) + 1e-6) * g, rtol=1e-12)


def test_chain_glue_oracles(orc, oracle):
    x = oracle.rng(2).draw(orc.DIST_NORMAL, 2 * 3 * 7 * 9).reshape(2, 3, 7, 9)
    y = oracle.maxpool2d(x, 3, 2, 1)
    assert y.shape == (2, 3, 4, 5)
    xp = np.full((2, 3, 9, 11), -np.inf, np.float32)
    xp[:, :, 1:8, 1:10] = x
    exp = np.stack([[ [[xp[b, c, 2 * i:2 * i + 3, 2 * j:2 * j + 3].max() for j in range(5)] for i in range(4)] for c in range(3)] for b in range(2)])
    assert np.array_equal(y, exp.astype(np.float32))
    a, b = oracle.quantize(orc.FP16, x.ravel()), oracle.quantize(orc.FP16, x.ravel()[::-1].copy())
    assert np.array_equal(oracle.add_relu(orc.FP16, a, b, True), np.maximum(oracle.quantize(orc.FP16, a + b), 0))


def test_e4m3_grid_matches_an_independent_conversion():
    """The FP8 E4M3 rounding used to prepare inputs for the FP8 extension (round to nearest even, saturating) against
    torch's float8_e4m3fn conversion, values and bit patterns, including subnormals, ties, signed zero and the largest
    finite value; and every value of the grid is exactly an FP16 value (so the FP16 oracle applies)."""
    import torch
    from oracle import oracle as orc_mod
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.uniform(-1, 1, 50000), rng.normal(0, 100, 50000), rng.uniform(-0.02, 0.02, 50000),
                        [0.0, -0.0, 448, 449, 500, -1000, 2 ** -9, 2 ** -10, 1.5 * 2 ** -9, 2.5 * 2 ** -9, 0.0625 * 1.0625]]).astype(np.float32)
    q = orc_mod.e4m3_quantize(x)
    t = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert np.array_equal(q, t.float().numpy())
    assert np.array_equal(orc_mod.e4m3_bits(q), t.view(torch.uint8).numpy())
    assert np.array_equal(q, q.astype(np.float16).astype(np.float32))
