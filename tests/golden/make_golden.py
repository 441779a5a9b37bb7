"""Generates the golden fixtures in this directory from the reference library's OWN oracle (oracle/_ref/libgie_ref.so,
built by `make -C oracle ref` where the reference checkout exists).  Run here, commit the .npz files; the tests then
check the C restatement (oracle/gie_oracle.c) -- and through it the CUDA path -- against them on any machine.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import __graft_entry__ as entry  # noqa: E402

orc = entry.load_oracle()
orc.build(ref=True)
ref = orc.Reference()

# 1. generator streams and distributions
np.savez_compressed(os.path.join(HERE, "rng.npz"),
                    u64_seed0=ref.rng_u64(0, 64), u64_seed_c0ffee=ref.rng_u64(0xC0FFEE, 64),
                    **{f"dist{d}_seed{s}": ref.rng_draw(s, d, 257) for d in range(4) for s in (0, 12345)})

# 2. storage rounding on a value set with ties, subnormals, overflow, signed zero, inf
rs = np.random.RandomState(0)
vals = np.concatenate([
    (rs.randn(4000) * 10.0 ** rs.randint(-10, 6, 4000)).astype(np.float32),
    np.array([0.0, -0.0, 65504, 65519.996, 65520, 65536, 1e-8, 5.9604645e-8, 2.9802322e-8, 2.9802326e-8, 6.1035156e-5,
              6.0975552e-5, 1 + 2 ** -11, 1 + 2 ** -10 + 2 ** -11, 1 + 2 ** -12, 3.3895314e38, np.inf, -np.inf, 1 + 2 ** -8, 1 + 2 ** -9],
             np.float32)])
np.savez_compressed(os.path.join(HERE, "quantize.npz"), values=vals,
                    fp16=ref.quantize(orc.FP16, vals), bf16=ref.quantize(orc.BF16, vals), tf32=ref.quantize(orc.TF32, vals))

# 3. convolution outputs + scales for a subset of the reference's correctness shapes (small enough to commit)
conv = {}
names = ["tiny_1ch_5x5_k3", "scalar_1x1_k1", "rgb_8x8_k3p1", "odd_unequal_k5s2", "irregular_c7_o9_s2",
         "kernel_eq_map_7x7", "small_b8_4x4", "boundary_pad2_3x3", "boundary_pad4_k5", "aniso_k3x5_s2x1", "k1x3", "k3x1"]
cell = 0
for name in names:
    for prec in (orc.FP32, orc.FP16, orc.BF16):
        mode = cell % 3
        dist = cell % 4
        seed = 0xC0FFEE + cell
        cell += 1
        p = orc.Problem.P(*orc.CORRECTNESS_SHAPES[name], precision=prec, bias=mode >= 1, relu=mode == 2)
        x, w, b = ref.make_conv_data(p, seed, dist)
        y, sc = ref.conv2d(p, x, w, b if p.has_bias else None)
        key = f"{name}|{prec}|{mode}|{dist}|{seed}"
        conv[key + "|y"] = y
        conv[key + "|scale"] = sc
        conv[key + "|xsum"] = np.array([x.astype(np.float64).sum(), w.astype(np.float64).sum(), b.astype(np.float64).sum()])
np.savez_compressed(os.path.join(HERE, "conv.npz"), **conv)

# 4. tolerance model samples
tol = {}
for prec in (orc.FP32, orc.FP16, orc.BF16, orc.TF32):
    p = orc.Problem.P(1, 64, 8, 8, 8, 3, 3, 1, 1, 1, 1, precision=prec)
    tol[f"{prec}"] = np.array([ref.tol(p, r, s, ir) for r in (0.0, 0.5, -3.0) for s in (0.1, 2.0) for ir in (False, True)])
np.savez_compressed(os.path.join(HERE, "tolerance.npz"), **tol)
print("golden fixtures written:", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
