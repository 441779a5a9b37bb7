"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol include/gie_b200.h declares, and
its host-side logic (validation status codes, capability answers, workspace layout, configuration selection) behaves
as the reference's (tests/test_cpu_reference.cpp:158-171, tests/test_dispatcher.cpp, tests/test_validation.cpp).
No GPU is touched: nothing here launches or allocates on a device."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gie_b200.h")).read()
    return sorted(set(re.findall(r"GIEB_API\s+[\w\s\*]+?\b(gieb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    names = declared_symbols()
    assert len(names) >= 17, names
    out = subprocess.check_output(["nm", "-D", "--defined-only", pkg.LIB_PATH], text=True)
    exported = set(re.findall(r"\b(gieb_\w+)\b", out))
    assert set(names) <= exported, sorted(set(names) - exported)
    lib = pkg.lib()
    for n in names:
        assert getattr(lib, n) is not None
    assert lib.gieb_version() >= 1


def P(pkg, *a, **k):
    return pkg.ConvProblem(*a, **k)


def test_validate_status_codes(pkg):
    ok = P(pkg, 1, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1)
    pkg.validate_problem(ok)
    for bad in [P(pkg, 0, 1, 5, 5, 1, 3, 3), P(pkg, 1, 1, 2, 2, 1, 5, 5), P(pkg, 1, 1, 5, 5, 1, 3, 3, 0, 1),
                P(pkg, 1, 1, 5, 5, 1, 3, 3, 1, 1, -1, 0), P(pkg, 30000, 1, 512, 512, 1, 1, 1), P(pkg, 1, 1, 5, 5, 1, 3, 3, precision=9)]:
        with pytest.raises(pkg.GieError) as e:
            pkg.validate_problem(bad)
        assert e.value.code == pkg.INVALID_ARGUMENT, bad
    for uns in [P(pkg, 1, 1, 9, 9, 1, 3, 3, dilation_h=2), P(pkg, 1, 4, 9, 9, 4, 3, 3, groups=2)]:
        with pytest.raises(pkg.GieError) as e:
            pkg.validate_problem(uns)
        assert e.value.code == pkg.UNSUPPORTED
    assert "dilation" in pkg.last_error() or "grouped" in pkg.last_error()


def test_validation_matches_oracle_on_the_correctness_shapes(pkg, orc, oracle):
    for name, args in orc.CORRECTNESS_SHAPES.items():
        for prec in (orc.FP32, orc.FP16, orc.BF16):
            p = orc.Problem.P(*args, precision=prec)
            assert oracle.validate(p) == 0
            cp = P(pkg, *args, precision=prec)
            pkg.validate_problem(cp)
            assert (cp.out_h, cp.out_w, cp.flops) == (p.out_h, p.out_w, p.flops)
            info = pkg.query(cp)
            assert info.supported == 1, (name, prec, info.reason)   # no (shape, precision) cell may be left without a kernel


def test_epilogue_warp_count_follows_the_plan(pkg):
    """CTAs that own their SM run 16 epilogue warps (640 threads): every 256-column tile whose ring leaves no room for a
    second CTA, and 128-column tiles with one tile per CTA; everything else keeps 8 (384 threads)."""
    c2 = pkg.query(P(pkg, 32, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1, precision=pkg.FP16))
    # a long reduction with enough pixels: 256-pixel tiles of CTA pairs, each CTA alone on its SM
    assert c2.supported and c2.threads_per_block == 640 and (c2.cfg.tile_m, c2.cfg.tile_n, c2.cfg.split_k, c2.cfg.cta_pair) == (256, 128, 1, 2)
    single = pkg.query(P(pkg, 32, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1, precision=pkg.FP16), pkg.make_cfg(cta_pair=1))
    assert single.supported and single.threads_per_block == 640 and (single.cfg.tile_m, single.cfg.tile_n, single.cfg.cta_pair) == (128, 128, 1)
    c3 = pkg.query(P(pkg, 64, 512, 28, 28, 128, 1, 1, precision=pkg.FP16))
    assert c3.supported and c3.variant == 2 and c3.threads_per_block == 384 and c3.launches == 1   # 416 tiles on 148 CTAs; weights in place
    wide = pkg.query(P(pkg, 16, 128, 54, 54, 256, 3, 3, 2, 2, 1, 1, precision=pkg.FP16), pkg.make_cfg(tile_n=256, tile_k=64, stages=4))
    assert wide.supported and wide.threads_per_block == 640                                         # 27 x 27 output planes: pixel-lane kernel
    shallow = pkg.query(P(pkg, 16, 128, 54, 54, 256, 3, 3, 2, 2, 1, 1, precision=pkg.FP16), pkg.make_cfg(tile_n=128, tile_k=64, stages=2))
    assert shallow.supported and shallow.threads_per_block == 384                                   # two CTAs share an SM
    # NCHW output planes of 28 x 28 (16-byte multiples): transposed accumulator, a short epilogue on eight warps
    tr = pkg.query(P(pkg, 64, 512, 28, 28, 128, 1, 1, precision=pkg.FP16), pkg.make_cfg(tile_m=128, tile_n=128, tile_k=64, stages=6))
    assert tr.supported and tr.threads_per_block == 384 and tr.dynamic_smem_bytes == 1024 + 3072 + 6 * 32768 + 8 * 2048


def test_query_precision_routing_and_reasons(pkg):
    base = (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1)
    i32 = pkg.query(P(pkg, *base, precision=pkg.FP32))
    assert i32.supported and i32.variant == 3 and i32.workspace_bytes == 0 and i32.launches == 1
    i16 = pkg.query(P(pkg, *base, precision=pkg.FP16))
    assert i16.supported and i16.variant == 1 and i16.threads_per_block == 384 and i16.padded_channels == 64
    ipw = pkg.query(P(pkg, 2, 64, 14, 14, 64, 1, 1, precision=pkg.BF16))
    assert ipw.supported and ipw.variant == 4                       # 1x1 / stride 1 / pad 0 -> tiled activation loads
    idr = pkg.query(P(pkg, 2, 64, 28, 28, 64, 1, 1, precision=pkg.BF16))
    assert idr.supported and idr.variant == 2                       # H*W % 8 == 0 -> straight from NCHW, no activation repack
    assert not pkg.query(P(pkg, 2, 64, 14, 14, 64, 1, 1, precision=pkg.FP16), pkg.make_cfg(variant=2)).supported
    tf = pkg.query(P(pkg, *base, precision=pkg.TF32))  # FP32 storage on the tensor cores (kind::tf32)
    assert tf.supported and tf.variant in (1, 4) and tf.cfg.tile_k in (8, 16, 32)
    assert not pkg.query(P(pkg, *base, precision=pkg.TF32, flags=pkg.FLAG_OUTPUT_NHWC)).supported
    big_stride = pkg.query(P(pkg, 1, 16, 64, 64, 16, 3, 3, 9, 9, 1, 1, precision=pkg.FP16))
    assert not big_stride.supported and b"stride" in big_stride.reason
    assert not pkg.query(P(pkg, *base, precision=pkg.FP16), pkg.make_cfg(variant=3)).supported
    assert not pkg.query(P(pkg, *base, precision=pkg.FP16), pkg.make_cfg(variant=4)).supported
    assert not pkg.query(P(pkg, *base, precision=pkg.FP32), pkg.make_cfg(variant=1)).supported


def test_query_rejects_impossible_configurations(pkg):
    p = P(pkg, 8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, precision=pkg.FP16)
    too_much_smem = pkg.query(p, pkg.make_cfg(tile_n=128, tile_k=64, stages=8))
    assert not too_much_smem.supported and b"shared memory" in too_much_smem.reason
    assert not pkg.query(p, pkg.make_cfg(tile_n=48)).supported
    assert not pkg.query(p, pkg.make_cfg(tile_k=48)).supported
    assert not pkg.query(p, pkg.make_cfg(tile_m=64)).supported
    assert not pkg.query(p, pkg.make_cfg(stages=1)).supported
    short = pkg.query(P(pkg, 8, 64, 14, 14, 64, 1, 1, precision=pkg.FP16), pkg.make_cfg(split_k=4))
    assert not short.supported and b"split" in short.reason          # reduction too short (one slab)
    assert not pkg.query(p, pkg.make_cfg(tile_m=256, tile_n=256, tile_k=64, stages=4)).supported  # 4 x 64 KiB ring


def test_workspace_layout_and_padding(pkg):
    # C=130 -> padded channels; workspace = align256(B*H*W*Cp*2) + align256(O*R*S*Cp*2) (+ split * align4(|Y|) * 4)
    p = P(pkg, 2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1, precision=pkg.FP16)
    a256 = lambda v: (v + 255) // 256 * 256
    for tk, cp in ((16, 144), (32, 160), (64, 192)):
        i = pkg.query(p, pkg.make_cfg(tile_k=tk, split_k=1))
        assert i.padded_channels == cp
        assert i.workspace_bytes == a256(2 * 81 * cp * 2) + a256(130 * 9 * cp * 2)
    i = pkg.query(p, pkg.make_cfg(tile_k=32, split_k=3))
    ys = 2 * 130 * 81
    assert i.cfg.split_k == 3 and i.workspace_bytes == a256(2 * 81 * 160 * 2) + a256(130 * 9 * 160 * 2) + a256(3 * ((ys + 3) // 4 * 4) * 4)
    assert i.launches == 3
    pre = P(pkg, 2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1, precision=pkg.FP16, flags=pkg.FLAG_WEIGHTS_PREPACKED)
    assert pkg.query(pre, pkg.make_cfg(tile_k=32, split_k=1)).workspace_bytes == a256(2 * 81 * 160 * 2)
    stem = P(pkg, 1, 3, 224, 224, 64, 7, 7, 2, 2, 3, 3, precision=pkg.FP16)
    assert pkg.query(stem, pkg.make_cfg(variant=1)).padded_channels == 16
    auto = pkg.query(stem)  # few channels: the 7 taps of a filter row become 7 * 3 -> 32 channels of a 7 x 1 convolution
    assert auto.variant == 5 and auto.padded_channels == 32
    # stride 2, 3 channels: column pairs are stored once (115 positions of 16 bytes per input row: 2 of padding on the left,
    # 112 pairs, 1 on the right) and adjacent windows overlap in memory
    assert auto.workspace_bytes == a256(1 * 224 * 115 * 16) + a256(64 * 7 * 32 * 2)
    assert pkg.query(P(pkg, 1, 96, 27, 27, 192, 5, 5, 1, 1, 2, 2, precision=pkg.FP16)).padded_channels == 96


def test_selection_is_deterministic_and_fills_the_machine(pkg):
    """Ranking determinism (tests/test_dispatcher.cpp) and sanity of the choice: never more split-K than the
    reduction allows, every slice non-empty, grid within limits, shared memory within the per-CTA limit."""
    shapes = [(32, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1), (64, 512, 28, 28, 128, 1, 1, 1, 1, 0, 0), (8, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1),
              (16, 128, 56, 56, 256, 3, 3, 2, 2, 1, 1), (1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1), (256, 64, 56, 56, 256, 1, 1, 1, 1, 0, 0),
              (256, 3, 224, 224, 64, 7, 7, 2, 2, 3, 3), (1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0)]
    for a in shapes:
        p = P(pkg, *a, precision=pkg.FP16, has_bias=True, relu=True)
        i1, i2 = pkg.query(p), pkg.query(p)
        c = i1.cfg
        assert (c.tile_m, c.tile_n, c.tile_k, c.stages, c.split_k) == (i2.cfg.tile_m, i2.cfg.tile_n, i2.cfg.tile_k, i2.cfg.stages, i2.cfg.split_k)
        assert i1.supported and c.tile_m in (128, 256) and c.tile_n in (32, 64, 128, 256) and c.tile_k in (16, 32, 64)
        assert 2 <= c.stages <= 8 and i1.dynamic_smem_bytes <= 232448
        total_kb = a[5] * a[6] * (i1.padded_channels // c.tile_k)
        assert 1 <= c.split_k <= max(1, total_kb // 2)
        pixels = a[0] * p.out_h * p.out_w
        rows = a[0] * -(-(a[2] * a[3]) // 64) * 64 if i1.variant == 2 else pixels   # direct NCHW route counts 64-pixel boxes
        if i1.variant == 5 and a[8] == 2 and a[1] <= 4 and p.out_w <= 128:
            rows = a[0] * p.out_h * 128   # position strips: one 128-row box per output row
        ctas_per_tile = 2 if c.cta_pair == 2 else 1   # a 256-pixel tile of a CTA pair is two CTAs
        assert i1.num_blocks == -(-rows // c.tile_m) * -(-a[4] // c.tile_n) * c.split_k * ctas_per_tile
    # the small deep layer gets split-K, the big ones do not
    assert pkg.query(P(pkg, 1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1, precision=pkg.FP16)).cfg.split_k > 1
    assert pkg.query(P(pkg, 256, 64, 56, 56, 256, 1, 1, precision=pkg.FP16)).cfg.split_k == 1


def test_static_scratch_size_check_needs_no_gpu(pkg):
    """The allocation-free entry point refuses oversized problems before touching the device."""
    big = P(pkg, 64, 512, 28, 28, 128, 1, 1, precision=pkg.FP16)
    with pytest.raises(pkg.GieError) as e:
        pkg.conv_forward_static(big, 256, 256, None, 256, 0)
    assert e.value.code == pkg.WORKSPACE_TOO_SMALL


def test_rmsnorm_argument_checks_need_no_gpu(pkg):
    for args in [(1, 4, 16, 32, 16, None, None), (1, 4, 16, 32, 48, 64, None), (1, 0, 16, 32, 48, None, None), (0, 4, 16, 32, 48, None, None),
                 (1, 4, None, 32, 48, None, None)]:
        rows, hidden, x, g, y, ri, ro = args
        with pytest.raises(pkg.GieError) as e:
            pkg.rmsnorm_forward(rows, hidden, 1e-6, 0, x, g, y, ri, ro, 0)
        assert e.value.code == pkg.INVALID_ARGUMENT
