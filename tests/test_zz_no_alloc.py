"""gieb_conv_forward_static: the forward call for callers that may not allocate device memory (its scratch is an array
inside the library image).  Collected last on purpose.  It must give the same bits as the plan API, on two calls in a
row that share the built-in scratch, whether this file runs alone in a fresh process or after every other test."""
import numpy as np
import pytest

import gpu_util as gu

pytestmark = pytest.mark.gpu


def _both_ways(pkg, orc, oracle, args, prec, seed, cfg_kw):
    import torch
    p = orc.Problem.P(*args, precision=prec, bias=True, relu=True)
    x, w, b = oracle.make_conv_data(p, seed, seed % 4)
    cfg = pkg.make_cfg(**cfg_kw) if cfg_kw else None
    # existing entry points: plan + caller workspace
    y_plan, plan, out_plan = gu.run_conv(pkg, oracle, p, x, w, b, cfg=cfg)
    # new entry point: no plan, no workspace
    tx, px = gu.to_device_storage(oracle, p.precision, x)
    tw, pw = gu.to_device_storage(oracle, p.precision, w)
    tb, pb = gu.to_device_storage(oracle, p.precision, b)
    out = gu.OutBuf(p.precision, int(np.prod(p.y_shape)))
    st = torch.cuda.current_stream().cuda_stream
    pkg.conv_forward_static(gu.pkg_problem(pkg, p), px, pw, pb, out.ptr, st, cfg)  # first call: address look-up, module load
    assert pkg.conv_static_status(st) == 0
    torch.cuda.synchronize()
    out.t.view(torch.uint8).fill_(0xFF)
    free_before = torch.cuda.mem_get_info()[0]
    pkg.conv_forward_static(gu.pkg_problem(pkg, p), px, pw, pb, out.ptr, st, cfg)
    assert pkg.conv_static_status(st) == 0, "a bounded device-side wait ran out inside the allocation-free call"
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
    got = out.read(oracle).reshape(p.y_shape)  # also checks the guard bands
    assert np.array_equal(out.raw_bits(), out_plan.raw_bits()), "static-scratch call differs from the plan API"
    ref, scale = oracle.conv2d(p, x, w, b)
    assert oracle.compare(p, got, ref, scale).passed()


def test_static_scratch_call_matches_plan_api_twice_in_a_row(pkg, orc, oracle):
    # two different problems back to back: the second one sees the first one's leftovers in the shared scratch
    _both_ways(pkg, orc, oracle, (4, 24, 12, 12, 40, 3, 3, 1, 1, 1, 1), orc.FP16, 101, dict(tile_n=64, tile_k=32, stages=3, split_k=3))
    _both_ways(pkg, orc, oracle, (2, 70, 9, 11, 33, 3, 3, 2, 2, 1, 1), orc.BF16, 102, None)
    # and the first one again, after the scratch has held something else
    _both_ways(pkg, orc, oracle, (4, 24, 12, 12, 40, 3, 3, 1, 1, 1, 1), orc.FP16, 101, dict(tile_n=64, tile_k=32, stages=3, split_k=3))


def test_static_scratch_refuses_problems_beyond_its_size(pkg, orc):
    import torch
    big = orc.BASELINE_CONFIGS["c3_fp16"]           # needs ~51 MB of scratch
    t = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(pkg.GieError) as e:
        pkg.conv_forward_static(gu.pkg_problem(pkg, big), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 0)
    assert e.value.code == pkg.WORKSPACE_TOO_SMALL
    assert "bytes of scratch" in str(e.value)
    torch.cuda.synchronize()


def test_static_scratch_call_refuses_a_fused_residual(pkg, orc):
    """The allocation-free call has no residual operand: the flag is refused before anything is launched."""
    import torch
    p = orc.Problem.P(2, 32, 8, 8, 32, 3, 3, 1, 1, 1, 1, precision=orc.FP16, bias=True, relu=True)
    t = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(pkg.GieError) as e:
        pkg.conv_forward_static(gu.pkg_problem(pkg, p, pkg.FLAG_RESIDUAL | pkg.FLAG_OUTPUT_NHWC), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                t.data_ptr(), 0)
    assert e.value.code == pkg.UNSUPPORTED
    torch.cuda.synchronize()
