"""GPU parity of the ResNet-50-shaped convolution chain: every layer's output is checked against the CPU oracle fed
with the GPU's OWN input of that layer (so tolerances stay meaningful over 53 layers), the glue operators bit-exactly,
and the CUDA-graph replay bit-exactly against the eager run (tests/test_cuda_graph.cu:110-137 analogue)."""
import numpy as np
import pytest

import gpu_util as gu

pytestmark = pytest.mark.gpu


def _host_weights(orc, oracle, ops, precision, seed):
    from cuda_inference_b200.chain import layer_weight_bound
    out = []
    li = 0
    for op in ops:
        if op.kind != "conv":
            continue
        s = op.shape
        r = oracle.rng(seed + li)
        w = oracle.quantize(precision, r.draw(orc.DIST_UNIFORM, s.w_elems, layer_weight_bound(s, op.relu)))
        b = oracle.quantize(precision, r.uniform(-0.1, 0.1, s.out_channels))
        out.append((w, b))
        li += 1
    return out


def _run_chain_case(pkg, orc, oracle, batch, image, precision, seed, layout="nchw", tune=False, fuse_residual=None):
    import torch
    from cuda_inference_b200.chain import ConvChain
    from cuda_inference_b200 import workloads as wl
    ops, _ = wl.resnet50_chain(batch, precision, image)
    hw = _host_weights(orc, oracle, ops, precision, seed)
    chain = ConvChain(batch, precision, image, weights=[(oracle.to_bits16(precision, w), oracle.to_bits16(precision, b)) for w, b in hw],
                      layout=layout, tune=tune, fuse_residual=fuse_residual)
    x = oracle.quantize(precision, oracle.rng(seed + 1000).draw(orc.DIST_NORMAL, batch * 3 * image * image))
    chain.input.view(torch.int16).copy_(torch.from_numpy(oracle.to_bits16(precision, x).view(np.int16)).cuda())
    for t in list(chain.slots.values())[1:]:
        t.view(torch.int16).fill_(-1)  # NaN pattern
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        chain.enqueue(stream.cuda_stream)
    stream.synchronize()
    assert chain.device_status() == 0

    def slot(i):
        c, h, w = chain.slot_shapes[i]
        raw = chain.slots[i].view(torch.int16).cpu().numpy().view(np.uint16)
        vals = oracle.from_bits16(precision, raw)
        if layout == "nhwc" and i != 0:  # every tensor but the input image is channel-contiguous
            return np.ascontiguousarray(vals.reshape(batch, h, w, c).transpose(0, 3, 1, 2))
        return vals.reshape(batch, c, h, w)

    ci = 0
    worst = 0.0
    for op in chain.ops:
        got = slot(op.dst)
        assert np.all(np.isfinite(got)), f"non-finite output at {op.kind} -> slot {op.dst}"
        if op.kind == "conv":
            s = op.shape
            fused = chain.fused and op.other >= 0
            p = orc.Problem.P(s.batch, s.in_channels, s.in_h, s.in_w, s.out_channels, s.kernel, s.kernel, s.stride, s.stride, s.pad, s.pad,
                              precision, True, op.relu and not fused)
            w, b = hw[op.layer]
            ci += 1
            ref, scale = oracle.conv2d(p, slot(op.src), w.reshape(p.w_shape), b)
            if fused:  # y = act(conv + bias + residual), one rounding
                res = slot(op.other).astype(np.float64)
                ref = ref.astype(np.float64) + res
                if op.relu:
                    ref = np.maximum(ref, 0.0)
                ref = ref.astype(np.float32)
                scale = (scale.astype(np.float64) + np.abs(res)).astype(np.float32)
            m = oracle.compare(p, got, ref, scale)
            assert m.passed(), f"conv {ci} {s}: {m.summary()}"
            worst = max(worst, m.worst_tol_ratio)
        elif op.kind == "maxpool":
            _, _, _, k, st, pad = op.pool
            assert np.array_equal(got, oracle.maxpool2d(slot(op.src), k, st, pad))
        else:
            assert np.array_equal(got.ravel(), oracle.add_relu(precision, slot(op.src).ravel(), slot(op.other).ravel(), op.relu))
    eager = chain.output.view(torch.int16).cpu().numpy().copy()
    assert np.abs(slot(len(chain.slots) - 1)).max() < 6e4
    # one CUDA graph for the whole chain; replay must reproduce the eager bits
    chain.capture(stream)
    nodes = chain.launches
    chain.output.view(torch.int16).fill_(-1)
    with torch.cuda.stream(stream):
        chain.replay()
    stream.synchronize()
    assert np.array_equal(chain.output.view(torch.int16).cpu().numpy(), eager)
    return worst, nodes


def test_chain_small_images_batch2_fp16(pkg, orc, oracle):
    worst, nodes = _run_chain_case(pkg, orc, oracle, batch=2, image=64, precision=orc.FP16, seed=0)
    assert nodes >= 53 + 17 + 17  # every convolution, pool and add; a repack launch only where a tensor must be rearranged


def test_chain_channel_contiguous_fused_residual_fp16(pkg, orc, oracle):
    """Channel-contiguous chain: prepacked weights, no repack between layers, residual add + ReLU inside the epilogue
    of each block's last convolution.  One launch per convolution except the stem (which repacks the NCHW image)."""
    worst, nodes = _run_chain_case(pkg, orc, oracle, batch=2, image=64, precision=orc.FP16, seed=0, layout="nhwc")
    assert 53 + 2 <= nodes <= 53 + 2 + 20  # convolutions + stem repack + max-pool (+ workspace reductions of tiny layers)


def test_chain_nchw_fused_residual(pkg, orc, oracle):
    """NCHW tensors throughout, residual add + ReLU inside the epilogue of each block's last convolution (no add launches).
    At 224 x 224 the 56 x 56 and 28 x 28 layers take the transposed-accumulator kernels, which read the residual as the
    lane's own 64-byte pixel runs; the small case runs BF16 through the pixel-lane kernels."""
    worst, nodes = _run_chain_case(pkg, orc, oracle, batch=1, image=224, precision=orc.FP16, seed=4, fuse_residual=True)
    assert nodes <= 53 + 1 + 53 + 20  # no add launches: convolutions, max-pool, at most one repack each (+ reductions)
    _run_chain_case(pkg, orc, oracle, batch=3, image=32, precision=orc.BF16, seed=6, fuse_residual=True)


def test_chain_with_measured_configurations(pkg, orc, oracle):
    """tune=True times candidate configurations per layer and keeps the fastest: whatever wins must still match the
    oracle layer by layer."""
    _run_chain_case(pkg, orc, oracle, batch=2, image=64, precision=orc.FP16, seed=9, layout="nhwc", tune=True)
    _run_chain_case(pkg, orc, oracle, batch=2, image=64, precision=orc.FP16, seed=9, layout="nchw", tune=True)


def test_chain_channel_contiguous_bf16(pkg, orc, oracle):
    _run_chain_case(pkg, orc, oracle, batch=3, image=32, precision=orc.BF16, seed=5, layout="nhwc")


def test_chain_channel_contiguous_full_size_image(pkg, orc, oracle):
    _run_chain_case(pkg, orc, oracle, batch=1, image=224, precision=orc.FP16, seed=3, layout="nhwc")


def test_chain_full_size_image_batch1_fp16(pkg, orc, oracle):
    _run_chain_case(pkg, orc, oracle, batch=1, image=224, precision=orc.FP16, seed=3)


def test_chain_bf16(pkg, orc, oracle):
    _run_chain_case(pkg, orc, oracle, batch=3, image=32, precision=orc.BF16, seed=5)


def test_batch_shards_are_independent_replicas(pkg, orc, oracle):
    """Images do not interact: running images [0,2) and [2,4) as two chains gives the same bits as one chain of 4
    when both use the same tile configuration per layer (replica correctness, the basis of the multi-GPU run)."""
    import torch
    from cuda_inference_b200.chain import ConvChain
    prec, image = orc.FP16, 32
    full = ConvChain(4, prec, image, seed=11)
    x = torch.randn(4 * 3 * image * image, device="cuda").to(torch.float16)
    full.input.copy_(x)
    st = torch.cuda.current_stream().cuda_stream
    full.enqueue(st)
    torch.cuda.synchronize()
    whole = full.output.float().cpu().numpy().reshape(4, -1)
    for r in range(2):
        part = ConvChain(2, prec, image, seed=11)
        part.input.copy_(x.view(4, -1)[2 * r:2 * r + 2].reshape(-1))
        part.enqueue(st)
        torch.cuda.synchronize()
        got = part.output.float().cpu().numpy().reshape(2, -1)
        ref = whole[2 * r:2 * r + 2]
        assert np.all(np.isfinite(got))
        # split-K choices may differ with the batch, so allow FP16 rounding-level differences
        assert np.allclose(got, ref, rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(ref).max())))
