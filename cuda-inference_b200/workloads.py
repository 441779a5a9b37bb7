"""Benchmark workloads: the convolution shapes the headline numbers are quoted on, the RMSNorm shape, and the layer
list of the ResNet-50-shaped convolution chain.  Pure shape data -- no tensors, no device code."""
from __future__ import annotations

from dataclasses import dataclass

FP32, FP16, BF16 = 0, 1, 2
FP8_E4M3 = 4  # x and w as FP8 E4M3 bytes, float bias, FP16 y (an extension of this library)


@dataclass(frozen=True)
class ConvShape:
    batch: int
    in_channels: int
    in_h: int
    in_w: int
    out_channels: int
    kernel: int
    stride: int
    pad: int
    precision: int = FP16

    @property
    def out_h(self) -> int:
        return (self.in_h + 2 * self.pad - self.kernel) // self.stride + 1

    @property
    def out_w(self) -> int:
        return (self.in_w + 2 * self.pad - self.kernel) // self.stride + 1

    @property
    def flops(self) -> int:
        return 2 * self.batch * self.out_h * self.out_w * self.out_channels * self.in_channels * self.kernel * self.kernel

    @property
    def elem_size(self) -> int:
        """Bytes per element of x and w (y is FP16 for FP8 inputs, else the same type)."""
        return 4 if self.precision == FP32 else (1 if self.precision == FP8_E4M3 else 2)

    @property
    def x_elems(self) -> int:
        return self.batch * self.in_channels * self.in_h * self.in_w

    @property
    def w_elems(self) -> int:
        return self.out_channels * self.in_channels * self.kernel * self.kernel

    @property
    def y_elems(self) -> int:
        return self.batch * self.out_channels * self.out_h * self.out_w

    @property
    def algorithmic_bytes(self) -> int:
        """X + W + Y + bias, each moved once, in the storage type."""
        if self.precision == FP8_E4M3:
            return self.x_elems + self.w_elems + 2 * self.y_elems + 4 * self.out_channels
        return (self.x_elems + self.w_elems + self.y_elems + self.out_channels) * self.elem_size


# name -> (shape, roofline bound).  All run with fused bias + ReLU.
CONV_WORKLOADS = {
    "c1": (ConvShape(1, 64, 56, 56, 64, 3, 1, 1, FP32), "fp32"),
    "c2": (ConvShape(32, 256, 14, 14, 256, 3, 1, 1, FP16), "tensor"),
    "c3_fp16": (ConvShape(64, 512, 28, 28, 128, 1, 1, 0, FP16), "hbm"),
    "c3_bf16": (ConvShape(64, 512, 28, 28, 128, 1, 1, 0, BF16), "hbm"),
    "c2_fp8": (ConvShape(32, 256, 14, 14, 256, 3, 1, 1, FP8_E4M3), "tensor"),   # c2 with FP8 E4M3 inputs (an extension; FP16 output)
    "c4a": (ConvShape(8, 512, 7, 7, 512, 3, 1, 1, FP16), "tensor"),
    "c4b": (ConvShape(16, 128, 56, 56, 256, 3, 2, 1, FP16), "tensor"),
    # the first layer of the chain at 32 images per replica: 3 input channels, the row-gather route
    "stem": (ConvShape(32, 3, 224, 224, 64, 7, 2, 3, FP16), "tensor"),
}

RMSNORM_WORKLOAD = dict(rows=8192, hidden=4096, dtype=BF16, eps=1e-6)


@dataclass(frozen=True)
class ChainOp:
    """One node of the convolution chain.  kind: 'conv' | 'maxpool' | 'add'.  Tensors are named by integer slots."""
    kind: str
    src: int
    dst: int
    shape: ConvShape | None = None
    relu: bool = True
    other: int = -1          # second operand of 'add'; residual slot of a fused 'conv' (-1: none)
    pool: tuple = ()         # (channels, h, w, kernel, stride, pad) of 'maxpool'
    layer: int = -1          # 'conv': index in the order resnet50_chain emits convolutions (names its weights and seed)


def resnet50_chain(batch: int, precision: int = FP16, image: int = 224):
    """Layer list of the ResNet-50-shaped inference chain: 7x7/2 stem (64 ch, pad 3), 3x3/2 max-pool (pad 1), stages of
    [3, 4, 6, 3] bottleneck blocks with widths 64/128/256/512 and expansion 4.  A block is 1x1 -> 3x3 -> 1x1 with folded
    batch-norm (bias) and fused ReLU; the stride-2 of stages 2-4 sits on the 3x3 of the first block; stage entries have
    a 1x1 projection shortcut (stride 2 except in stage 1); the block output is relu(main + shortcut).
    Returns (ops, slot_shapes) where slot_shapes[slot] = (channels, h, w).  53 convolutions."""
    ops, slots = [], {}

    def new_slot(c, h, w):
        slots[len(slots)] = (c, h, w)
        return len(slots) - 1

    cur = new_slot(3, image, image)
    stem = ConvShape(batch, 3, image, image, 64, 7, 2, 3, precision)
    s1 = new_slot(64, stem.out_h, stem.out_w)
    ops.append(ChainOp("conv", cur, s1, stem, True))
    ph = (stem.out_h + 2 - 3) // 2 + 1
    s2 = new_slot(64, ph, ph)
    ops.append(ChainOp("maxpool", s1, s2, pool=(64, stem.out_h, stem.out_w, 3, 2, 1)))
    cur, c_in, h = s2, 64, ph
    for stage, (blocks, width) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512))):
        for blk in range(blocks):
            stride = 2 if (blk == 0 and stage > 0) else 1
            c_out = width * 4
            a = ConvShape(batch, c_in, h, h, width, 1, 1, 0, precision)
            sa = new_slot(width, h, h)
            ops.append(ChainOp("conv", cur, sa, a, True))
            b = ConvShape(batch, width, h, h, width, 3, stride, 1, precision)
            h2 = b.out_h
            sb = new_slot(width, h2, h2)
            ops.append(ChainOp("conv", sa, sb, b, True))
            c = ConvShape(batch, width, h2, h2, c_out, 1, 1, 0, precision)
            sc = new_slot(c_out, h2, h2)
            ops.append(ChainOp("conv", sb, sc, c, False))
            if blk == 0:
                proj = ConvShape(batch, c_in, h, h, c_out, 1, stride, 0, precision)
                sp = new_slot(c_out, h2, h2)
                ops.append(ChainOp("conv", cur, sp, proj, False))
                short = sp
            else:
                short = cur
            so = new_slot(c_out, h2, h2)
            ops.append(ChainOp("add", sc, so, relu=True, other=short))
            cur, c_in, h = so, c_out, h2
    n = 0
    for i, op in enumerate(ops):
        if op.kind == "conv":
            ops[i] = ChainOp(op.kind, op.src, op.dst, op.shape, op.relu, op.other, op.pool, n)
            n += 1
    return ops, slots


def fuse_residuals(ops):
    """The same chain with every 'add' folded into the convolution that produces its first operand: that convolution
    moves behind whatever computes the other operand (the projection shortcut of a stage's first block), takes it as
    its residual, applies the add's ReLU and writes the add's destination slot."""
    out = []
    for op in ops:
        if op.kind != "add":
            out.append(op)
            continue
        idx = next(i for i in range(len(out) - 1, -1, -1) if out[i].kind == "conv" and out[i].dst == op.src)
        conv = out.pop(idx)
        out.append(ChainOp("conv", conv.src, op.dst, conv.shape, op.relu, other=op.other, layer=conv.layer))
    return out


def chain_flops(ops) -> int:
    return sum(op.shape.flops for op in ops if op.kind == "conv")
