"""GPU parity of the tcgen05 implicit-GEMM convolution against the oracle's direct convolution
(fp64 accumulation), through `fml_conv` of the C ABI.

The tensor-core path is taken when the weights are stored tap-major with the output channel
innermost (layout (3, 2, 0, 1) of OIHW), the input is dense NCHW with a row length that is a
multiple of 4, and stride = dilation = group = 1.  Tolerances: 3xTF32 5e-5 (the reduction is
up to 4608 long and the TMEM accumulator truncates), TF32 2e-3 of max|ref|.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT
from oracle import oracle as orc

RNG = np.random.Generator(np.random.PCG64(2718))
PACKED = [3, 2, 0, 1]


def rnd(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def relerr(got, ref):
    ref = ref.astype(np.float64)
    return float(np.abs(got.astype(np.float64) - ref).max() / max(1e-30, np.abs(ref).max()))


CASES = [  # (x shape, w shape, pads) -- VGG blocks, ragged tiles, 1x1, 5x5, few channels, batches
    ((1, 3, 32, 32), (64, 3, 3, 3), (1, 1)),
    ((1, 64, 56, 56), (64, 64, 3, 3), (1, 1)),
    ((2, 64, 28, 28), (128, 64, 3, 3), (1, 1)),
    ((1, 128, 20, 24), (256, 128, 3, 3), (1, 1)),
    ((1, 40, 17, 12), (48, 40, 3, 3), (1, 1)),
    ((1, 96, 16, 16), (32, 96, 1, 1), (0, 0)),
    ((1, 16, 30, 36), (32, 16, 5, 5), (2, 2)),
    ((1, 32, 12, 40), (64, 32, 3, 3), (0, 0)),
    # row lengths that are not a multiple of 4: whole rows loaded as one run of the H*W plane
    ((1, 512, 14, 14), (64, 512, 3, 3), (1, 1)),
    ((2, 48, 18, 10), (32, 48, 3, 3), (1, 1)),
    ((1, 24, 22, 14), (32, 24, 5, 5), (2, 2)),
    # 1x1 kernels over 7 x 7 planes: whole planes fetched with a plain bulk copy
    ((1, 64, 7, 7), (96, 64, 1, 1), (0, 0)),
    ((3, 1152, 7, 7), (192, 1152, 1, 1), (0, 0)),
    # one k block per tile and more pixel tiles than SMs: output tiles wider than 128 channels
    ((6, 24, 56, 56), (144, 24, 1, 1), (0, 0)),    # 160-wide tile, one operand stage, two CTAs per SM
    ((20, 32, 28, 28), (240, 32, 1, 1), (0, 0)),   # 256-wide tile
]


@pytest.mark.parametrize("xs,ws,pads", CASES)
@pytest.mark.parametrize("prec", [cabi.GEMM_3XTF32, cabi.GEMM_TF32])
def test_conv_tensor_cores(xs, ws, pads, prec):
    x, w, b = rnd(*xs), rnd(*ws) * 0.1, rnd(ws[0])
    oh, ow = xs[2] + 2 * pads[0] - ws[2] + 1, xs[3] + 2 * pads[1] - ws[3] + 1
    oshape = (xs[0], ws[0], oh, ow)
    ref = orc.conv(x, w, b, np.empty(oshape, np.float32), list(pads), [1, 1], [1, 1], 1, acc64=True)
    ref = np.maximum(ref, 0)
    out = DT(oshape, np.float32)
    dx, dw = DT.from_numpy(x), DT.from_numpy(w, PACKED)
    assert cabi.conv_uses_tensor_cores(dx, dw, out, list(pads), prec)
    assert not cabi.conv_uses_tensor_cores(dx, DT.from_numpy(w), out, list(pads), prec)  # OIHW weights: CUDA cores
    cabi.conv(dx, dw, DT.from_numpy(b), out, list(pads), [1, 1], [1, 1], 1,
              act=cabi.ACT_RELU, precision=prec)
    cabi.check_device()
    assert relerr(out.numpy(), ref) <= (5e-5 if prec == cabi.GEMM_3XTF32 else 2e-3)


@pytest.mark.parametrize("xs,ws,pads,gate_shape", [
    ((2, 96, 16, 16), (32, 96, 1, 1), (0, 0), (2, 96, 1, 1)),      # box patches
    ((3, 1152, 7, 7), (192, 1152, 1, 1), (0, 0), (3, 1152, 1, 1)), # whole planes, split over the channel blocks
    ((2, 480, 14, 14), (112, 480, 1, 1), (0, 0), (2, 480, 1, 1)),  # flat rows
    ((1, 40, 17, 12), (48, 40, 3, 3), (1, 1), (1, 40, 1, 1)),      # channel tail (40 = 32 + 8), 3 x 3 with padding
    ((2, 64, 28, 28), (128, 64, 3, 3), (1, 1), (1, 64, 1, 1)),     # one gate for every image
])
@pytest.mark.parametrize("packed", [True, False])
def test_conv_with_scaled_input_equals_mul_then_conv(xs, ws, pads, gate_shape, packed):
    """fml_conv_scaled rounds x * gate to fp32 before the convolution, like MulCommon followed by
    Conv: the same kernel fed the pre-multiplied tensor gives the same bits (tensor-core path with
    packed weights, general implicit GEMM with OIHW weights); and the oracle's Mul -> Conv (fp64
    accumulation) is matched within the 3xTF32 tolerance."""
    x, w, b, gate = rnd(*xs), rnd(*ws) * 0.1, rnd(ws[0]), rnd(*gate_shape)
    oh, ow = xs[2] + 2 * pads[0] - ws[2] + 1, xs[3] + 2 * pads[1] - ws[3] + 1
    oshape = (xs[0], ws[0], oh, ow)
    prod = orc.binary("Mul", x, gate, np.empty(xs, np.float32))
    ref = orc.conv(prod, w, b, np.empty(oshape, np.float32), list(pads), [1, 1], [1, 1], 1, acc64=True)
    dw = DT.from_numpy(w, PACKED if packed else None)
    fused, plain = DT(oshape, np.float32), DT(oshape, np.float32)
    cabi.conv_scaled(DT.from_numpy(x), DT.from_numpy(gate), dw, DT.from_numpy(b), fused, list(pads), [1, 1], [1, 1],
                     act=cabi.ACT_SILU)
    cabi.check_device()
    if packed:
        cabi.conv(DT.from_numpy(prod), dw, DT.from_numpy(b), plain, list(pads), [1, 1], [1, 1], 1, act=cabi.ACT_SILU)
        assert np.array_equal(fused.numpy(), plain.numpy())
    pre = ref.astype(np.float64)
    ref_act = pre / (1.0 + np.exp(-pre))
    assert relerr(fused.numpy(), ref_act) <= 5e-5


def test_conv_paths_agree_and_repeat():
    """Same operands through the tensor-core path (packed weights) and the CUDA-core path (OIHW
    weights): equal within the 3xTF32 tolerance; the tensor-core result is bit-stable."""
    x, w, b = rnd(1, 64, 28, 28), rnd(128, 64, 3, 3) * 0.1, rnd(128)
    outs = []
    for layout in (PACKED, PACKED, None):
        out = DT((1, 128, 28, 28), np.float32)
        cabi.conv(DT.from_numpy(x), DT.from_numpy(w, layout), DT.from_numpy(b), out, [1, 1], [1, 1], [1, 1], 1)
        outs.append(out.numpy())
    cabi.check_device()
    assert np.array_equal(outs[0], outs[1])
    assert relerr(outs[0], outs[2]) <= 2e-5


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("act", [cabi.ACT_SIGMOID, cabi.ACT_SILU])
def test_single_pixel_convolution_is_a_skinny_gemm(packed, act):
    """Squeeze-and-excite convolutions (1 x 1 images): the product [N, IC] x [IC, OC] with bias and
    gate in the epilogue, on the weight-streaming kernel."""
    x, w, b = rnd(4, 1152, 1, 1), rnd(48, 1152, 1, 1) * 0.05, rnd(48)
    t = orc.conv(x, w, b, np.empty((4, 48, 1, 1), np.float32), [0, 0], [1, 1], [1, 1], 1, acc64=True).astype(np.float64)
    sig = 1.0 / (1.0 + np.exp(-t))
    ref = sig if act == cabi.ACT_SIGMOID else t * sig
    out = DT((4, 48, 1, 1), np.float32)
    cabi.conv(DT.from_numpy(x), DT.from_numpy(w, PACKED if packed else None), DT.from_numpy(b), out, [0, 0], [1, 1],
              [1, 1], 1, act=act)
    cabi.check_device()
    assert relerr(out.numpy(), ref) <= 1e-5


def test_conv_shapes_left_to_the_cuda_cores():
    w = DT.from_numpy(rnd(32, 16, 3, 3), PACKED)
    # 7 x 7 planes do not start on 16-byte steps; 50 columns neither fit a box nor one tile
    for hw in ((7, 7), (9, 50)):  # (3 x 3 kernels: the 7 x 7 case needs a halo, unlike 1 x 1 kernels)
        x, y = DT.from_numpy(rnd(1, 16, *hw)), DT((1, 32, *hw), np.float32)
        assert not cabi.conv_uses_tensor_cores(x, w, y, [1, 1])
        cabi.conv(x, w, None, y, [1, 1], [1, 1], [1, 1], 1)
    cabi.check_device()


@pytest.mark.parametrize("xs,oc", [((8, 768, 128), 384), ((2, 96, 50), 40), ((1, 64, 12, 20), 32)])
def test_pointwise_convolution_with_row_major_weights_is_a_gemm(xs, oc):
    """1 x 1 kernels over dense planes with OIHW weights (the 1-D pointwise convolution of
    ConvBERT's separable convolution): W [OC, IC] x X [IC, pixels] per image through fml_gemm."""
    nd = len(xs) - 2
    x, w, b = rnd(*xs), rnd(oc, xs[1], *([1] * nd)) * 0.05, rnd(oc)
    oshape = (xs[0], oc, *xs[2:])
    ref = orc.conv(x, w, b, np.empty(oshape, np.float32), [0] * nd, [1] * nd, [1] * nd, 1, acc64=True)
    out = DT(oshape, np.float32)
    cabi.conv(DT.from_numpy(x), DT.from_numpy(w), DT.from_numpy(b), out, [0] * nd, [1] * nd, [1] * nd, 1)
    cabi.check_device()
    assert relerr(out.numpy(), ref) <= 2e-5
