"""ConvInteger / QLinearConv parity: int32 accumulators and requantised bytes equal."""
import json
import os

import numpy as np
import pytest
import torch

import cases
import oracle as orc
import ovk_b200
from gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
# last kernel of the filters x patches route: the product itself, or the pass that puts several images' results back
GEMM_ROUTE = ("mmi_tc", "conv_unbatch")


@pytest.mark.parametrize("c_in,c_out,h,w,stride,dil,pads,xs,ws", [
    (64, 32, 20, 20, 1, 1, (1, 1, 1, 1), False, False),
    (32, 48, 18, 22, 2, 2, (2, 0, 1, 3), True, True),
    (32, 16, 15, 15, 1, 1, (1, 1, 1, 1), False, True),
])
def test_reference_geometries(c_in, c_out, h, w, stride, dil, pads, xs, ws):
    """crates/onnx-vulkan-core/tests/conv_integer_im2col.rs:185-247."""
    x = cases.lcg_bytes_fast(c_in * h * w, 11).reshape(1, c_in, h, w)
    wt = cases.lcg_bytes_fast(c_out * c_in * 9, 5).reshape(c_out, c_in, 3, 3)
    x = x.view(np.int8) if xs else x
    wt = wt.view(np.int8) if ws else wt
    x_zp = -5 if xs else 129
    wq = ctx().qconv_prepack(dev(wt))
    got = ctx().conv_integer(wq, dev(x), x_zp, 7, pads=pads, strides=(stride, stride), dilations=(dil, dil))
    want = orc.conv_integer(x, wt, x_zp, 7, strides=(stride, stride), dilations=(dil, dil), pads=pads)
    assert np.array_equal(host(got), want)


def test_literal_vectors():
    """crates/onnx-vulkan-core/tests/qlinear.rs:106-236."""
    v = json.load(open(os.path.join(GOLDEN, "qlinear_literal_vectors.json")))
    for name, xs, ws in (("conv_per_channel", (1, 1, 3, 3), (2, 1, 2, 2)),
                         ("conv_per_tensor", (1, 1, 3, 3), (2, 1, 2, 2)),
                         ("conv_no_bias", (1, 1, 2, 2), (1, 1, 2, 2))):
        c = v[name]
        x = np.array(c["x"], dtype=np.uint8).reshape(xs)
        w = np.array(c["w"], dtype=np.int8).reshape(ws)
        w_scale = np.atleast_1d(np.array(c["w_scale"], dtype=np.float32))
        bias = np.array(c["bias"], dtype=np.int32) if "bias" in c else None
        want = orc.qlinear_conv(x, c["x_scale"], c["x_zp"], w, w_scale, 0, c["y_scale"], c["y_zp"], bias=bias)
        ratio = orc.requantize_ratio(c["x_scale"], w_scale, c["y_scale"])
        wq = ctx().qconv_prepack(dev(w))
        got = ctx().qlinear_conv(wq, dev(x), c["x_zp"], 0, ratio, None if bias is None else dev(bias), c["y_zp"])
        assert np.array_equal(host(got), want), name


def _resnet_block(batch, seed_cfg=4):
    x = cases.rng_for(seed_cfg, 0).integers(0, 256, size=(batch, 64, 56, 56), dtype=np.uint8)
    w = cases.rng_for(seed_cfg, 1).integers(-127, 128, size=(64, 64, 3, 3), dtype=np.int8)
    w_scale = cases.rng_for(seed_cfg, 2).uniform(0.001, 0.01, size=64).astype(np.float32)
    bias = cases.rng_for(seed_cfg, 3).integers(-1000, 1001, size=64, dtype=np.int32)
    return x, w, w_scale, bias


def test_resnet_block_small_batch_every_output():
    """Config 4 at batch 2: u8 NCHW 64ch 56x56, int8 3x3 per-channel weights,
    int32 bias, pad 1; uint8 outputs and int32 accumulators equal."""
    x, w, w_scale, bias = _resnet_block(2)
    wq = ctx().qconv_prepack(dev(w))
    acc = ctx().conv_integer(wq, dev(x), 128, 0, pads=(1, 1, 1, 1))
    want_acc = orc.conv_integer(x, w, 128, 0, pads=(1, 1, 1, 1))
    assert np.array_equal(host(acc), want_acc)
    ratio = orc.requantize_ratio(0.02, w_scale, 0.05)
    got = ctx().qlinear_conv(wq, dev(x), 128, 0, ratio, dev(bias), 128, pads=(1, 1, 1, 1))
    want = orc.requantize(want_acc, 56 * 56, ratio, 128, bias)
    assert np.array_equal(host(got), want)


def test_resnet_block_full_batch_sampled_images_and_batch_independence():
    """Config 4 at batch 64: images 0, 31 and 63 against the oracle, and the
    batched result equal to the same images run one at a time."""
    x, w, w_scale, bias = _resnet_block(64)
    ratio = orc.requantize_ratio(0.02, w_scale, 0.05)
    wq = ctx().qconv_prepack(dev(w))
    xd = dev(x)
    got = host(ctx().qlinear_conv(wq, xd, 128, 0, ratio, dev(bias), 128, pads=(1, 1, 1, 1)))
    for i in (0, 31, 63):
        want = orc.qlinear_conv(x[i:i + 1], 0.02, 128, w, w_scale, 0, 0.05, 128, bias=bias, pads=(1, 1, 1, 1))
        assert np.array_equal(got[i:i + 1], want), i
        single = host(ctx().qlinear_conv(wq, xd[i:i + 1].contiguous(), 128, 0, ratio, dev(bias), 128, pads=(1, 1, 1, 1)))
        assert np.array_equal(single, got[i:i + 1])


@pytest.mark.parametrize("group,c_in,c_out", [(4, 16, 8), (16, 16, 16)])
def test_grouped_and_depthwise(group, c_in, c_out):
    """src/shaders/conv_integer.rs:73-110: the direct form is the only one groups can use."""
    x = cases.lcg_bytes_fast(2 * c_in * 9 * 11, 3).reshape(2, c_in, 9, 11)
    w = cases.lcg_bytes_fast(c_out * (c_in // group) * 9, 4).reshape(c_out, c_in // group, 3, 3).view(np.int8)
    wq = ctx().qconv_prepack(dev(w), group=group)
    got = ctx().conv_integer(wq, dev(x), 120, 3, pads=(1, 1, 1, 1), strides=(2, 1))
    want = orc.conv_integer(x, w, 120, 3, pads=(1, 1, 1, 1), strides=(2, 1), group=group)
    assert np.array_equal(host(got), want)


@pytest.mark.parametrize("c,h,w,kh,kw,strides,dil,pads,batch,w_zp", [
    (144, 28, 31, 3, 3, (2, 2), 1, (1, 1, 1, 1), 3, 0),
    (1024, 1, 1000, 1, 9, (1, 1), 1, (0, 4, 0, 4), 1, 0),   # the encoder's depthwise layer
    (32, 19, 17, 5, 3, (1, 2), 2, (4, 2, 4, 2), 2, 9),
])
def test_depthwise_convolutions_have_a_kernel_of_their_own(c, h, w, kh, kw, strides, dil, pads, batch, w_zp):
    """One filter per channel: a block owns one plane, its filter in shared memory.  All three stores against the
    CPU port (strides, dilation, uneven pads, an asymmetric weight)."""
    rng = np.random.default_rng(c + h + kw)
    x = rng.integers(0, 256, size=(batch, c, h, w), dtype=np.uint8)
    wt = rng.integers(-127, 128, size=(c, 1, kh, kw), dtype=np.int8)
    wq = ctx().qconv_prepack(dev(wt), group=c)
    kwargs = dict(pads=pads, strides=strides, dilations=(dil, dil))
    got = ctx().conv_integer(wq, dev(x), 131, w_zp, **kwargs)
    assert ctx().last_kernel == "conv_depthwise"
    want = orc.conv_integer(x, wt, 131, w_zp, group=c, **kwargs)
    assert np.array_equal(host(got), want)
    scale = rng.uniform(1e-4, 1e-3, c).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, c).astype(np.float32)
    slot = torch.zeros(2, dtype=torch.int32, device="cuda")
    f = ctx().conv_integer_scale_bias(wq, dev(x), 131, w_zp, dev(scale), dev(bias), relu=True, range_slot=slot, **kwargs)
    want_f = _fused_oracle(want, scale, bias, relu=True)
    assert np.array_equal(host(f).view(np.uint32), want_f.view(np.uint32))
    lo_hi = host(slot).view(np.float32)
    assert lo_hi[0] == max(-want_f.min(), 0.0) and lo_hi[1] == max(want_f.max(), 0.0)
    if w_zp == 0:
        ratio = orc.requantize_ratio(0.02, rng.uniform(0.001, 0.01, size=c).astype(np.float32), 0.05)
        ibias = rng.integers(-1000, 1001, size=c, dtype=np.int32)
        q = ctx().qlinear_conv(wq, dev(x), 131, 0, ratio, dev(ibias), 3, **kwargs)
        assert np.array_equal(host(q), orc.requantize(want, want.shape[2] * want.shape[3], ratio, 3, bias=ibias))


def test_signed_output_and_one_dimensional_conv():
    x = cases.lcg_bytes_fast(3 * 8 * 40, 6).reshape(3, 8, 40, 1).view(np.int8)
    w = cases.lcg_bytes_fast(12 * 8 * 5, 8).reshape(12, 8, 5, 1).view(np.int8)
    w_scale = np.linspace(0.002, 0.02, 12).astype(np.float32)
    ratio = orc.requantize_ratio(0.05, w_scale, 0.4)
    wq = ctx().qconv_prepack(dev(w))
    got = ctx().qlinear_conv(wq, dev(x), -3, 0, ratio, None, -11, y_signed=True, pads=(2, 0, 2, 0))
    want = orc.qlinear_conv(x, 0.05, -3, w, w_scale, 0, 0.4, -11, out_signed=True, pads=(2, 0, 2, 0))
    assert np.array_equal(host(got), want)


def test_requantize_pass_matches():
    """src/shaders/qlinear.rs:28-63 on its own, ragged length."""
    acc = cases.rng_for(4, 9).integers(-2 ** 20, 2 ** 20, size=(3, 5, 7), dtype=np.int32)
    ratio = np.linspace(1e-4, 3e-3, 5).astype(np.float32)
    bias = np.arange(-2, 3, dtype=np.int32) * 1000
    got = ctx().requantize(dev(acc), 7, dev(ratio), 17, bias=dev(bias))
    assert np.array_equal(host(got), orc.requantize(acc, 7, ratio, 17, bias))


def test_resnet_block_takes_the_tensor_core_kernel():
    """Which kernel ran (the role of pipeline_keys in
    crates/onnx-vulkan-core/tests/conv_integer_im2col.rs:163-178): group 1,
    symmetric weights, strides up to 4 -> the tcgen05 convolution kernel; an asymmetric weight or a longer
    stride -> filters x patches on the tcgen05 MatMulInteger kernels."""
    x, w, w_scale, bias = _resnet_block(2)
    wq = ctx().qconv_prepack(dev(w))
    ctx().conv_integer(wq, dev(x), 128, 0, pads=(1, 1, 1, 1))
    assert ctx().last_kernel.startswith("qconv_tc")
    ctx().conv_integer(wq, dev(x), 128, 5, pads=(1, 1, 1, 1))
    assert ctx().last_kernel.startswith(GEMM_ROUTE)  # an asymmetric weight: filters x patches, with the patches' sums
    ctx().conv_integer(wq, dev(x), 128, 0, pads=(1, 1, 1, 1), strides=(2, 2))
    assert ctx().last_kernel.startswith("qconv_tc")
    ctx().conv_integer(wq, dev(x), 128, 0, pads=(1, 1, 1, 1), strides=(5, 5))
    assert ctx().last_kernel.startswith(GEMM_ROUTE)  # two images: filters x patches on the MatMulInteger kernels
    x9, _, _, _ = _resnet_block(9)
    ctx().conv_integer(wq, dev(x9), 128, 0, pads=(1, 1, 1, 1), strides=(5, 5))
    assert ctx().last_kernel.startswith(GEMM_ROUTE)  # any batch, where the convolution kernel does not take the geometry


@pytest.mark.parametrize("c_in,c_out,h,w,k,dil,pads,xs", [
    (32, 40, 20, 20, 3, 1, (1, 1, 1, 1), False),
    (64, 48, 24, 24, 1, 1, (0, 0, 0, 0), False),
    (128, 64, 14, 18, 3, 2, (2, 2, 2, 2), True),
    (256, 32, 12, 12, 3, 1, (1, 0, 2, 1), False),
    (64, 100, 9, 33, 3, 1, (1, 1, 1, 1), True),
    (32, 24, 11, 13, 5, 1, (2, 2, 2, 2), False),
    (64, 128, 30, 30, 3, 1, (1, 1, 1, 1), False),
    (64, 256, 30, 30, 1, 1, (0, 0, 0, 0), False),
    (32, 200, 40, 36, 1, 1, (0, 0, 0, 0), True),
    (32, 32, 5, 320, 3, 1, (1, 1, 1, 1), False),
    (256, 64, 14, 14, 1, 1, (0, 0, 0, 0), False),
    (384, 64, 28, 28, 1, 1, (0, 0, 0, 0), True),
    (128, 64, 14, 14, 3, 1, (1, 1, 1, 1), False),
    (64, 32, 8, 7, 3, 1, (1, 2, 1, 0), True),
])
def test_tensor_core_geometries(c_in, c_out, h, w, k, dil, pads, xs):
    """Channel counts 32/64/128/256 (one to two K slices per tap), dilation,
    uneven pads, pointwise and 5x5 filters, signed x, C_out off the tile size,
    and 128 / 200 / 256 output channels: four, two and two accumulators in
    flight, so the epilogue warps of a lane quarter split into four or two tile
    groups, over several tiles per CTA.  The last rows are for the layout pass
    in front of the kernel: rows wider than 256 pixels, an unpadded plane whose
    rows are no whole words (turned as one row), three channel groups, padded
    planes with rows of 14 and of 7 bytes (taken two and four rows at a time)."""
    x = cases.lcg_bytes_fast(3 * c_in * h * w, 21).reshape(3, c_in, h, w)
    wt = cases.lcg_bytes_fast(c_out * c_in * k * k, 23).reshape(c_out, c_in, k, k).view(np.int8)
    x = x.view(np.int8) if xs else x
    x_zp = -9 if xs else 131
    wq = ctx().qconv_prepack(dev(wt))
    got = ctx().conv_integer(wq, dev(x), x_zp, 0, pads=pads, dilations=(dil, dil))
    assert ctx().last_kernel.startswith("qconv_tc"), ctx().last_kernel
    want = orc.conv_integer(x, wt, x_zp, 0, dilations=(dil, dil), pads=pads)
    assert np.array_equal(host(got), want)


@pytest.mark.parametrize("c_in,c_out,h,w,k,batch", [(128, 320, 30, 30, 3, 5), (256, 288, 30, 31, 3, 5), (128, 128, 28, 28, 3, 6),
                                                    (256, 600, 30, 30, 1, 6), (512, 96, 21, 21, 3, 8)])
def test_filter_banks_larger_than_shared_memory_take_several_launches(c_in, c_out, h, w, k, batch):
    """A bank that does not fit in shared memory beside the pixel stages (3 x 3 over 128 and more channels, the
    deeper stages of a ResNet) is taken in slices of as many filters as fit, multiples of 32 up to 256: every
    slice addresses its own filters, sums, constants and output channels - equal slices as rows of one grid
    (320 = 2 x 160, 96 = 3 x 32), a bank with a narrower last slice as one launch per slice (288, 600).  int32
    accumulators, the fused f32 store with per-channel constants and the requantised bytes (NCHW, and
    channels-last where C_out allows) equal the CPU port."""
    rng = np.random.default_rng(c_in * 7 + c_out)
    x = rng.integers(0, 256, size=(batch, c_in, h, w), dtype=np.uint8)
    wt = rng.integers(-127, 128, size=(c_out, c_in, k, k), dtype=np.int8)
    pads = (k // 2,) * 4
    wq = ctx().qconv_prepack(dev(wt))
    before = ctx().launches
    got = ctx().conv_integer(wq, dev(x), 131, 0, pads=pads)
    assert ctx().last_kernel.startswith("qconv_tc"), ctx().last_kernel
    launches = ctx().launches - before - 1  # the layout pass
    if c_out in (288, 600):
        assert launches >= 2, launches
    want = orc.conv_integer(x, wt, 131, 0, pads=pads)
    assert np.array_equal(host(got), want)
    scale = rng.uniform(1e-5, 1e-4, c_out).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, c_out).astype(np.float32)
    f = ctx().conv_integer_scale_bias(wq, dev(x), 131, 0, dev(scale), dev(bias), relu=True, pads=pads)
    assert np.array_equal(host(f).view(np.uint32), _fused_oracle(want, scale, bias, relu=True).view(np.uint32))
    w_scale = rng.uniform(0.001, 0.01, size=c_out).astype(np.float32)
    ibias = rng.integers(-1000, 1001, size=c_out, dtype=np.int32)
    ratio = orc.requantize_ratio(0.02, w_scale, 0.9)
    want_q = orc.requantize(want, h * w, ratio, 3, bias=ibias)
    q = ctx().qlinear_conv(wq, dev(x), 131, 0, ratio, dev(ibias), 3, pads=pads)
    assert np.array_equal(host(q), want_q)
    if c_out % 16 == 0:
        frame = (1, 2, 0, 1)
        out = torch.full((batch, h + frame[0] + frame[2], w + frame[1] + frame[3], c_out), 77, dtype=torch.uint8, device="cuda")
        ctx().qlinear_conv_channels_last(wq, dev(x), 131, 0, ratio, dev(ibias), 3, out, frame, pads=pads, x_nchw=True)
        inner = host(out)[:, frame[0]:frame[0] + h, frame[1]:frame[1] + w, :]
        assert np.array_equal(np.moveaxis(inner, -1, 1), want_q)
        o = host(out)
        assert (o[:, :frame[0]] == 77).all() and (o[:, :, :frame[1]] == 77).all() and (o[:, :, frame[1] + w:] == 77).all()


@pytest.mark.parametrize("c_in,c_out,h,w,k,strides,pads", [(64, 64, 56, 56, 3, (2, 2), (1, 1, 1, 1)), (128, 96, 29, 31, 3, (2, 1), (1, 0, 1, 2)),
                                                           (256, 320, 28, 28, 1, (2, 2), (0, 0, 0, 0)), (32, 48, 25, 40, 5, (3, 2), (2, 2, 2, 2)),
                                                           (64, 64, 30, 30, 3, (4, 4), (0, 0, 0, 0))])
def test_strided_convolutions_on_the_tensor_core_kernel(c_in, c_out, h, w, k, strides, pads):
    """Strides up to 4 (the stage transitions and downsampling layers of a ResNet): the tensor-core kernel forms the
    products at every position of the padded grid and stores those on the stride lattice.  int32 and requantised
    bytes against the CPU port, odd sizes, different strides along H and W, several launches of a large bank."""
    rng = np.random.default_rng(c_in + c_out + k)
    x = rng.integers(0, 256, size=(3, c_in, h, w), dtype=np.uint8)
    wt = rng.integers(-127, 128, size=(c_out, c_in, k, k), dtype=np.int8)
    wq = ctx().qconv_prepack(dev(wt))
    got = ctx().conv_integer(wq, dev(x), 129, 0, pads=pads, strides=strides)
    assert ctx().last_kernel.startswith(("qconv_tc",) + GEMM_ROUTE), ctx().last_kernel
    want = orc.conv_integer(x, wt, 129, 0, strides=strides, pads=pads)
    assert host(got).shape == want.shape and np.array_equal(host(got), want)
    ratio = orc.requantize_ratio(0.02, rng.uniform(0.001, 0.01, size=c_out).astype(np.float32), 0.9)
    ibias = rng.integers(-1000, 1001, size=c_out, dtype=np.int32)
    q = ctx().qlinear_conv(wq, dev(x), 129, 0, ratio, dev(ibias), 3, pads=pads, strides=strides)
    assert np.array_equal(host(q), orc.requantize(want, want.shape[2] * want.shape[3], ratio, 3, bias=ibias))


@pytest.mark.parametrize("c_in,c_out,hw,k,batch", [(256, 256, 14, 3, 1), (512, 512, 7, 3, 1), (2048, 512, 7, 1, 8), (64, 64, 5, 3, 1),
                                                   (32, 32, 1, 1, 1), (128, 40, 3, 3, 2)])
def test_small_images_stay_on_the_tensor_core_kernel(c_in, c_out, hw, k, batch):
    """The last stages of a ResNet at batch 1 (14 x 14 and 7 x 7 planes: one or two pixel tiles, banks of up to
    2.4 MB in launches of 32-256 filters), down to a single pixel: int32 and requantised bytes against the CPU port."""
    rng = np.random.default_rng(c_in + c_out + hw)
    x = rng.integers(0, 256, size=(batch, c_in, hw, hw), dtype=np.uint8)
    wt = rng.integers(-127, 128, size=(c_out, c_in, k, k), dtype=np.int8)
    pads = (k // 2,) * 4
    wq = ctx().qconv_prepack(dev(wt))
    got = ctx().conv_integer(wq, dev(x), 131, 0, pads=pads)
    assert ctx().last_kernel.startswith(("qconv_tc",) + GEMM_ROUTE), ctx().last_kernel
    want = orc.conv_integer(x, wt, 131, 0, pads=pads)
    assert np.array_equal(host(got), want)
    ratio = orc.requantize_ratio(0.02, rng.uniform(0.001, 0.01, size=c_out).astype(np.float32), 0.9)
    ibias = rng.integers(-1000, 1001, size=c_out, dtype=np.int32)
    q = ctx().qlinear_conv(wq, dev(x), 131, 0, ratio, dev(ibias), 3, pads=pads)
    assert np.array_equal(host(q), orc.requantize(want, hw * hw, ratio, 3, bias=ibias))


@pytest.mark.parametrize("c_in,c_out,h,w,k,strides,dil,pads,batch", [
    (80, 80, 40, 40, 3, (1, 1), 1, (1, 1, 1, 1), 2),       # a channel count the convolution kernel does not take
    (96, 300, 17, 23, 3, (2, 2), 1, (1, 1, 1, 1), 1),      # strided, odd sizes
    (48, 272, 20, 20, 3, (1, 2), 2, (2, 1, 2, 3), 3),      # dilated, uneven pads, different strides
    (512, 512, 7, 7, 3, (1, 1), 1, (1, 1, 1, 1), 1),       # the last stage of a ResNet, one image
    (16, 64, 30, 30, 5, (3, 3), 1, (2, 2, 2, 2), 4),
    (3, 64, 64, 64, 7, (2, 2), 1, (3, 3, 3, 3), 6),        # the stem: K = 147 padded to 160, any batch
    (20, 48, 19, 19, 1, (1, 1), 1, (0, 0, 0, 0), 2),       # 1 x 1 over a channel count that is no multiple of 16
    (4, 64, 70, 66, 5, (2, 3), 2, (3, 1, 4, 2), 3),        # few long rows (patches built a row of pixels at a time), dilated
])
def test_convolution_as_filters_times_patches(c_in, c_out, h, w, k, strides, dil, pads, batch):
    """Up to four images whose filter bank the convolution kernel cannot hold at once: the patch matrix of an image
    (any stride, dilation and padding; padding positions hold the zero point) times the filter bank on the
    MatMulInteger tensor-core kernels, constants by row.  All three stores against the CPU port."""
    rng = np.random.default_rng(c_in * 3 + c_out + h)
    x = rng.integers(0, 256, size=(batch, c_in, h, w), dtype=np.uint8)
    wt = rng.integers(-127, 128, size=(c_out, c_in, k, k), dtype=np.int8)
    wq = ctx().qconv_prepack(dev(wt))
    kw = dict(pads=pads, strides=strides, dilations=(dil, dil))
    got = ctx().conv_integer(wq, dev(x), 77, 0, **kw)
    assert ctx().last_kernel.startswith(GEMM_ROUTE), ctx().last_kernel
    want = orc.conv_integer(x, wt, 77, 0, **kw)
    assert host(got).shape == want.shape and np.array_equal(host(got), want)
    scale = rng.uniform(1e-5, 1e-4, c_out).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, c_out).astype(np.float32)
    f = ctx().conv_integer_scale_bias(wq, dev(x), 77, 0, dev(scale), dev(bias), relu=True, **kw)
    assert np.array_equal(host(f).view(np.uint32), _fused_oracle(want, scale, bias, relu=True).view(np.uint32))
    ratio = orc.requantize_ratio(0.02, rng.uniform(0.001, 0.01, size=c_out).astype(np.float32), 0.9)
    ibias = rng.integers(-1000, 1001, size=c_out, dtype=np.int32)
    q = ctx().qlinear_conv(wq, dev(x), 77, 0, ratio, dev(ibias), 3, **kw)
    assert np.array_equal(host(q), orc.requantize(want, want.shape[2] * want.shape[3], ratio, 3, bias=ibias))
    # an asymmetric weight (uint8 filters, zero point 119): the same route, the patches' sums from one more pass;
    # where K is padded to 16-byte rows the padding of both operands holds the operand's zero point
    wu = wt.view(np.uint8)
    wqu = ctx().qconv_prepack(dev(wu))
    got_u = ctx().conv_integer(wqu, dev(x), 77, 119, **kw)
    assert ctx().last_kernel.startswith(GEMM_ROUTE), ctx().last_kernel
    want_u = orc.conv_integer(x, wu, 77, 119, **kw)
    assert np.array_equal(host(got_u), want_u)
    q_u = ctx().qlinear_conv(wqu, dev(x), 77, 119, ratio, dev(ibias), 3, **kw)
    assert np.array_equal(host(q_u), orc.requantize(want_u, want.shape[2] * want.shape[3], ratio, 3, bias=ibias))


def _fused_layer(c_in, c_out, hw, k, x_signed, w_signed):
    x = cases.lcg_bytes_fast(c_in * hw[0] * hw[1], 1).reshape(1, c_in, *hw)
    wt = cases.lcg_bytes_fast(c_out * c_in * k * k, 2).reshape(c_out, c_in, k, k)
    rng = np.random.default_rng(c_in * 131 + c_out)
    bias = rng.uniform(-0.5, 0.5, c_out).astype(np.float32)
    scale = (np.abs(rng.uniform(-1e-4, 1e-4, c_out)) + 1e-5).astype(np.float32)
    return (x.view(np.int8) if x_signed else x), (wt.view(np.int8) if w_signed else wt), scale, bias


def _fused_oracle(acc, scale, bias, product=None, relu=False):
    """The four unfused steps on channel-last data: Cast, Mul [by fl(scale*product)], Add, [Relu]."""
    last = np.ascontiguousarray(np.moveaxis(acc, 1, -1))
    out = orc.scale_bias_epilogue(last, scale, int(scale.size > 1), bias, int(bias.size > 1), product=product,
                                  product_step=0, relu=relu)
    return np.ascontiguousarray(np.moveaxis(out, -1, 1))


@pytest.mark.parametrize("c_in,c_out,hw,k,stride,pad,ws,xs,per_channel_scale,kernel", [
    (64, 40, (20, 20), 3, 1, 1, True, False, False, "qconv_tc"),
    (32, 24, (15, 15), 3, 2, 1, False, True, True, "mmi_tc"),
    (64, 48, (24, 24), 1, 1, 0, True, False, False, "qconv_tc"),
    (64, 1, (24, 24), 1, 1, 0, True, False, False, ""),
    (256, 32, (88, 88), 3, 1, 1, True, False, False, "qconv_tc"),
    (4096, 16, (10, 13), 7, 1, 3, False, False, True, "mmi_tc"),
    (24, 20, (15, 15), 3, 1, 1, False, False, True, "mmi_tc"),  # asymmetric weights, K = 216 padded to 224 with the zero points
])
def test_conv_integer_scale_bias_is_bit_identical_to_the_four_nodes(c_in, c_out, hw, k, stride, pad, ws, xs,
                                                                    per_channel_scale, kernel):
    """The layers of crates/onnx-vulkan-core/tests/conv_integer_epilogue.rs:248-372:
    ConvInteger -> Cast -> Mul -> Add fused must answer bit for bit like the
    four nodes, with a scalar scale that is the product of two scales or one
    scale per channel, on both kernels."""
    import torch
    x, wt, scale, bias = _fused_layer(c_in, c_out, hw, k, xs, ws)
    x_zp, w_zp = (-5 if xs else 131), (0 if ws else 121)
    pads, strides = (pad,) * 4, (stride, stride)
    wq = ctx().qconv_prepack(dev(wt))
    if per_channel_scale:
        s_dev, prod, prod_dev = dev(scale), None, None
    else:
        scale, prod = np.array([0.0123], dtype=np.float32), np.array([3.1e-3], dtype=np.float32)
        s_dev, prod_dev = dev(scale), dev(prod)
    got = ctx().conv_integer_scale_bias(wq, dev(x), x_zp, w_zp, s_dev, dev(bias), product=prod_dev, pads=pads,
                                        strides=strides)
    assert ctx().last_kernel.startswith(kernel), ctx().last_kernel
    acc = ctx().conv_integer(wq, dev(x), x_zp, w_zp, pads=pads, strides=strides)
    s_eff = (s_dev * prod_dev if prod_dev is not None else s_dev).reshape(1, -1, 1, 1)
    unfused = acc.to(torch.float32) * s_eff + dev(bias).reshape(1, -1, 1, 1)
    assert torch.equal(got.view(torch.int32), unfused.view(torch.int32))
    want = _fused_oracle(orc.conv_integer(x, wt, x_zp, w_zp, strides=strides, pads=pads), scale, bias, product=prod)
    assert np.array_equal(host(got).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("c_in,c_out,hw,batch,xs", [(256, 320, (1, 1000), 1, False), (128, 272, (20, 50), 2, True),
                                                    (96, 300, (7, 33), 1, False), (1024, 2048, (1, 1000), 1, False)])
def test_pointwise_convolution_takes_the_matmul_kernels(c_in, c_out, hw, batch, xs):
    """A 1 x 1, stride-1, unpadded convolution with more filters than the convolution kernel holds in shared
    memory (the encoder's pointwise layers, 1024 -> 2048 over a thousand frames) is the product filters x image
    on the MatMulInteger tensor-core kernels, the image turned to pixels-major first and the per-channel
    constants applied by row.  int32 accumulators, the fused scale and bias (per channel, with Relu and the range
    fold) and the requantised bytes all equal the CPU port bit for bit; pixel counts that are no multiple of
    four (7 x 33) take the register stores and byte loads."""
    import torch
    big = c_in * c_out * hw[0] * hw[1] > 5e8  # the largest case: sampled channels only on the CPU
    rng = np.random.default_rng(c_in + c_out)
    x = rng.integers(0, 256, size=(batch, c_in, *hw), dtype=np.uint8)
    wt = rng.integers(-127, 128, size=(c_out, c_in, 1, 1), dtype=np.int8)
    x = x.view(np.int8) if xs else x
    x_zp = -5 if xs else 131
    wq = ctx().qconv_prepack(dev(wt))
    got = ctx().conv_integer(wq, dev(x), x_zp, 0)
    assert ctx().last_kernel.startswith(GEMM_ROUTE), ctx().last_kernel
    rows = np.arange(0, c_out, 97) if big else np.arange(c_out)
    want = orc.conv_integer(x, wt[rows], x_zp, 0)
    assert np.array_equal(host(got)[:, rows], want)
    scale = rng.uniform(1e-5, 1e-4, c_out).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, c_out).astype(np.float32)
    for relu in (False, True):
        slot = torch.zeros(2, dtype=torch.int32, device="cuda")
        f = ctx().conv_integer_scale_bias(wq, dev(x), x_zp, 0, dev(scale), dev(bias), relu=relu, range_slot=slot)
        assert ctx().last_kernel.startswith(GEMM_ROUTE), ctx().last_kernel
        want_f = _fused_oracle(want, scale[rows], bias[rows], relu=relu)
        assert np.array_equal(host(f)[:, rows].view(np.uint32), want_f.view(np.uint32))
        if not big:
            lo_hi = host(slot).view(np.float32)
            assert lo_hi[0] == max(-want_f.min(), 0.0) and lo_hi[1] == max(want_f.max(), 0.0)
    w_scale = rng.uniform(0.001, 0.01, size=c_out).astype(np.float32)
    ibias = rng.integers(-1000, 1001, size=c_out, dtype=np.int32)
    ratio = orc.requantize_ratio(0.02, w_scale, 0.9)
    q = ctx().qlinear_conv(wq, dev(x), x_zp, 0, ratio, dev(ibias), 3)
    assert ctx().last_kernel.startswith(GEMM_ROUTE), ctx().last_kernel
    want_q = orc.requantize(want, hw[0] * hw[1], ratio[rows], 3, bias=ibias[rows])
    assert np.array_equal(host(q)[:, rows], want_q)


def test_conv_integer_scale_bias_relu_range_and_batch():
    """Relu and the range slot of the DynamicQuantizeLinear that follows, batch 3, on both kernels."""
    import torch
    x = cases.lcg_bytes_fast(3 * 64 * 18 * 18, 7).reshape(3, 64, 18, 18)
    wt = cases.lcg_bytes_fast(40 * 64 * 9, 9).reshape(40, 64, 3, 3).view(np.int8)
    rng = np.random.default_rng(5)
    scale = rng.uniform(1e-5, 1e-4, 40).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, 40).astype(np.float32)
    wq = ctx().qconv_prepack(dev(wt))
    for strides, kernel in (((1, 1), "qconv_tc"), ((2, 2), "qconv_tc"), ((5, 5), GEMM_ROUTE)):
        for relu in (False, True):
            slot = torch.zeros(2, dtype=torch.int32, device="cuda")
            got = ctx().conv_integer_scale_bias(wq, dev(x), 128, 0, dev(scale), dev(bias), relu=relu, range_slot=slot,
                                                pads=(1, 1, 1, 1), strides=strides)
            assert ctx().last_kernel.startswith(kernel), ctx().last_kernel
            want = _fused_oracle(orc.conv_integer(x, wt, 128, 0, pads=(1, 1, 1, 1), strides=strides), scale, bias,
                                 relu=relu)
            assert np.array_equal(host(got).view(np.uint32), want.view(np.uint32))
            lo_hi = host(slot).view(np.float32)
            assert lo_hi[0] == max(-want.min(), 0.0) and lo_hi[1] == max(want.max(), 0.0)


def test_conv_integer_scale_bias_refusals():
    wt = np.zeros((8, 16, 3, 3), dtype=np.int8)
    wq = ctx().qconv_prepack(dev(wt))
    x = dev(np.zeros((1, 16, 6, 6), dtype=np.uint8))
    ok = dev(np.ones(8, dtype=np.float32))
    with pytest.raises(ovk_b200.OvkError) as err:
        ctx().conv_integer_scale_bias(wq, x, 0, 0, dev(np.ones(6, dtype=np.float32)), ok)
    assert "step" in str(err.value)


# ------------------------------------------------------------------ channels-last chain

def _nhwc(a):
    return np.ascontiguousarray(np.moveaxis(a, 1, -1))


def test_layout_converters_round_trip():
    x = cases.lcg_bytes_fast(3 * 64 * 10 * 12, 9).reshape(3, 64, 10, 12)
    pads = (1, 2, 3, 0)
    xp = ctx().to_padded_nhwc(dev(x), pads, 131)
    got = host(xp)
    assert got.shape == (3, 14, 14, 64)
    want = np.full(got.shape, 131, dtype=np.uint8)
    want[:, 1:11, 2:14, :] = _nhwc(x)
    assert np.array_equal(got, want)
    assert np.array_equal(host(ctx().from_padded_nhwc(xp, pads)), x)
    odd = cases.lcg_bytes_fast(2 * 8 * 5 * 7, 4).reshape(2, 8, 5, 7)  # a width that is no multiple of 4: the general pass
    xo = ctx().to_padded_nhwc(dev(odd), (1, 1, 1, 1), 7)
    assert np.array_equal(host(ctx().from_padded_nhwc(xo, (1, 1, 1, 1))), odd)


def test_two_layer_chain_stays_channels_last():
    """Config 4's block twice in a row, batch 3: NCHW -> [layer 1] -> padded NHWC -> [layer 2] -> padded NHWC
    -> NCHW.  Layer 1 pays the layout pass once; layer 2 reads what layer 1 stored - straight into the
    interior of a buffer whose frame already holds layer 2's x_zero_point - and launches ONE kernel.  Bytes
    equal the operator applied twice (the CPU port), and nothing outside the interior is written."""
    x, w, w_scale, bias = _resnet_block(3)
    w2 = cases.rng_for(4, 11).integers(-127, 128, size=(64, 64, 3, 3), dtype=np.int8)
    ratio1 = orc.requantize_ratio(0.02, w_scale, 0.05)
    ratio2 = orc.requantize_ratio(0.05, w_scale[::-1].copy(), 0.04)
    wq1, wq2 = ctx().qconv_prepack(dev(w)), ctx().qconv_prepack(dev(w2))
    frame = (1, 1, 1, 1)
    mid = torch.full((3, 58, 58, 64), 128, dtype=torch.uint8, device="cuda")  # frame = layer 2's x_zp
    end = torch.full((3, 58, 57, 64), 9, dtype=torch.uint8, device="cuda")   # an uneven frame (2, 0, 0, 1), value 9
    ctx().qlinear_conv_channels_last(wq1, dev(x), 128, 0, ratio1, dev(bias), 128, mid, frame, pads=frame, x_nchw=True)
    assert ctx().last_kernel == "qconv_tc_halo"
    before = ctx().launches
    ctx().qlinear_conv_channels_last(wq2, mid, 128, 0, ratio2, None, 100, end, (2, 0, 0, 1), pads=frame)
    assert ctx().launches - before == 1 and ctx().last_kernel == "qconv_tc_halo"
    y1 = orc.qlinear_conv(x, 0.02, 128, w, w_scale, 0, 0.05, 128, bias=bias, pads=frame)
    y2 = orc.qlinear_conv(y1, 0.05, 128, w2, w_scale[::-1].copy(), 0, 0.04, 100, pads=frame)
    got_mid, got_end = host(mid), host(end)
    assert np.array_equal(got_mid[:, 1:57, 1:57, :], _nhwc(y1))
    frame_mask = np.ones(got_mid.shape, dtype=bool)
    frame_mask[:, 1:57, 1:57, :] = False
    assert (got_mid[frame_mask] == 128).all()
    assert np.array_equal(got_end[:, 2:58, 0:56, :], _nhwc(y2))
    end_mask = np.ones(got_end.shape, dtype=bool)
    end_mask[:, 2:58, 0:56, :] = False
    assert (got_end[end_mask] == 9).all()
    # the same second layer back into the operator's layout
    nchw = torch.empty((3, 64, 56, 56), dtype=torch.uint8, device="cuda")
    ctx().qlinear_conv_channels_last(wq2, mid, 128, 0, ratio2, None, 100, nchw, None, pads=frame)
    assert np.array_equal(host(nchw), y2)
    assert np.array_equal(host(ctx().from_padded_nhwc(end[:, 2:58, 0:56, :].contiguous(), (0, 0, 0, 0))), y2)


def test_channels_last_signed_dilated_and_refusals():
    import ovk_b200
    x = cases.lcg_bytes_fast(2 * 32 * 18 * 22, 6).reshape(2, 32, 18, 22).view(np.int8)
    w = cases.lcg_bytes_fast(48 * 32 * 9, 8).reshape(48, 32, 3, 3).view(np.int8)
    w_scale = np.linspace(0.002, 0.02, 48).astype(np.float32)
    ratio = orc.requantize_ratio(0.05, w_scale, 0.4)
    wq = ctx().qconv_prepack(dev(w))
    pads = (2, 0, 1, 3)
    xp = ctx().to_padded_nhwc(dev(x), pads, -5)
    want = orc.qlinear_conv(x, 0.05, -5, w, w_scale, 0, 0.4, -11, out_signed=True, pads=pads, dilations=(2, 2))
    out = torch.zeros((2, want.shape[2] + 2, want.shape[3] + 2, 48), dtype=torch.int8, device="cuda")
    ctx().qlinear_conv_channels_last(wq, xp, -5, 0, ratio, None, -11, out, (1, 1, 1, 1), y_signed=True, pads=pads,
                                     dilations=(2, 2))
    assert np.array_equal(host(out)[:, 1:-1, 1:-1, :], _nhwc(want))
    with pytest.raises(ovk_b200.OvkError) as e:  # stride 5: the direct kernel's geometry, NCHW only
        ctx().qlinear_conv_channels_last(wq, xp, -5, 0, ratio, None, -11, out, (1, 1, 1, 1), y_signed=True, pads=pads,
                                         strides=(5, 5))
    assert e.value.status == ovk_b200.UNSUPPORTED
    w40 = ctx().qconv_prepack(dev(w[:40].copy()))
    with pytest.raises(ovk_b200.OvkError) as e:  # 40 output channels are not whole 16-byte groups
        ctx().qlinear_conv_channels_last(w40, xp, -5, 0, ratio[:40], None, -11, out, (1, 1, 1, 1), y_signed=True, pads=pads)
    assert e.value.status == ovk_b200.UNSUPPORTED
