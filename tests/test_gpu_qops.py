"""QLinearAdd, MaxPool on codes, QLinearGlobalAveragePool, QuantizeLinear, DequantizeLinear: bytes equal."""
import numpy as np
import pytest
import torch

import cases
import oracle as orc
from gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def test_qlinear_add_every_input_pair():
    """crates/onnx-vulkan-core/tests/qlinear.rs:356-373."""
    scales, zps = (0.03207505, 0.061237868, 0.067996934), (116, 145, 125)
    a = (np.arange(65536) % 256).astype(np.uint8)
    b = (np.arange(65536) // 256).astype(np.uint8)
    got = host(ctx().qlinear_add(dev(a), scales[0], zps[0], dev(b), scales[1], zps[1], scales[2], zps[2]))
    assert ctx().last_kernel == "qlinear_add"
    for av, bv, cpu in [(129, 91, 82), (162, 147, 148), (195, 203, 214)]:
        assert got[bv * 256 + av] == cpu
    assert np.array_equal(got, orc.qlinear_add(a, scales[0], zps[0], b, scales[1], zps[1], scales[2], zps[2]))


@pytest.mark.parametrize("a_shape,b_shape,signed", [
    ((2, 3), (3,), False),                    # tests/qlinear.rs:279-314: a bias row on logits
    ((1,), (256,), False),                    # :376-392: a broadcast first operand is exchanged
    ((4, 1000), (1000,), False),
    ((2, 64, 7, 5), (1, 64, 1, 1), True),     # a per-channel addend, int8
    ((3, 1, 5), (1, 4, 1), False),            # both sides broadcast
    ((2, 256, 56, 56), (2, 256, 56, 56), False),  # the residual add of a ResNet block
])
def test_qlinear_add_broadcasts(a_shape, b_shape, signed):
    rng = cases.rng_for(41, len(a_shape) * 10 + len(b_shape))
    dt = np.int8 if signed else np.uint8
    lo, hi = (-128, 128) if signed else (0, 256)
    a = rng.integers(lo, hi, size=a_shape).astype(dt)
    b = rng.integers(lo, hi, size=b_shape).astype(dt)
    args = (0.264079, -5 if signed else 128, 0.081802, 17 if signed else 205, 0.110314, -9 if signed else 43)
    got = ctx().qlinear_add(dev(a), args[0], args[1], dev(b), args[2], args[3], args[4], args[5])
    want = orc.qlinear_add(a, args[0], args[1], b, args[2], args[3], args[4], args[5])
    assert tuple(got.shape) == want.shape and np.array_equal(host(got), want)


@pytest.mark.parametrize("shape,kernel,strides,pads,dil,signed", [
    ((1, 1, 4, 4), (2, 2), (2, 2), (0, 0, 0, 0), (1, 1), False),       # tests/qlinear.rs:395-416
    ((2, 64, 112, 112), (3, 3), (2, 2), (1, 1, 1, 1), (1, 1), False),  # the stem pooling of resnet50-int8
    ((3, 5, 17, 13), (3, 2), (1, 2), (1, 0, 0, 1), (2, 1), True),
])
def test_maxpool_q(shape, kernel, strides, pads, dil, signed):
    x = cases.lcg_bytes_fast(int(np.prod(shape)), 13).reshape(shape)
    x = x.view(np.int8) if signed else x
    got = ctx().maxpool_q(dev(x), kernel, strides, pads, dil)
    want = orc.maxpool_q(x, kernel, strides, pads, dil)
    assert tuple(got.shape) == want.shape and np.array_equal(host(got), want)


@pytest.mark.parametrize("shape,signed", [((1, 2, 2, 2), False), ((8, 2048, 7, 7), False), ((3, 10, 5, 9), True)])
def test_qlinear_global_average_pool(shape, signed):
    """tests/qlinear.rs:419-452 and the 7x7 pooling both classifier models end on."""
    x = cases.lcg_bytes_fast(int(np.prod(shape)), 29).reshape(shape)
    x = x.view(np.int8) if signed else x
    zps = (-4, 9) if signed else (15, 7)
    got = ctx().qlinear_global_average_pool(dev(x), 0.02, zps[0], 0.05, zps[1])
    want = orc.qlinear_global_average_pool(x, 0.02, zps[0], 0.05, zps[1])
    assert tuple(got.shape) == want.shape and np.array_equal(host(got), want)


def test_quantize_linear_ties_and_per_axis():
    x = np.array([-13.5, -12.5, 0.49, 0.5, 1.5, 2.5, 300.0, -300.0], dtype=np.float32)
    one = dev(np.array([1.0], dtype=np.float32))
    assert host(ctx().quantize_linear(dev(x), one, dev(np.array([10], dtype=np.uint8)))).tolist() == \
        [0, 0, 10, 10, 12, 12, 255, 0]
    assert host(ctx().quantize_linear(dev(x), one, dev(np.array([-3], dtype=np.int8)))).tolist() == \
        [-17, -15, -3, -3, -1, -1, 127, -128]
    xa = cases.rng_for(42, 0).standard_normal((4, 96, 28, 28), dtype=np.float32) * 3
    scale = cases.rng_for(42, 1).uniform(0.01, 0.1, size=96).astype(np.float32)
    zp = cases.rng_for(42, 2).integers(0, 256, size=96).astype(np.uint8)
    got = ctx().quantize_linear(dev(xa), dev(scale), dev(zp), axis=1)
    assert np.array_equal(host(got), orc.quantize_linear(xa, scale, zp, axis=1))
    no_zp = ctx().quantize_linear(dev(xa), dev(scale[:1].copy()), None, signed=True)
    assert no_zp.dtype == torch.int8 and np.array_equal(host(no_zp), orc.quantize_linear(xa, scale[:1], None, signed=True))


@pytest.mark.parametrize("dtype", [np.uint8, np.int8, np.int32])
def test_dequantize_linear(dtype):
    rng = cases.rng_for(43, np.dtype(dtype).itemsize)
    info = np.iinfo(dtype)
    x = rng.integers(max(info.min, -100000), min(info.max, 100000) + 1, size=(2, 48, 9, 9)).astype(dtype)
    scale = rng.uniform(0.001, 0.1, size=48).astype(np.float32)
    zp = rng.integers(max(info.min, -50), min(info.max, 50) + 1, size=48).astype(dtype)
    got = ctx().dequantize_linear(dev(x), dev(scale), dev(zp), axis=1)
    assert np.array_equal(host(got).view(np.uint32), orc.dequantize_linear(x, scale, zp, axis=1).view(np.uint32))
    flat = ctx().dequantize_linear(dev(x), dev(scale[:1].copy()), None)
    assert np.array_equal(host(flat), orc.dequantize_linear(x, scale[:1], None))
