"""Node-level parity: the operators driven the way the reference's interpreter
drives them - a node, named tensors in an environment - against the CPU port."""
import json
import os

import numpy as np
import pytest

import cases
import oracle as orc
from gpu_util import assert_close

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def hl():
    from ovk_b200 import host_layer
    return host_layer


@pytest.fixture()
def env(hl):
    e = hl.Env(0)
    yield e
    e.close()


def set_nbits(env, a, nib, zp, scale, block_size):
    env.set("a", a)
    env.set("quant", orc.pack_nibbles(nib, block_size), initializer=True)
    env.set("scales", scale.reshape(-1), initializer=True)
    if zp is not None:
        env.set("zp", orc.pack_zero_points(zp), initializer=True)


@pytest.mark.parametrize("m,k,n,bs", cases.NBITS_REFERENCE_CASES[:4] + [(3, 128, 4096, 32), (1, 80, 33, 16)])
def test_matmul_nbits_reference_cases(hl, env, m, k, n, bs):
    """crates/onnx-vulkan-core/tests/matmul_nbits.rs:64-127: same node, same closed-form inputs, 1e-4."""
    a, nib, zp, scale = cases.nbits_reference_case(m, k, n, bs)
    set_nbits(env, a, nib, zp, scale, bs)
    node = hl.Node("MatMulNBits", ["a", "quant", "scales", "zp"], ["y"], domain="com.microsoft",
                   K=k, N=n, bits=4, block_size=bs)
    env.execute(node)
    got = env.host("y")
    assert got.shape == (m, n) and got.dtype == np.float32
    assert_close(got, cases.nbits_expected_f64(a, nib, zp, scale, bs), 1e-4, 1e-4)


def test_matmul_nbits_weight_prepared_once_and_leading_dims(hl, env):
    """The packed weight is cached by initializer name (cache.rs:231); A keeps its leading dimensions."""
    a, nib, zp, scale = cases.nbits_synthetic(21, 6, 256, 96, 32)
    set_nbits(env, a.reshape(2, 3, 256), nib, zp, scale, 32)
    node = hl.Node("MatMulNBits", ["a", "quant", "scales", "zp"], ["y"], K=256, N=96, bits=4, block_size=32)
    env.execute(node)
    first = env.host("y")
    assert first.shape == (2, 3, 96) and first.dtype == np.float16
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(zp), 256, 96, 32)
    assert_close(first.reshape(6, 96), want, 1e-3, 1e-3)
    env.set("a", a[:1])
    env.execute(node)
    assert_close(env.host("y"), want[:1], 1e-3, 1e-3)


def test_matmul_nbits_k_mismatch_is_an_error(hl, env):
    """interp.rs:6441-6447."""
    a, nib, zp, scale = cases.nbits_reference_case(1, 64, 8, 32)
    set_nbits(env, a, nib, zp, scale, 32)
    node = hl.Node("MatMulNBits", ["a", "quant", "scales", "zp"], ["y"], K=96, N=8, bits=4, block_size=32)
    with pytest.raises(hl.OvkError, match="disagrees with K=96"):
        env.execute(node)


def test_dynamic_quantize_then_matmul_integer_chain(hl, env):
    """DynamicQuantizeLinear -> MatMulInteger with the zero point staying on the device (interp.rs:1945-2183)."""
    x = cases.rng_for(22, 0).standard_normal((70, 96), dtype=np.float32)
    b = cases.lcg_bytes_fast(96 * 50, 9).reshape(96, 50).view(np.int8)
    env.set("x", x)
    env.set("b", b, initializer=True)
    env.execute(hl.Node("DynamicQuantizeLinear", ["x"], ["xq", "xs", "xz"]))
    env.execute(hl.Node("MatMulInteger", ["xq", "b", "xz"], ["acc"]))
    yq, scale, zp = orc.dynamic_quantize(x)
    assert np.array_equal(env.host("xq"), yq)
    assert env.host("xs").reshape(()) == scale and int(env.host("xz").reshape(())) == zp
    assert np.array_equal(env.host("acc"), orc.matmul_integer(yq, b, zp, 0))


@pytest.mark.parametrize("relu,col_scale", [(0, True), (1, False)])
def test_matmul_integer_scale_bias(hl, env, relu, col_scale):
    """crates/onnx-vulkan-core/tests/integer_epilogue.rs: bit-equal to the unfused Cast, Mul, Add [, Relu]."""
    m, k, n = 33, 64, 40
    a = cases.lcg_bytes_fast(m * k, 5).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 17).reshape(k, n).view(np.int8)
    scale = cases.rng_for(23, 0).uniform(1e-3, 2e-2, size=n if col_scale else 1).astype(np.float32)
    bias = cases.rng_for(23, 1).standard_normal(n, dtype=np.float32)
    env.set("a", a)
    env.set("b", b, initializer=True)
    env.set("az", np.array([121], dtype=np.uint8))
    env.set("s", scale, initializer=True)
    env.set("bias", bias, initializer=True)
    env.execute(hl.Node("MatMulIntegerScaleBias", ["a", "b", "az", "", "s", "bias"], ["y"], relu=relu))
    acc = orc.matmul_integer(a, b, 121, 0)
    want = orc.scale_bias_epilogue(acc, scale, int(col_scale), bias, 1, relu=bool(relu))
    assert np.array_equal(env.host("y").view(np.uint32), want.view(np.uint32))


# (A shape, N, W int8?, scale kind, relu): the layers of tests/matmul_integer_epilogue.rs that the reference does NOT
# fuse (:423, :471, :517, :596, :722) - a scale over rows - which run as MatMulInteger, Cast, Mul, Add [, Relu]
UNFUSED_LAYERS = [((64, 32), 32, False, "rows", False), ((40, 3), 24, False, "rows", False),
                  ((64, 32), 32, False, "rows", True), ((48, 36), 40, False, "rows_x_cols", True),
                  ((2, 5, 16), 12, True, "rows3", False)]


@pytest.mark.parametrize("a_shape,n,w_int8,kind,relu", UNFUSED_LAYERS)
def test_scale_over_rows_runs_the_unfused_nodes(hl, env, a_shape, n, w_int8, kind, relu):
    """interp.rs:2600-2665: a scale that broadcasts over rows has no column step, so the fused store does not
    apply and the node runs MatMulInteger then Cast, Mul, Add [, Relu] - same bits as the separate nodes."""
    k = a_shape[-1]
    rows = int(np.prod(a_shape[:-1]))
    a = cases.lcg_bytes_fast(rows * k, 3).reshape(a_shape)
    b = cases.lcg_bytes_fast(k * n, 2).reshape(k, n)
    b = b.view(np.int8) if w_int8 else b
    rng = np.random.default_rng(rows + n)
    bias = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    inputs = ["a", "b", "az", "bz", "s", "bias"]
    if kind == "rows":
        scale = rng.uniform(1e-3, 2e-2, (rows, 1)).astype(np.float32)
        s_full = np.broadcast_to(scale, (rows, n))
    elif kind == "rows3":
        scale = rng.uniform(1e-3, 2e-2, a_shape[:-1] + (1,)).astype(np.float32)
        s_full = np.broadcast_to(scale.reshape(rows, 1), (rows, n))
    else:  # a per-row scale times a per-column second factor, multiplied first (:722)
        scale = rng.uniform(1e-3, 2e-2, (rows, 1)).astype(np.float32)
        prod = rng.uniform(0.5, 2.0, n).astype(np.float32)
        env.set("p", prod, initializer=True)
        inputs.append("p")
        s_full = (np.broadcast_to(scale, (rows, n)) * prod[None, :]).astype(np.float32)
    env.set("a", a)
    env.set("b", b, initializer=True)
    env.set("az", np.array([131], dtype=np.uint8))
    env.set("bz", np.array([-7], dtype=np.int8) if w_int8 else np.array([121], dtype=np.uint8))
    env.set("s", scale, initializer=True)
    env.set("bias", bias, initializer=True)
    env.execute(hl.Node("MatMulIntegerScaleBias", inputs, ["y"], relu=int(relu)))
    assert env.last_kernel == "scale_bias_broadcast"
    acc = orc.matmul_integer(a.reshape(rows, k), b, 131, -7 if w_int8 else 121)
    want = (acc.astype(np.float32) * s_full).astype(np.float32) + bias[None, :]
    want = np.maximum(want, np.float32(0)) if relu else want
    got = env.host("y")
    assert got.shape == tuple(a_shape[:-1]) + (n,)
    assert np.array_equal(got.reshape(rows, n).view(np.uint32), want.astype(np.float32).view(np.uint32))


def test_a_scale_that_broadcasts_neither_way_is_refused(hl, env):
    env.set("a", np.zeros((4, 8), dtype=np.uint8))
    env.set("b", np.zeros((8, 6), dtype=np.int8), initializer=True)
    env.set("s", np.ones((2, 1), dtype=np.float32), initializer=True)  # 2 rows against 4
    env.set("bias", np.zeros(6, dtype=np.float32), initializer=True)
    with pytest.raises(hl.OvkError) as err:
        env.execute(hl.Node("MatMulIntegerScaleBias", ["a", "b", "", "", "s", "bias"], ["y"]))
    assert err.value.status == 2


@pytest.mark.parametrize("bias_shape,fused", [((1, 40, 1, 1), True), ((40, 1, 1), True), ((1, 1, 1, 20), False)])
def test_conv_integer_scale_bias_node(hl, env, bias_shape, fused):
    """crates/onnx-vulkan-core/tests/conv_integer_epilogue.rs:248-311: a bias per
    channel fuses; one along the width has no channel step and stays four nodes."""
    x = cases.lcg_bytes_fast(64 * 20 * 20, 1).reshape(1, 64, 20, 20)
    w = cases.lcg_bytes_fast(40 * 64 * 9, 2).reshape(40, 64, 3, 3).view(np.int8)
    bias = np.random.default_rng(3).uniform(-0.5, 0.5, bias_shape).astype(np.float32)
    env.set("x", x)
    env.set("w", w, initializer=True)
    env.set("xz", np.array(131, dtype=np.uint8), initializer=True)
    env.set("s", np.array(0.0123, dtype=np.float32))
    env.set("s2", np.array(3.1e-3, dtype=np.float32), initializer=True)
    env.set("bias", bias, initializer=True)
    node = hl.Node("ConvIntegerScaleBias", ["x", "w", "xz", "", "s", "bias", "s2"], ["y"], kernel_shape=[3, 3],
                   pads=[1, 1, 1, 1])
    if not fused:
        with pytest.raises(hl.OvkError) as err:
            env.execute(node)
        assert err.value.status == 2 and "not fused" in str(err.value)
        return
    env.execute(node)
    acc = np.ascontiguousarray(np.moveaxis(orc.conv_integer(x, w, 131, 0, pads=(1, 1, 1, 1)), 1, -1))
    want = orc.scale_bias_epilogue(acc, np.array([0.0123], np.float32), 0, bias.reshape(-1), 1,
                                   product=np.array([3.1e-3], np.float32), product_step=0)
    assert np.array_equal(env.host("y").view(np.uint32), np.moveaxis(want, -1, 1).view(np.uint32))


def literal(name):
    return json.load(open(os.path.join(GOLDEN, "qlinear_literal_vectors.json")))[name]


def set_qlinear_conv(env, c, x_shape, w_shape):
    env.set("x", np.array(c["x"], dtype=np.uint8).reshape(x_shape))
    env.set("xs", np.array(c["x_scale"], dtype=np.float32), initializer=True)
    env.set("xz", np.array(c["x_zp"], dtype=np.uint8), initializer=True)
    env.set("w", np.array(c["w"], dtype=np.int8).reshape(w_shape), initializer=True)
    ws = np.array(c["w_scale"], dtype=np.float32)
    env.set("ws", ws, initializer=True)
    env.set("wz", np.zeros(ws.shape, dtype=np.int8), initializer=True)
    env.set("ys", np.array(c["y_scale"], dtype=np.float32), initializer=True)
    env.set("yz", np.array(c["y_zp"], dtype=np.uint8), initializer=True)
    if "bias" in c:
        env.set("bias", np.array(c["bias"], dtype=np.int32), initializer=True)


@pytest.mark.parametrize("name,xs,ws", [("conv_per_channel", (1, 1, 3, 3), (2, 1, 2, 2)),
                                        ("conv_per_tensor", (1, 1, 3, 3), (2, 1, 2, 2)),
                                        ("conv_no_bias", (1, 1, 2, 2), (1, 1, 2, 2))])
def test_qlinear_conv_literal_vectors(hl, env, name, xs, ws):
    """crates/onnx-vulkan-core/tests/qlinear.rs:106-236, driven as a node."""
    c = literal(name)
    set_qlinear_conv(env, c, xs, ws)
    ins = ["x", "xs", "xz", "w", "ws", "wz", "ys", "yz"] + (["bias"] if "bias" in c else [])
    node = hl.Node("QLinearConv", ins, ["y"], kernel_shape=list(ws[2:]))
    assert env.unsupported_quantization(node) is None
    env.execute(node)
    w_scale = np.atleast_1d(np.array(c["w_scale"], dtype=np.float32))
    want = orc.qlinear_conv(np.array(c["x"], dtype=np.uint8).reshape(xs), c["x_scale"], c["x_zp"],
                            np.array(c["w"], dtype=np.int8).reshape(ws), w_scale, 0, c["y_scale"], c["y_zp"],
                            bias=np.array(c["bias"], dtype=np.int32) if "bias" in c else None)
    assert np.array_equal(env.host("y"), want)


def test_qlinear_conv_refusals_use_the_reference_wording(hl, env):
    """interp.rs:781-847 and tests/qlinear.rs:238-330."""
    c = literal("conv_per_channel")
    set_qlinear_conv(env, c, (1, 1, 3, 3), (2, 1, 2, 2))
    ins = ["x", "xs", "xz", "w", "ws", "wz", "ys", "yz", "bias"]
    node = hl.Node("QLinearConv", ins, ["y"])
    env.set("wz", np.array([0, 3], dtype=np.int8), initializer=True)
    assert env.unsupported_quantization(node) == \
        "QLinearConv: w per-channel zero point is not zero (asymmetric weights)"
    with pytest.raises(hl.OvkError, match="asymmetric weights"):
        env.execute(node)
    env.set("wz", np.zeros(1, dtype=np.int8), initializer=True)
    assert env.unsupported_quantization(node) == "QLinearConv: w scale and zero point have different lengths"
    env.set("wz", np.zeros(2, dtype=np.int8), initializer=True)
    env.set("xs", np.array(c["x_scale"], dtype=np.float32), initializer=False)
    assert env.unsupported_quantization(node) == "QLinearConv: x scale or zero point is not a constant"
    env.set("xs", np.array([0.1, 0.2], dtype=np.float32), initializer=True)
    assert env.unsupported_quantization(node) == "QLinearConv: x scale or zero point is not per-tensor"
    env.set("xs", np.array(c["x_scale"], dtype=np.float32), initializer=True)
    env.set("bias", np.zeros(2, dtype=np.float32), initializer=True)
    assert env.unsupported_quantization(node) == "QLinearConv: B bias is not int32"


@pytest.mark.parametrize("auto_pad", ["SAME_UPPER", "SAME_LOWER", "VALID"])
def test_conv_integer_auto_pad(hl, env, auto_pad):
    """conv_geometry resolves auto_pad on the host (interp.rs:3425-3536)."""
    x = cases.lcg_bytes_fast(2 * 16 * 13 * 10, 3).reshape(2, 16, 13, 10)
    w = cases.lcg_bytes_fast(24 * 16 * 3 * 4, 8).reshape(24, 16, 3, 4).view(np.int8)
    env.set("x", x)
    env.set("w", w, initializer=True)
    env.set("xz", np.array(131, dtype=np.uint8), initializer=True)
    env.execute(hl.Node("ConvInteger", ["x", "w", "xz"], ["y"], strides=[2, 1], auto_pad=auto_pad))
    want = orc.conv_integer(x, w, 131, 0, strides=(2, 1), auto_pad=auto_pad)
    assert np.array_equal(env.host("y"), want)


def test_conv_integer_one_dimensional(hl, env):
    """A 1-D convolution runs as H x 1 (interp.rs:3455-3470)."""
    x = cases.lcg_bytes_fast(3 * 8 * 50, 4).reshape(3, 8, 50)
    w = cases.lcg_bytes_fast(12 * 8 * 5, 6).reshape(12, 8, 5)
    env.set("x", x)
    env.set("w", w, initializer=True)
    env.set("xz", np.array(7, dtype=np.uint8), initializer=True)
    env.set("wz", np.array(100, dtype=np.uint8), initializer=True)
    env.execute(hl.Node("ConvInteger", ["x", "w", "xz", "wz"], ["y"], pads=[2, 1], strides=[2]))
    want = orc.conv_integer(x[..., None], w[..., None], 7, 100, strides=(2, 1), pads=(2, 0, 1, 0))
    got = env.host("y")
    assert got.shape == want.shape[:3] and np.array_equal(got, want[..., 0])


def test_qlinear_matmul(hl, env):
    """interp.rs:4845-4875: MatMulInteger then requantize with one ratio per column."""
    m, k, n = 19, 48, 24
    a = cases.lcg_bytes_fast(m * k, 2).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 7).reshape(k, n).view(np.int8)
    bs = cases.rng_for(24, 0).uniform(0.01, 0.03, size=n).astype(np.float32)
    env.set("a", a)
    env.set("as", np.array(0.02, dtype=np.float32), initializer=True)
    env.set("az", np.array(128, dtype=np.uint8), initializer=True)
    env.set("b", b, initializer=True)
    env.set("bs", bs, initializer=True)
    env.set("bz", np.zeros(n, dtype=np.int8), initializer=True)
    env.set("ys", np.array(0.5, dtype=np.float32), initializer=True)
    env.set("yz", np.array(-3, dtype=np.int8), initializer=True)
    env.execute(hl.Node("QLinearMatMul", ["a", "as", "az", "b", "bs", "bz", "ys", "yz"], ["y"]))
    acc = orc.matmul_integer(a, b, 128, 0)
    want = orc.requantize(acc, 1, orc.requantize_ratio(0.02, bs, 0.5), -3, out_signed=True)
    got = env.host("y")
    assert got.dtype == np.int8 and np.array_equal(got, want)


def test_gather_block_quantized_node(hl, env):
    """crates/onnx-vulkan-core/tests/gather_block_quantized.rs:85-160: the same node, attributes and inputs."""
    from test_oracle_golden import gbq_case
    _, _, scale, table, zpk = gbq_case(32, 128, 32)
    idx = np.array([[0, 31, 7, 7, -1]], dtype=np.int64)
    env.set("table", table, initializer=True)
    env.set("indices", idx)
    env.set("scales", scale, initializer=True)
    env.set("zp", zpk, initializer=True)
    node = hl.Node("GatherBlockQuantized", ["table", "indices", "scales", "zp"], ["out"], domain="com.microsoft",
                   bits=4, block_size=32, gather_axis=0, quantize_axis=1)
    assert node.implemented
    env.execute(node)
    got = env.host("out")
    assert got.shape == (1, 5, 128) and np.array_equal(got, orc.gather_block_quantized(table, idx, scale, zpk, 32))
    env.set("indices", np.array([32], dtype=np.int64))
    with pytest.raises(hl.OvkError, match="outside the 32-row table"):
        env.execute(node)
    assert not hl.Node("GatherBlockQuantized", ["table", "indices", "scales", "zp"], ["out"], block_size=32,
                       gather_axis=1).implemented


@pytest.mark.parametrize("shape,axis,keepdims", [((4, 1000), 1, 1), ((2, 5, 3, 3), 1, 0), ((1, 1, 151936), -1, 0)])
def test_argmax_node(hl, env, shape, axis, keepdims):
    """crates/onnx-vulkan-core/tests/argmax.rs:90-164."""
    x = cases.rng_for(25, 0).standard_normal(shape, dtype=np.float32)
    env.set("x", x)
    node = hl.Node("ArgMax", ["x"], ["out"], axis=axis, keepdims=keepdims)
    env.execute(node)
    got = env.host("out")
    want = orc.argmax(x, axis)
    assert got.dtype == np.int64
    assert np.array_equal(got, np.expand_dims(want, axis % x.ndim) if keepdims else want)
    assert not hl.Node("ArgMax", ["x"], ["out"], axis=axis, select_last_index=1).implemented


def test_quantized_residual_tail_as_nodes(hl, env):
    """QLinearAdd -> MaxPool -> QLinearGlobalAveragePool -> DequantizeLinear -> QuantizeLinear, driven as the
    reference's tests drive them (crates/onnx-vulkan-core/tests/qlinear.rs:279-452): bytes equal to the port."""
    rng = cases.rng_for(26, 0)
    a = rng.integers(0, 256, size=(2, 16, 8, 8)).astype(np.uint8)
    b = rng.integers(0, 256, size=(1, 16, 1, 1)).astype(np.uint8)
    env.set("A", a)
    env.set("B", b, initializer=True)
    for name, value, dt in (("A_scale", 0.02, np.float32), ("A_zp", 128, np.uint8), ("B_scale", 0.05, np.float32),
                            ("B_zp", 100, np.uint8), ("C_scale", 0.03, np.float32), ("C_zp", 30, np.uint8),
                            ("y_scale", 0.07, np.float32), ("y_zp", 3, np.uint8)):
        env.set(name, np.array(value, dtype=dt), initializer=True)
    add = hl.Node("QLinearAdd", ["A", "A_scale", "A_zp", "B", "B_scale", "B_zp", "C_scale", "C_zp"], ["sum"],
                  domain="com.microsoft")
    assert add.implemented and env.unsupported_quantization(add) is None
    env.execute(add)
    want_sum = orc.qlinear_add(a, 0.02, 128, b, 0.05, 100, 0.03, 30)
    assert np.array_equal(env.host("sum"), want_sum)
    env.execute(hl.Node("MaxPool", ["sum"], ["pooled"], kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1]))
    want_pool = orc.maxpool_q(want_sum, (3, 3), (2, 2), (1, 1, 1, 1))
    assert np.array_equal(env.host("pooled"), want_pool)
    env.execute(hl.Node("QLinearGlobalAveragePool", ["pooled", "C_scale", "C_zp", "y_scale", "y_zp"], ["gap"],
                        domain="com.microsoft"))
    want_gap = orc.qlinear_global_average_pool(want_pool, 0.03, 30, 0.07, 3)
    got_gap = env.host("gap")
    assert got_gap.shape == (2, 16, 1, 1) and np.array_equal(got_gap, want_gap)
    env.execute(hl.Node("DequantizeLinear", ["gap", "y_scale", "y_zp"], ["real"]))
    want_real = orc.dequantize_linear(want_gap, np.array([0.07], dtype=np.float32), np.array([3], dtype=np.uint8))
    assert np.array_equal(env.host("real"), want_real)
    env.execute(hl.Node("QuantizeLinear", ["real", "C_scale", "C_zp"], ["again"]))
    assert np.array_equal(env.host("again"), orc.quantize_linear(want_real, np.array([0.03], dtype=np.float32),
                                                                 np.array([30], dtype=np.uint8)))
    # a scale that is not a constant is refused with the reference's wording (interp.rs:781-812)
    env.set("A_scale", np.array(0.02, dtype=np.float32), initializer=False)
    assert env.unsupported_quantization(add) == "QLinearAdd: A scale or zero point is not a constant"
    # float pooling is not this layer's
    env.set("f", np.zeros((1, 1, 4, 4), dtype=np.float32))
    with pytest.raises(hl.OvkError) as err:
        env.execute(hl.Node("MaxPool", ["f"], ["g"], kernel_shape=[2, 2]))
    assert err.value.status == 2


def test_replacing_an_initializer_rebuilds_its_prepared_weight(hl, env):
    """Weights are prepared once per initializer NAME (cache.rs:231).  When the
    environment replaces a tensor under that name the prepared weight must go
    with it: a MatMulNBits weight points into the old device buffers (also those
    of its scales), the MatMulInteger and convolution weights hold a packed copy
    of the old bytes."""
    # MatMulNBits: new nibbles, then new scales only
    a, nib, zp, scale = cases.nbits_synthetic(31, 2, 128, 48, 32)
    set_nbits(env, a, nib, zp, scale, 32)
    node = hl.Node("MatMulNBits", ["a", "quant", "scales", "zp"], ["y"], K=128, N=48, bits=4, block_size=32)
    env.execute(node)
    env.host("y")
    _, nib2, zp2, scale2 = cases.nbits_synthetic(32, 2, 128, 48, 32)
    env.set("quant", orc.pack_nibbles(nib2, 32), initializer=True)
    env.execute(node)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib2, 32), scale, orc.pack_zero_points(zp), 128, 48, 32)
    assert_close(env.host("y"), want, 1e-3, 1e-3, "after replacing the nibbles")
    env.set("scales", scale2.reshape(-1), initializer=True)
    env.execute(node)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib2, 32), scale2, orc.pack_zero_points(zp), 128, 48, 32)
    assert_close(env.host("y"), want, 1e-3, 1e-3, "after replacing the scales")

    # MatMulInteger
    xa = cases.lcg_bytes_fast(40 * 64, 3).reshape(40, 64)
    b1 = cases.lcg_bytes_fast(64 * 24, 4).reshape(64, 24).view(np.int8)
    b2 = cases.lcg_bytes_fast(64 * 24, 5).reshape(64, 24).view(np.int8)
    env.set("xa", xa)
    env.set("b", b1, initializer=True)
    mm = hl.Node("MatMulInteger", ["xa", "b"], ["acc"])
    env.execute(mm)
    assert np.array_equal(env.host("acc"), orc.matmul_integer(xa, b1, 0, 0))
    env.set("b", b2, initializer=True)
    env.execute(mm)
    assert np.array_equal(env.host("acc"), orc.matmul_integer(xa, b2, 0, 0))

    # ConvInteger
    x = cases.lcg_bytes_fast(32 * 12 * 12, 6).reshape(1, 32, 12, 12)
    w1 = cases.lcg_bytes_fast(16 * 32 * 9, 7).reshape(16, 32, 3, 3).view(np.int8)
    w2 = cases.lcg_bytes_fast(16 * 32 * 9, 8).reshape(16, 32, 3, 3).view(np.int8)
    env.set("x", x)
    env.set("w", w1, initializer=True)
    cv = hl.Node("ConvInteger", ["x", "w"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    env.execute(cv)
    assert np.array_equal(env.host("c"), orc.conv_integer(x, w1, 0, 0, pads=(1, 1, 1, 1)))
    env.set("w", w2, initializer=True)
    env.execute(cv)
    assert np.array_equal(env.host("c"), orc.conv_integer(x, w2, 0, 0, pads=(1, 1, 1, 1)))


def test_decomposed_gelu_quantize_node_and_the_range_a_producer_folded(hl, env):
    """The Parakeet FF block as nodes (rewrite.rs:445-542, :699-735): MatMulIntegerScaleBias folds the range of
    its output, the DynamicQuantizeLinear after it runs one pass; DecomposedGeluQuantize keeps the GELU's
    inputs and attribute and the quantization's outputs."""
    import math
    m, k, n = 70, 96, 64
    a = cases.lcg_bytes_fast(m * k, 5).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 17).reshape(k, n).view(np.int8)
    scale = np.array([2e-3], dtype=np.float32)
    bias = cases.rng_for(23, 1).standard_normal(n, dtype=np.float32)
    env.set("a", a)
    env.set("b", b, initializer=True)
    env.set("az", np.array([121], dtype=np.uint8))
    env.set("s", scale, initializer=True)
    env.set("bias", bias, initializer=True)
    env.execute(hl.Node("MatMulIntegerScaleBias", ["a", "b", "az", "", "s", "bias"], ["h"], range=1))
    env.execute(hl.Node("DynamicQuantizeLinear", ["h"], ["hq", "hs", "hz"]))
    assert env.last_kernel == "dql_quantize"
    h = orc.scale_bias_epilogue(orc.matmul_integer(a, b, 121, 0), scale, 0, bias, 1)
    assert np.array_equal(env.host("h").view(np.uint32), h.view(np.uint32))
    want = orc.dynamic_quantize(h)
    assert np.array_equal(env.host("hq"), want[0]) and env.host("hs").reshape(()) == want[1]
    # the GELU of the same tensor, quantized without being stored
    for name, v in (("c1", math.sqrt(2.0)), ("c2", 1.0), ("c3", 0.5)):
        env.set(name, np.array(v, dtype=np.float32), initializer=True)
    env.execute(hl.Node("DecomposedGeluQuantize", ["h", "c1", "c2", "c3"], ["gq", "gs", "gz"], factor_first=1))
    gq, gs, gz = orc.decomposed_gelu_quantize(h, float(np.float32(math.sqrt(2.0))), 1.0, 0.5, True)
    assert np.array_equal(env.host("gq"), gq) and env.host("gs").reshape(()) == gs and int(env.host("gz").reshape(())) == gz
    env.execute(hl.Node("DecomposedGelu", ["h", "c1", "c2", "c3"], ["g"], factor_first=1))
    g = orc.decomposed_gelu(h, float(np.float32(math.sqrt(2.0))), 1.0, 0.5, True)
    assert np.array_equal(env.host("g").view(np.uint32), g.view(np.uint32))
    # a constant that is a vector is the form the reference replays as five nodes: refused here
    env.set("c1", np.full(n, math.sqrt(2.0), dtype=np.float32), initializer=True)
    with pytest.raises(hl.OvkError) as err:
        env.execute(hl.Node("DecomposedGelu", ["h", "c1", "c2", "c3"], ["g2"]))
    assert err.value.status == 2 and "replays" in str(err.value)
