"""The C++ node-level layer: library loads, exports its symbols, and its claim
predicate takes and refuses the node forms the reference's does (no GPU)."""
import ctypes
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def hl():
    from ovk_b200 import host_layer
    if not os.path.exists(host_layer.LIB_PATH):
        subprocess.run([sys.executable, os.path.join(ROOT, "onnx-vulkan-rs_b200", "build.py")], check=True)
    return host_layer


def test_library_exports_every_bound_symbol(hl):
    lib = ctypes.CDLL(hl.LIB_PATH)
    assert not [n for n in hl.SIGNATURES if not hasattr(lib, n)]


def nbits_node(hl, **over):
    attrs = dict(K=64, N=8, bits=4, block_size=32)
    attrs.update(over.pop("attrs", {}))
    inputs = over.pop("inputs", ["a", "quant", "scales", "zp"])
    return hl.Node("MatMulNBits", inputs, ["y"], domain="com.microsoft", **attrs)


def test_matmul_nbits_predicate(hl):
    """interp.rs:452-464: 4 bits, block_size a multiple of 8, no g_idx, no bias."""
    assert nbits_node(hl).implemented
    assert not nbits_node(hl, attrs={"bits": 8}).implemented
    assert not nbits_node(hl, attrs={"bits": 2}).implemented
    assert not nbits_node(hl, attrs={"block_size": 12}).implemented
    assert not nbits_node(hl, attrs={"block_size": 0}).implemented
    assert not nbits_node(hl, inputs=["a", "quant", "scales", "zp", "g_idx"]).implemented
    assert not nbits_node(hl, inputs=["a", "quant", "scales", "zp", "", "bias"]).implemented
    assert not nbits_node(hl, inputs=["a", "quant"]).implemented
    # accepted beyond the reference: no zero point input means the implicit 8
    assert nbits_node(hl, inputs=["a", "quant", "scales"]).implemented
    assert nbits_node(hl, inputs=["a", "quant", "scales", ""]).implemented


def test_qlinear_conv_predicate(hl):
    """interp.rs:560-572: the eight quantization inputs present, a known auto_pad."""
    ins = ["x", "xs", "xz", "w", "ws", "wz", "ys", "yz"]
    assert hl.Node("QLinearConv", ins, ["y"]).implemented
    assert hl.Node("QLinearConv", ins + ["b"], ["y"], auto_pad="SAME_UPPER").implemented
    assert not hl.Node("QLinearConv", ins[:7], ["y"]).implemented
    assert not hl.Node("QLinearConv", ["x", "xs", "", "w", "ws", "wz", "ys", "yz"], ["y"]).implemented
    assert not hl.Node("QLinearConv", ins, ["y"], auto_pad="SAME").implemented


def test_other_operators_of_the_path(hl):
    assert hl.Node("DynamicQuantizeLinear", ["x"], ["y", "s", "z"]).implemented
    assert not hl.Node("DynamicQuantizeLinear", ["x"], ["y"]).implemented
    assert hl.Node("MatMulInteger", ["a", "b"], ["y"]).implemented
    assert hl.Node("MatMulInteger", ["a", "b", "az", "bz"], ["y"]).implemented
    assert hl.Node("MatMulIntegerScaleBias", ["a", "b", "az", "bz", "s", "bias"], ["y"], relu=1).implemented
    assert hl.Node("ConvInteger", ["x", "w", "xz"], ["y"]).implemented
    assert hl.Node("ConvIntegerScaleBias", ["x", "w", "xz", "wz", "s", "bias"], ["y"]).implemented
    assert hl.Node("ConvIntegerScaleBias", ["x", "w", "xz", "wz", "s", "bias", "s2"], ["y"], relu=1).implemented
    assert not hl.Node("ConvIntegerScaleBias", ["x", "w", "xz", "wz", "s"], ["y"]).implemented
    assert hl.Node("QLinearMatMul", ["a", "as", "az", "b", "bs", "bz", "ys", "yz"], ["y"]).implemented
    assert not hl.Node("QLinearMatMul", ["a", "as", "az", "b"], ["y"]).implemented
    # everything outside the quantized matrix products stays with the host runtime
    for op in ("MatMul", "Conv", "Softmax", "QLinearAdd", "Gemm"):
        assert not hl.Node(op, ["a", "b"], ["y"]).implemented
