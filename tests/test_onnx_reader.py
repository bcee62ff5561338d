"""The minimal .onnx reader: nodes, attributes and initializers out of the wire format (no GPU)."""
import os

import numpy as np
import pytest

import cases
import onnx_writer as ow
from ovk_b200 import onnx_reader


def nbits_model(raw=True):
    a, nib, zp, scale = cases.nbits_reference_case(1, 64, 8, 32)
    import oracle as orc
    inits = {"quant": orc.pack_nibbles(nib, 32), "scales": scale.reshape(-1), "zp": orc.pack_zero_points(zp),
             "idx": np.array([[3, -1]], dtype=np.int64), "half": np.array([0.5, -2.0], dtype=np.float16),
             "bias": np.array([-70000, 5], dtype=np.int32)}
    nodes = [ow.node("MatMulNBits", ["a", "quant", "scales", "zp"], ["y"], domain="com.microsoft", name="mm",
                     K=64, N=8, bits=4, block_size=32),
             ow.node("Conv", ["y", "w"], ["z"], kernel_shape=[3, 3], auto_pad="SAME_UPPER", alpha=0.25)]
    return ow.model(nodes, inits, inputs=["a", "quant"], outputs=["z"], raw=raw), inits


@pytest.mark.parametrize("raw", [True, False])
def test_reads_nodes_attributes_and_initializers(raw):
    data, inits = nbits_model(raw)
    m = onnx_reader.parse(data)
    assert [n.op for n in m.nodes] == ["MatMulNBits", "Conv"]
    mm = m.nodes[0]
    assert (mm.domain, mm.name, mm.inputs, mm.outputs) == ("com.microsoft", "mm", ["a", "quant", "scales", "zp"], ["y"])
    assert mm.attrs == {"K": 64, "N": 8, "bits": 4, "block_size": 32}
    assert m.nodes[1].attrs["kernel_shape"] == [3, 3] and m.nodes[1].attrs["auto_pad"] == "SAME_UPPER"
    assert m.nodes[1].attrs["alpha"] == 0.25
    assert m.inputs == ["a"] and m.outputs == ["z"]          # an initializer is not a graph input
    assert m.opsets == {"": 21, "com.microsoft": 1}
    for name, want in inits.items():
        got = m.initializers[name]
        assert got.dtype == want.dtype and got.shape == want.shape and np.array_equal(got, want), name


def test_refuses_what_it_cannot_decode():
    with pytest.raises(onnx_reader.OnnxFormatError):
        onnx_reader.parse(b"\x0a\x02hi")                      # a model without a graph
    with pytest.raises(onnx_reader.OnnxFormatError):
        onnx_reader.parse(ow.blob(7, b"\x2a\xff\x01"))        # an initializer that runs past its message
    ext = ow.blob(1, b"") + ow.field(2, 0, ow.varint(1)) + ow.blob(8, b"w") + ow.field(14, 0, ow.varint(1))
    with pytest.raises(onnx_reader.OnnxFormatError, match="external"):
        onnx_reader.parse(ow.blob(7, ow.blob(5, ext)))


# ---------------------------------------------------------------------------
# The reference's own model files (crates/onnx-vulkan-frontend/tests/models,
# crates/onnx-vulkan/tests/models), written by the `onnx` Python package, and the
# facts its loader tests state about them (crates/onnx-vulkan-frontend/tests/frontend.rs).

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name):
    return onnx_reader.load(os.path.join(GOLDEN, name))


def test_every_storage_form_decodes_to_the_bytes_onnx_declares():
    """frontend.rs:30-57: raw_data, typed repeated fields, and narrow types packed into int32_data."""
    m = golden("mixed.onnx")
    want = {"w_raw": [0, 0, 192, 63, 0, 0, 32, 192, 0, 0, 0, 63, 0, 0, 64, 64],
            "w_typed": [0, 0, 128, 63, 0, 0, 0, 64, 0, 0, 64, 64],
            "i64": [249, 255, 255, 255, 255, 255, 255, 255, 9, 0, 0, 0, 0, 0, 0, 0],
            "u8": [0, 1, 254, 255], "i8": [128, 0, 127], "bool_": [1, 0, 1], "f16": [192, 115, 0, 122]}
    for name, data in want.items():
        assert list(m.initializers[name].tobytes()) == data, name
    shapes = {"w_raw": (np.float32, (2, 2)), "w_typed": (np.float32, (3,)), "i64": (np.int64, (2,)),
              "u8": (np.uint8, (4,)), "i8": (np.int8, (3,)), "bool_": (np.bool_, (3,)), "f16": (np.float16, (2,))}
    for name, (dtype, shape) in shapes.items():  # frontend.rs:60-77
        assert m.initializers[name].dtype == dtype and m.initializers[name].shape == shape, name


def test_nodes_inputs_and_attributes_of_the_mixed_model():
    """frontend.rs:83-138."""
    m = golden("mixed.onnx")
    assert m.inputs == ["x"] and m.outputs == ["out"] and "w_raw" in m.initializers
    assert [n.op for n in m.nodes] == ["Constant", "MatMul", "Concat", "Clip", "LeakyRelu"]
    clip = m.nodes[3]
    assert clip.name == "clip" and clip.inputs == ["y", "", "hi"]  # a missing optional input keeps its position
    assert m.opsets == {"": 17} and all(n.domain == "" for n in m.nodes)
    by_name = {n.name: n for n in m.nodes}
    assert by_name["cat"].attrs["axis"] == 1
    assert by_name["lrelu"].attrs["alpha"] == 0.125
    konst = by_name["konst"].attrs["value"]
    assert konst.shape == () and konst.tobytes() == np.float32(6.0).tobytes()


def test_external_weights_give_the_same_model_and_need_the_models_directory():
    """frontend.rs:141-166."""
    inline, external = golden("mixed.onnx"), golden("external.onnx")
    assert [(n.op, n.name, n.inputs, n.outputs) for n in external.nodes] == \
           [(n.op, n.name, n.inputs, n.outputs) for n in inline.nodes]
    assert external.initializers.keys() == inline.initializers.keys()
    for name, arr in inline.initializers.items():
        got = external.initializers[name]
        assert got.dtype == arr.dtype and got.shape == arr.shape and got.tobytes() == arr.tobytes(), name
    with open(os.path.join(GOLDEN, "external.onnx"), "rb") as fh:
        data = fh.read()
    with pytest.raises(onnx_reader.OnnxFormatError, match="w_raw"):
        onnx_reader.parse(data)  # bytes alone do not say where the weights are


def test_the_other_model_files_read_node_for_node():
    m = golden("shapes.onnx")
    assert [n.op for n in m.nodes][:12] == ["Conv", "Relu", "Add", "MaxPool", "Resize", "Pad", "GlobalAveragePool",
                                            "Flatten", "Gemm", "Softmax", "TopK", "Transpose"]
    conv = m.nodes[0]
    assert conv.inputs == ["x", "w", "b"] and conv.attrs == {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [2, 2]}
    assert m.nodes[4].inputs == ["pooled", "", "", "sizes"] and m.nodes[4].attrs["mode"] == "nearest"
    assert m.initializers["w"].shape == (8, 3, 3, 3) and m.initializers["pads"].dtype == np.int64
    assert m.inputs == ["x"] and m.opsets == {"": 18}
    r = golden("reduce_axes_input.onnx")  # frontend.rs:171-183 (the axes stay an input here: this reader folds nothing)
    assert [(n.op, n.inputs, n.attrs) for n in r.nodes] == [("ReduceSum", ["x", "axes"], {"keepdims": 1})]
    assert r.initializers["axes"].tolist() == [1]
    a = golden("affine.onnx")  # crates/onnx-vulkan/tests/device_values.rs:4-15: y = x * scale + shift over [1, 8192]
    assert [(n.op, n.inputs, n.outputs) for n in a.nodes] == [("Mul", ["x", "scale"], ["t"]), ("Add", ["t", "shift"], ["y"])]
    assert a.initializers["scale"].shape == (8192,) and a.initializers["shift"].dtype == np.float32
    with pytest.raises(onnx_reader.OnnxFormatError):
        onnx_reader.parse(b"this is not an ONNX protobuf")  # frontend.rs:185-191


@pytest.mark.gpu
def test_exported_weights_run_through_the_host_layer():
    """File bytes -> reader -> environment -> MatMulNBits node on the device, against the port."""
    import oracle as orc
    from ovk_b200 import host_layer
    data, inits = nbits_model()
    m = onnx_reader.parse(data)
    claimed = onnx_reader.to_nodes(m)
    assert [info.op for info, _ in claimed] == ["MatMulNBits"]
    env = host_layer.Env(0)
    try:
        onnx_reader.to_env(m, env, [info for info, _ in claimed])
        a, nib, zp, scale = cases.nbits_reference_case(1, 64, 8, 32)
        env.set("a", a)
        env.execute(claimed[0][1])
        want = cases.nbits_expected_f64(a, nib, zp, scale, 32)
        assert np.allclose(env.host("y"), want, atol=1e-4, rtol=1e-4)
    finally:
        env.close()
