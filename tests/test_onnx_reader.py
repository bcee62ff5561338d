"""The minimal .onnx reader: nodes, attributes and initializers out of the wire format (no GPU)."""
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
