"""A minimal reader of ``.onnx`` files: nodes and initializers only.

Enough to feed exported weights of the quantized matrix-product operators
through the C ABI without any ONNX package: it walks the protobuf wire format
of ``ModelProto -> GraphProto -> {NodeProto, TensorProto}``, external weight files included (the public ONNX
schema; the reference vendors it as crates/onnx-vulkan-frontend/proto/onnx.proto
and converts it in crates/onnx-vulkan-frontend/src/convert.rs) and ignores every
field it does not need.  It does no shape inference and follows no sub-graphs.

    model = onnx_reader.load("decoder.onnx")
    for node in model.nodes:                      # NodeInfo(op, domain, name, inputs, outputs, attrs)
        ...
    table = model.initializers["model.embed_tokens.weight_Q4"]   # numpy array

``to_env`` puts the initializers a set of nodes needs into a ``host_layer.Env``
and ``to_nodes`` turns ``NodeInfo`` records into ``host_layer.Node`` objects.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

# TensorProto.DataType -> numpy (crates/onnx-vulkan-core/src/graph.rs:13-41 uses the same codes)
_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_,
           10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}


class OnnxFormatError(ValueError):
    pass


@dataclass
class NodeInfo:
    op: str = ""
    domain: str = ""
    name: str = ""
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)
    attrs: dict = field(default_factory=dict)


@dataclass
class Model:
    nodes: list
    initializers: dict
    inputs: list
    outputs: list
    opsets: dict


def _varint(buf, pos):
    result = shift = 0
    while True:
        if pos >= len(buf):
            raise OnnxFormatError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise OnnxFormatError("varint too long")


def _fields(buf):
    """Yields (field number, wire type, value) of one message; value is an int or a memoryview."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _varint(buf, pos)
        number, wire = key >> 3, key & 7
        if wire == 0:
            value, pos = _varint(buf, pos)
        elif wire == 1:
            value, pos = bytes(buf[pos:pos + 8]), pos + 8
        elif wire == 2:
            size, pos = _varint(buf, pos)
            if pos + size > end:
                raise OnnxFormatError("length-delimited field runs past its message")
            value, pos = buf[pos:pos + size], pos + size
        elif wire == 5:
            value, pos = bytes(buf[pos:pos + 4]), pos + 4
        else:
            raise OnnxFormatError(f"wire type {wire} is not used by ONNX")
        yield number, wire, value


def _signed(v):
    return v - (1 << 64) if v >= 1 << 63 else v


def _packed_varints(value, wire):
    if wire == 0:
        return [_signed(value)]
    out, pos = [], 0
    while pos < len(value):
        v, pos = _varint(value, pos)
        out.append(_signed(v))
    return out


def _external_bytes(name, entries, base_dir, np_dtype, count):
    """The bytes of a tensor kept in a file beside the model (TensorProto.external_data: location, offset,
    length), as the reference's loader resolves them against the model's directory
    (crates/onnx-vulkan-frontend/src/lib.rs:52-63)."""
    import os
    if base_dir is None:
        raise OnnxFormatError(f"initializer {name!r} keeps its data in an external file, and the model was given as "
                              "bytes without the directory it came from")
    location = entries.get("location")
    if not location:
        raise OnnxFormatError(f"initializer {name!r}: external data without a location")
    path = os.path.normpath(os.path.join(base_dir, location))
    if os.path.isabs(location) or os.path.relpath(path, base_dir).startswith(".."):
        raise OnnxFormatError(f"initializer {name!r}: external data outside the model's directory ({location!r})")
    offset = int(entries.get("offset", "0") or 0)
    length = int(entries["length"]) if entries.get("length") else count * np_dtype.itemsize
    try:
        with open(path, "rb") as fh:
            fh.seek(offset)
            data = fh.read(length)
    except OSError as e:
        raise OnnxFormatError(f"initializer {name!r}: cannot read external data {location!r}: {e}") from e
    if len(data) != length:
        raise OnnxFormatError(f"initializer {name!r}: external file {location!r} is short ({len(data)} of {length} bytes)")
    return data


def _tensor(buf, base_dir=None):
    dims, dtype, name, raw = [], 0, "", None
    floats, ints32, ints64 = [], [], []
    external = False
    entries = {}
    for number, wire, value in _fields(buf):
        if number == 1:
            dims += _packed_varints(value, wire)
        elif number == 2:
            dtype = value
        elif number == 4:
            floats.append(bytes(value) if wire == 2 else value)
        elif number == 5:
            ints32 += _packed_varints(value, wire)
        elif number == 7:
            ints64 += _packed_varints(value, wire)
        elif number == 8:
            name = bytes(value).decode()
        elif number == 9:
            raw = bytes(value)
        elif number == 13 and wire == 2:  # StringStringEntryProto {key = 1, value = 2}
            key = val = ""
            for n2, _, v2 in _fields(value):
                if n2 == 1:
                    key = bytes(v2).decode()
                elif n2 == 2:
                    val = bytes(v2).decode()
            entries[key] = val
        elif number == 14 and value == 1:
            external = True
    if dtype not in _DTYPES:
        raise OnnxFormatError(f"initializer {name!r} has data type {dtype}, which this reader does not decode")
    np_dtype = np.dtype(_DTYPES[dtype])
    count = int(np.prod(dims, dtype=np.int64)) if dims else 1
    if external:
        raw = _external_bytes(name, entries, base_dir, np_dtype, count)
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np_dtype.newbyteorder("<"))
    elif dtype == 1:
        arr = np.frombuffer(b"".join(floats), dtype="<f4")
    elif dtype == 7:
        arr = np.array(ints64, dtype=np.int64)
    elif dtype == 10:  # float16 values travel as their bit patterns in int32_data
        arr = np.array(ints32, dtype=np.uint16).view(np.float16)
    else:
        arr = np.array(ints32).astype(np_dtype)
    if arr.size != count:
        raise OnnxFormatError(f"initializer {name!r}: {arr.size} values for shape {dims}")
    return name, np.ascontiguousarray(arr.astype(np_dtype, copy=False)).reshape(dims)


def _attribute(buf, base_dir=None):
    name, kind = "", 0
    f = i = s = t = None
    ints, floats, strings = [], [], []
    for number, wire, value in _fields(buf):
        if number == 1:
            name = bytes(value).decode()
        elif number == 20:
            kind = value
        elif number == 2:
            f = struct.unpack("<f", value)[0]
        elif number == 3:
            i = _signed(value)
        elif number == 4:
            s = bytes(value)
        elif number == 5:
            t = _tensor(value, base_dir)[1]
        elif number == 7:
            floats += list(struct.unpack(f"<{len(value) // 4}f", bytes(value))) if wire == 2 else [struct.unpack("<f", value)[0]]
        elif number == 8:
            ints += _packed_varints(value, wire)
        elif number == 9:
            strings.append(bytes(value))
    by_kind = {1: f, 2: i, 3: None if s is None else s.decode(errors="replace"), 4: t, 6: floats, 7: ints,
               8: [x.decode(errors="replace") for x in strings]}
    if kind in by_kind:
        return name, by_kind[kind]
    for candidate in (i, f, None if s is None else s.decode(errors="replace"), t):  # files without the discriminator
        if candidate is not None:
            return name, candidate
    return name, ints or floats or strings or None


def _node(buf, base_dir=None):
    node = NodeInfo()
    for number, _, value in _fields(buf):
        if number == 1:
            node.inputs.append(bytes(value).decode())
        elif number == 2:
            node.outputs.append(bytes(value).decode())
        elif number == 3:
            node.name = bytes(value).decode()
        elif number == 4:
            node.op = bytes(value).decode()
        elif number == 7:
            node.domain = bytes(value).decode()
        elif number == 5:
            key, val = _attribute(value, base_dir)
            node.attrs[key] = val
    return node


def _value_name(buf):
    for number, _, value in _fields(buf):
        if number == 1:
            return bytes(value).decode()
    return ""


def parse(data: bytes, base_dir: str | None = None) -> Model:
    """Parses the bytes of a ``.onnx`` file.  ``base_dir`` is the directory external weight files are
    looked up in; without it a model that has any is refused (the reference's ``load_from_bytes(bytes, None)``)."""
    view = memoryview(data)
    graph, opsets = None, {}
    for number, wire, value in _fields(view):
        if number == 7 and wire == 2:
            graph = value
        elif number == 8 and wire == 2:
            domain, version = "", 0
            for n2, _, v2 in _fields(value):
                if n2 == 1:
                    domain = bytes(v2).decode()
                elif n2 == 2:
                    version = v2
            opsets[domain] = version
    if graph is None:
        raise OnnxFormatError("no graph in the model")
    nodes, inits, inputs, outputs = [], {}, [], []
    for number, wire, value in _fields(graph):
        if wire != 2:
            continue
        if number == 1:
            nodes.append(_node(value, base_dir))
        elif number == 5:
            name, arr = _tensor(value, base_dir)
            inits[name] = arr
        elif number == 11:
            inputs.append(_value_name(value))
        elif number == 12:
            outputs.append(_value_name(value))
    return Model(nodes, inits, [n for n in inputs if n not in inits], outputs, opsets)


def load(path: str) -> Model:
    """Reads a model file; external weights are resolved against its directory."""
    import os
    with open(path, "rb") as fh:
        return parse(fh.read(), os.path.dirname(os.path.abspath(path)))


# ------------------------------------------------------------------ onto the host layer

def to_nodes(model: Model, only_implemented: bool = True):
    """``host_layer.Node`` objects for the model's nodes (by default only those the layer claims)."""
    from . import host_layer
    out = []
    for n in model.nodes:
        attrs = {k: v for k, v in n.attrs.items() if isinstance(v, (int, str)) or
                 (isinstance(v, list) and all(isinstance(x, int) for x in v))}
        node = host_layer.Node(n.op, n.inputs, n.outputs, domain=n.domain, name=n.name, **attrs)
        if node.implemented or not only_implemented:
            out.append((n, node))
    return out


def to_env(model: Model, env, nodes=None) -> None:
    """Uploads the initializers the given nodes (default: all) read into a ``host_layer.Env``."""
    wanted = None if nodes is None else {name for n in nodes for name in n.inputs}
    for name, arr in model.initializers.items():
        if wanted is None or name in wanted:
            env.set(name, arr, initializer=True)
