"""A tiny protobuf encoder, just enough to write the ``.onnx`` fixtures of the reader's tests."""
import struct

import numpy as np

_CODES = {np.dtype(np.float32): 1, np.dtype(np.uint8): 2, np.dtype(np.int8): 3, np.dtype(np.int32): 6,
          np.dtype(np.int64): 7, np.dtype(np.float16): 10}


def varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def field(number, wire, payload):
    return varint(number << 3 | wire) + payload


def blob(number, data):
    return field(number, 2, varint(len(data)) + data)


def tensor(name, arr, raw=True):
    arr = np.ascontiguousarray(arr)
    out = b"".join(field(1, 0, varint(d)) for d in arr.shape) + field(2, 0, varint(_CODES[arr.dtype]))
    if raw:
        out += blob(9, arr.tobytes())
    elif arr.dtype == np.float32:
        out += blob(4, arr.tobytes())
    elif arr.dtype == np.int64:
        out += blob(7, b"".join(varint(int(v)) for v in arr.reshape(-1)))
    elif arr.dtype == np.float16:
        out += blob(5, b"".join(varint(int(v)) for v in arr.reshape(-1).view(np.uint16)))
    else:
        out += blob(5, b"".join(varint(int(v)) for v in arr.reshape(-1)))
    return out + blob(8, name.encode())


def attribute(name, value):
    out = blob(1, name.encode())
    if isinstance(value, int):
        return out + field(3, 0, varint(value)) + field(20, 0, varint(2))
    if isinstance(value, float):
        return out + field(2, 5, struct.pack("<f", value)) + field(20, 0, varint(1))
    if isinstance(value, str):
        return out + blob(4, value.encode()) + field(20, 0, varint(3))
    return out + b"".join(field(8, 0, varint(int(v))) for v in value) + field(20, 0, varint(7))


def node(op, inputs, outputs, domain="", name="", **attrs):
    out = b"".join(blob(1, i.encode()) for i in inputs) + b"".join(blob(2, o.encode()) for o in outputs)
    out += blob(3, name.encode()) + blob(4, op.encode())
    out += b"".join(blob(5, attribute(k, v)) for k, v in attrs.items())
    return out + (blob(7, domain.encode()) if domain else b"")


def model(nodes, initializers, inputs=(), outputs=(), raw=True):
    graph = b"".join(blob(1, n) for n in nodes) + blob(2, b"g")
    graph += b"".join(blob(5, tensor(k, v, raw)) for k, v in initializers.items())
    graph += b"".join(blob(11, blob(1, n.encode())) for n in inputs)
    graph += b"".join(blob(12, blob(1, n.encode())) for n in outputs)
    opset = blob(8, blob(1, b"") + field(2, 0, varint(21))) + blob(8, blob(1, b"com.microsoft") + field(2, 0, varint(1)))
    return field(1, 0, varint(10)) + blob(2, b"ovk-tests") + blob(7, graph) + opset
