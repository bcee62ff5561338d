"""ctypes view of ``libovk_host.so``: the C++ node-level layer (``host/interp.cpp``).

That layer is the counterpart of the reference's operator functions
(crates/onnx-vulkan-core/src/interp.rs: ``is_implemented_node`` :338,
``unsupported_quantization`` :781, ``exec_dispatch`` :1071) for the quantized
matrix-product path: a node with named inputs, outputs and attributes runs
against an environment of named tensors, weights are prepared once per
initializer name.  This module only lets tests and Python hosts drive it; the
logic is in C++ and the arithmetic in ``libovk_cuda.so``.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import FLOAT, FLOAT16, INT8, INT32, INT64, UINT8, OvkError

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libovk_host.so")

_P, _I32, _I64, _SZ, _S = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_char_p
SIGNATURES = {
    "ovkh_env_create": (_I32, [_I32, C.POINTER(_P)]),
    "ovkh_env_destroy": (None, [_P]),
    "ovkh_last_error": (_S, [_P]),
    "ovkh_last_kernel": (_S, [_P]),
    "ovkh_set": (_I32, [_P, _S, _I32, C.POINTER(_I64), _I32, _P, _SZ, _I32]),
    "ovkh_info": (_I32, [_P, _S, C.POINTER(_I32), C.POINTER(_I32), C.POINTER(_I64), C.POINTER(_SZ)]),
    "ovkh_get": (_I32, [_P, _S, _P, _SZ]),
    "ovkh_node_create": (_P, [_S, _S, _S]),
    "ovkh_node_destroy": (None, [_P]),
    "ovkh_node_input": (None, [_P, _S]),
    "ovkh_node_output": (None, [_P, _S]),
    "ovkh_node_attr_int": (None, [_P, _S, _I64]),
    "ovkh_node_attr_ints": (None, [_P, _S, C.POINTER(_I64), _I32]),
    "ovkh_node_attr_str": (None, [_P, _S, _S]),
    "ovkh_is_implemented": (_I32, [_P]),
    "ovkh_unsupported_quantization": (_I32, [_P, _P]),
    "ovkh_execute": (_I32, [_P, _P]),
}

_NP = {FLOAT: np.float32, UINT8: np.uint8, INT8: np.int8, INT32: np.int32, INT64: np.int64, FLOAT16: np.float16}
_CODE = {np.dtype(v): k for k, v in _NP.items()}
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python onnx-vulkan-rs_b200/build.py`")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


class Node:
    """NodeIr (crates/onnx-vulkan-core/src/graph.rs:197): op, inputs ("" = absent), outputs, attributes."""

    def __init__(self, op: str, inputs, outputs, domain: str = "", name: str = "", **attrs):
        self._h = lib().ovkh_node_create(op.encode(), domain.encode(), name.encode())
        for i in inputs:
            lib().ovkh_node_input(self._h, i.encode())
        for o in outputs:
            lib().ovkh_node_output(self._h, o.encode())
        for key, v in attrs.items():
            if isinstance(v, str):
                lib().ovkh_node_attr_str(self._h, key.encode(), v.encode())
            elif isinstance(v, (list, tuple)):
                arr = (_I64 * len(v))(*v)
                lib().ovkh_node_attr_ints(self._h, key.encode(), arr, len(v))
            else:
                lib().ovkh_node_attr_int(self._h, key.encode(), int(v))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ovkh_node_destroy(self._h)
            self._h = None

    @property
    def implemented(self) -> bool:
        return bool(lib().ovkh_is_implemented(self._h))


class Env:
    """ExecutionEnv (crates/onnx-vulkan-core/src/execution.rs:15) on one CUDA device."""

    def __init__(self, device: int = 0):
        h = _P()
        rc = lib().ovkh_env_create(device, C.byref(h))
        if rc:
            raise OvkError(rc, "cannot create a context on this device")
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().ovkh_env_destroy(self._h)
            self._h = None

    __del__ = close

    def _check(self, rc: int):
        if rc:
            raise OvkError(rc, lib().ovkh_last_error(self._h).decode())

    def set(self, name: str, array, initializer: bool = False):
        a = np.ascontiguousarray(array)
        shape = (_I64 * max(a.ndim, 1))(*a.shape)
        self._check(lib().ovkh_set(self._h, name.encode(), _CODE[a.dtype], shape, a.ndim, a.ctypes.data, a.nbytes,
                                   int(initializer)))

    def host(self, name: str) -> np.ndarray:
        dtype, ndim, nbytes = _I32(), _I32(), _SZ()
        shape = (_I64 * 8)()
        self._check(lib().ovkh_info(self._h, name.encode(), C.byref(dtype), C.byref(ndim), shape, C.byref(nbytes)))
        out = np.empty(tuple(shape[i] for i in range(ndim.value)), dtype=_NP[dtype.value])
        assert out.nbytes == nbytes.value
        if out.nbytes:
            self._check(lib().ovkh_get(self._h, name.encode(), out.ctypes.data, out.nbytes))
        return out

    def unsupported_quantization(self, node: Node) -> str | None:
        if lib().ovkh_unsupported_quantization(self._h, node._h):
            return lib().ovkh_last_error(self._h).decode()
        return None

    def execute(self, node: Node):
        self._check(lib().ovkh_execute(self._h, node._h))

    @property
    def last_kernel(self) -> str:
        return lib().ovkh_last_kernel(self._h).decode()
