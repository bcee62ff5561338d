"""ctypes front end of the CPU oracle (``libovk_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The product
package never imports this module.

Each wrapper takes and returns numpy arrays; dtype codes are the reference's
``ElementType`` values (FLOAT=1, UINT8=2, INT8=3, INT32=6, FLOAT16=10,
crates/onnx-vulkan-core/src/graph.rs:13-41).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

FLOAT, UINT8, INT8, INT32, FLOAT16 = 1, 2, 3, 6, 10
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    """Compile the oracle with its Makefile (gcc, no GPU needed)."""
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return os.path.join(_HERE, "libovk_oracle.so")


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libovk_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_num_threads.restype = C.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _dt(a: np.ndarray) -> int:
    return {np.dtype(np.float32): FLOAT, np.dtype(np.float16): FLOAT16}[a.dtype]


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def n_blocks(k: int, block_size: int) -> int:
    return -(-k // block_size)


def pack_nibbles(nib: np.ndarray, block_size: int) -> np.ndarray:
    """``[N, K]`` values 0..15 -> ``[N, n_blocks, block_size/2]`` bytes, element
    2i in the low nibble (tests/matmul_nbits.rs:19-34)."""
    n, k = nib.shape
    nb = n_blocks(k, block_size)
    full = np.zeros((n, nb * block_size), dtype=np.uint8)
    full[:, :k] = nib
    return (full[:, 0::2] | (full[:, 1::2] << 4)).reshape(n, nb, block_size // 2)


def pack_zero_points(zp: np.ndarray) -> np.ndarray:
    """``[N, n_blocks]`` values 0..15 -> ``[N, ceil(n_blocks/2)]`` bytes, low
    nibble first (tests/matmul_nbits.rs:36-46)."""
    n, nb = zp.shape
    full = np.zeros((n, (nb + 1) // 2 * 2), dtype=np.uint8)
    full[:, :nb] = zp
    return full[:, 0::2] | (full[:, 1::2] << 4)


def matmul_nbits(a, b_packed, scales, zp_packed, k, n, block_size, out_dtype=None):
    a = np.ascontiguousarray(a)
    m = a.size // k
    out_dtype = np.dtype(out_dtype or a.dtype)
    y = np.empty((m, n), dtype=out_dtype)
    b = np.ascontiguousarray(b_packed, dtype=np.uint8)
    s = np.ascontiguousarray(scales)
    z = None if zp_packed is None else np.ascontiguousarray(zp_packed, dtype=np.uint8)
    rc = lib().orc_matmul_nbits(
        _p(a), _dt(a), C.c_int64(m), C.c_int64(k), C.c_int64(n), C.c_int64(block_size),
        _p(b), _p(s), _dt(s), _p(z), _p(y), _dt(y))
    if rc:
        raise ValueError(f"orc_matmul_nbits: status {rc}")
    return y


def matmul_nbits_f32_shader_order(a, b_packed, scales, zp_packed, k, n, block_size):
    a = np.ascontiguousarray(a, dtype=np.float32)
    m = a.size // k
    y = np.empty((m, n), dtype=np.float32)
    b = np.ascontiguousarray(b_packed, dtype=np.uint8)
    s = np.ascontiguousarray(scales, dtype=np.float32)
    z = None if zp_packed is None else np.ascontiguousarray(zp_packed, dtype=np.uint8)
    rc = lib().orc_matmul_nbits_f32_shader_order(
        _p(a), C.c_int64(m), C.c_int64(k), C.c_int64(n), C.c_int64(block_size),
        _p(b), _p(s), _p(z), _p(y))
    if rc:
        raise ValueError(f"orc_matmul_nbits_f32_shader_order: status {rc}")
    return y


def dynamic_quantize(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=np.uint8)
    scale = C.c_float(0)
    zp = C.c_uint8(0)
    lib().orc_dynamic_quantize(_p(x), C.c_size_t(x.size), _p(y), C.byref(scale), C.byref(zp))
    return y, np.float32(scale.value), int(zp.value)


def decomposed_gelu(x, divisor, offset, factor, factor_first=False):
    """DecomposedGelu (shaders/elementwise.rs:71-118): erf(x / divisor) + offset, times x and factor."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_decomposed_gelu(_p(x), C.c_size_t(x.size), C.c_float(divisor), C.c_float(offset), C.c_float(factor),
                              C.c_int(int(factor_first)), _p(out))
    return out


def decomposed_gelu_quantize(x, divisor, offset, factor, factor_first=False):
    """DynamicQuantizeLinear(DecomposedGelu(x)) (interp.rs:9125): the two nodes, one after the other."""
    return dynamic_quantize(decomposed_gelu(x, divisor, offset, factor, factor_first))


def erf_approx(x: float) -> float:
    f = lib().orc_erf_approx
    f.restype, f.argtypes = C.c_float, [C.c_float]
    return float(f(C.c_float(x)))


def exp_ieee(x: float) -> float:
    f = lib().orc_exp_ieee
    f.restype, f.argtypes = C.c_float, [C.c_float]
    return float(f(C.c_float(x)))


def _bytes(a):
    a = np.ascontiguousarray(a)
    assert a.dtype in (np.uint8, np.int8), a.dtype
    return a, int(a.dtype == np.int8)


def matmul_integer(a, b, a_zp=0, b_zp=0):
    a, a_signed = _bytes(a)
    b, b_signed = _bytes(b)
    k, n = b.shape
    m = a.size // k if k else 0
    out = np.empty(a.shape[:-1] + (n,), dtype=np.int32)
    rc = lib().orc_matmul_integer(
        _p(a), a_signed, _p(b), b_signed, C.c_int64(m), C.c_int64(k), C.c_int64(n),
        C.c_int32(int(a_zp)), C.c_int32(int(b_zp)), _p(out))
    if rc == 2:
        raise OverflowError("MatMulInteger: i32 overflow")
    if rc:
        raise RuntimeError(f"orc_matmul_integer: status {rc}")
    return out


def scale_bias_epilogue(acc, scale, scale_step, bias, bias_step, product=None, product_step=0,
                        relu=False, want_range=False):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    n = acc.shape[-1]
    m = acc.size // n
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    bias = np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
    if product is not None:
        product = np.ascontiguousarray(product, dtype=np.float32).reshape(-1)
    out = np.empty(acc.shape, dtype=np.float32)
    rng = np.zeros(2, dtype=np.float32)
    lib().orc_scale_bias_epilogue(
        _p(acc), C.c_int64(m), C.c_int64(n), _p(scale), scale_step, _p(product), product_step,
        _p(bias), bias_step, int(relu), _p(out), _p(rng) if want_range else None)
    return (out, rng) if want_range else out


class ConvGeom(C.Structure):
    _fields_ = [(name, C.c_int64) for name in (
        "n", "c_in", "c_out", "group", "gsi", "h_in", "w_in", "h_out", "w_out",
        "kh", "kw", "sh", "sw", "dh", "dw", "phb", "phe", "pwb", "pwe")]


_AUTO_PAD = {"NOTSET": 0, "VALID": 1, "SAME_UPPER": 2, "SAME_LOWER": 3}


def conv_geometry(x_shape, w_shape, strides=(1, 1), dilations=(1, 1), pads=(0, 0, 0, 0),
                  auto_pad="NOTSET", group=1) -> ConvGeom:
    """pads = (h_begin, w_begin, h_end, w_end), the ONNX order."""
    g = ConvGeom()
    arr = lambda v: (C.c_int64 * len(v))(*[int(i) for i in v])
    rc = lib().orc_conv_geometry(arr(x_shape), arr(w_shape), arr(strides), arr(dilations),
                                 arr(pads), _AUTO_PAD[auto_pad], C.c_int64(group), C.byref(g))
    if rc:
        raise ValueError("conv: degenerate output shape")
    return g


def conv_integer(x, w, x_zp=0, w_zp=0, **geom):
    x, x_signed = _bytes(x)
    w, w_signed = _bytes(w)
    g = conv_geometry(x.shape, w.shape, **geom)
    out = np.empty((g.n, g.c_out, g.h_out, g.w_out), dtype=np.int32)
    lib().orc_conv_integer(_p(x), x_signed, _p(w), w_signed, C.byref(g),
                           C.c_int32(int(x_zp)), C.c_int32(int(w_zp)), _p(out))
    return out


def requantize_ratio(x_scale, w_scale, y_scale):
    w = np.ascontiguousarray(w_scale, dtype=np.float32).reshape(-1)
    ratio = np.empty_like(w)
    lib().orc_requantize_ratio(C.c_float(x_scale), _p(w), C.c_size_t(w.size),
                               C.c_float(y_scale), _p(ratio))
    return ratio


def requantize(acc, inner, ratio, y_zp, bias=None, out_signed=False):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    ratio = np.ascontiguousarray(ratio, dtype=np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.int32)
    out = np.empty(acc.shape, dtype=np.uint8)
    lib().orc_requantize(_p(acc), C.c_size_t(acc.size), C.c_size_t(inner),
                         C.c_size_t(ratio.size), _p(bias), _p(ratio), C.c_int32(int(y_zp)),
                         int(out_signed), _p(out))
    return out.view(np.int8) if out_signed else out


def qlinear_conv(x, x_scale, x_zp, w, w_scale, w_zp, y_scale, y_zp, bias=None, out_signed=False,
                 **geom):
    """QLinearConv = ConvInteger + requantize (src/interp.rs:4796-4837)."""
    acc = conv_integer(x, w, x_zp, w_zp, **geom)
    ratio = requantize_ratio(x_scale, w_scale, y_scale)
    if ratio.size == 1:
        ratio = np.repeat(ratio, acc.shape[1])
    return requantize(acc, acc.shape[2] * acc.shape[3], ratio, y_zp, bias, out_signed)


def gather_block_quantized(table, indices, scales, zero_points, block_size):
    """GatherBlockQuantized (src/interp.rs:2874-2990): f32 rows of a 4-bit table."""
    table = np.ascontiguousarray(table, dtype=np.uint8)
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    scales = np.ascontiguousarray(scales)
    rows, cols = table.shape[0], table.shape[1] * 2
    if zero_points is not None:
        zero_points = np.ascontiguousarray(zero_points, dtype=np.uint8)
    out = np.empty(idx.shape + (cols,), dtype=np.float32)
    rc = lib().orc_gather_block_quantized(_p(table), _p(idx), C.c_size_t(idx.size), _p(scales), _dt(scales),
                                          _p(zero_points), C.c_int64(rows), C.c_int64(cols),
                                          C.c_int64(block_size), _p(out))
    if rc:
        raise IndexError(f"GatherBlockQuantized: an index falls outside the {rows}-row table")
    return out


def argmax(x, axis=-1):
    """First-occurrence ArgMax over one axis with the device kernels' candidate rule."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    axis = axis % x.ndim
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    c = x.shape[axis]
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    out = np.empty(x.shape[:axis] + x.shape[axis + 1:], dtype=np.int64)
    lib().orc_argmax(_p(x), C.c_int64(outer), C.c_int64(c), C.c_int64(inner), _p(out))
    return out


def _codes(a):
    a = np.ascontiguousarray(a)
    assert a.dtype in (np.uint8, np.int8), a.dtype
    return a, int(a.dtype == np.int8)


def _i64s(v):
    return (C.c_int64 * max(len(v), 1))(*[int(i) for i in v])


def qlinear_add(a, a_scale, a_zp, b, b_scale, b_zp, c_scale, c_zp):
    """QLinearAdd with MLAS's rounding and ORT's operand exchange (src/interp.rs:4878-4962)."""
    a, signed = _codes(a)
    b, _ = _codes(b)
    out = np.empty(np.broadcast_shapes(a.shape, b.shape), dtype=a.dtype)
    rc = lib().orc_qlinear_add(_p(a), _i64s(a.shape), a.ndim, C.c_float(a_scale), C.c_int32(int(a_zp)),
                               _p(b), _i64s(b.shape), b.ndim, C.c_float(b_scale), C.c_int32(int(b_zp)),
                               C.c_float(c_scale), C.c_int32(int(c_zp)), signed, _p(out))
    if rc:
        raise ValueError("QLinearAdd: shapes do not broadcast")
    return out


def maxpool_q(x, kernel, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1)):
    x, signed = _codes(x)
    n, c, h, w = x.shape
    ho = (h + pads[0] + pads[2] - (dilations[0] * (kernel[0] - 1) + 1)) // strides[0] + 1
    wo = (w + pads[1] + pads[3] - (dilations[1] * (kernel[1] - 1) + 1)) // strides[1] + 1
    out = np.empty((n, c, ho, wo), dtype=x.dtype)
    lib().orc_maxpool_q(_p(x), signed, C.c_int64(n), C.c_int64(c), C.c_int64(h), C.c_int64(w), _i64s(kernel),
                        _i64s(strides), _i64s(pads), _i64s(dilations), _p(out))
    return out


def _qdq_layout(shape, scale, axis):
    if scale.size <= 1:
        return 1, 1
    axis = axis % len(shape)
    return max(int(np.prod(shape[axis + 1:], dtype=np.int64)), 1), scale.size


def quantize_linear(x, scale, zero_point=None, axis=1, signed=False):
    x = np.ascontiguousarray(x, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    if zero_point is not None:
        zero_point, signed = _codes(np.asarray(zero_point).reshape(-1))
    inner, axis_len = _qdq_layout(x.shape, scale, axis)
    out = np.empty(x.shape, dtype=np.int8 if signed else np.uint8)
    lib().orc_quantize_linear(_p(x), C.c_int64(x.size), C.c_int64(inner), C.c_int64(axis_len), _p(scale),
                              _p(zero_point), int(signed), _p(out))
    return out


def dequantize_linear(x, scale, zero_point=None, axis=1):
    x = np.ascontiguousarray(x)
    kind = {np.dtype(np.uint8): 0, np.dtype(np.int8): 1, np.dtype(np.int32): 2}[x.dtype]
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    if zero_point is not None:
        zero_point = np.ascontiguousarray(np.asarray(zero_point, dtype=x.dtype).reshape(-1))
    inner, axis_len = _qdq_layout(x.shape, scale, axis)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_dequantize_linear(_p(x), kind, C.c_int64(x.size), C.c_int64(inner), C.c_int64(axis_len), _p(scale),
                                _p(zero_point), _p(out))
    return out


def qlinear_global_average_pool(x, x_scale, x_zp, y_scale, y_zp):
    x, signed = _codes(x)
    n, c = x.shape[:2]
    hw = int(np.prod(x.shape[2:], dtype=np.int64))
    out = np.empty((n, c) + (1,) * (x.ndim - 2), dtype=x.dtype)
    lib().orc_qlinear_global_average_pool(_p(x), signed, C.c_int64(n * c), C.c_int64(hw), C.c_float(x_scale),
                                          C.c_int32(int(x_zp)), C.c_float(y_scale), C.c_int32(int(y_zp)), _p(out))
    return out
