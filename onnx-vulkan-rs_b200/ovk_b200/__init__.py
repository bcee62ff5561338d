"""ctypes binding of ``libovk_cuda.so`` - the C ABI declared in ``include/ovk_cuda.h``.

The library is the product; this module only loads it, declares the
signatures and wraps device memory held in torch CUDA tensors (torch is the
allocator and the stream provider here, nothing more).  There is no fallback:
if the library is missing or was not built, importing the ops fails loudly.

The wrappers mirror the reference's operator functions
(crates/onnx-vulkan-core/src/interp.rs): ``matmul_nbits`` (:6429),
``dynamic_quantize`` (:1945), ``matmul_integer`` (:2090),
``matmul_integer_scale_bias`` (:2405), ``qlinear_matmul`` (:4845),
``conv_integer`` (:4421), ``qlinear_conv`` (:4796).
"""
from __future__ import annotations

import ctypes as C
import os

FLOAT, UINT8, INT8, INT32, INT64, FLOAT16 = 1, 2, 3, 6, 7, 10
OK, INVALID_ARGUMENT, UNSUPPORTED, BACKEND, TIMEOUT = 0, 1, 2, 3, 4
EPILOGUE_RELU, EPILOGUE_RANGE = 1, 2
NBITS_NO_DECODE_COPY = 1
COMM_HANDLE_BYTES = 64

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libovk_cuda.so")


class OvkError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[ovk status {status}] {message}")
        self.status = status
        self.message = message


class ConvParams(C.Structure):
    _fields_ = [("n", C.c_int64), ("c_in", C.c_int64), ("h", C.c_int64), ("w", C.c_int64),
                ("pads", C.c_int64 * 4), ("strides", C.c_int64 * 2), ("dilations", C.c_int64 * 2)]


_lib = None

# name -> (restype, argtypes); every symbol ovk_cuda.h declares
_P, _I32, _I64, _U32, _SZ = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_size_t
SIGNATURES = {
    "ovk_ctx_create": (_I32, [_I32, _P, C.POINTER(_P)]),
    "ovk_ctx_destroy": (None, [_P]),
    "ovk_last_error": (C.c_char_p, [_P]),
    "ovk_last_kernel": (C.c_char_p, [_P]),
    "ovk_launch_count": (C.c_uint64, [_P]),
    "ovk_stream": (_P, [_P]),
    "ovk_workspace_bytes": (_SZ, [_P]),
    "ovk_selftest_device_timeout": (_I32, [_P]),
    "ovk_probe_mma_rate": (_I32, [_P, _I32, C.POINTER(C.c_double)]),
    "ovk_flush": (_I32, [_P]),
    "ovk_alloc": (_I32, [_P, _SZ, C.POINTER(_P)]),
    "ovk_free": (_I32, [_P, _P]),
    "ovk_upload": (_I32, [_P, _P, _SZ, _P, _SZ]),
    "ovk_download": (_I32, [_P, _P, _SZ, _P, _SZ]),
    "ovk_fill": (_I32, [_P, _P, _SZ, _SZ, _U32]),
    "ovk_timer_start": (_I32, [_P]),
    "ovk_timer_stop": (_I32, [_P, C.POINTER(C.c_float)]),
    "ovk_nbits_prepack": (_I32, [_P, _P, _P, _I32, _P, _I64, _I64, _I64, _I64, _U32, C.POINTER(_P)]),
    "ovk_nbits_weight_destroy": (None, [_P, _P]),
    "ovk_matmul_nbits": (_I32, [_P, _P, _P, _I32, _I64, _P, _I32]),
    "ovk_matmul_nbits_group": (_I32, [_P, _I32, C.POINTER(_P), _P, _I32, _I64, C.POINTER(_P), _I32]),
    "ovk_comm_flag_bytes": (_SZ, []),
    "ovk_comm_alloc": (_I32, [_P, _SZ, C.POINTER(_P)]),
    "ovk_comm_export": (_I32, [_P, _P, _P]),
    "ovk_comm_import": (_I32, [_P, _P, C.POINTER(_P)]),
    "ovk_comm_release": (_I32, [_P, _P]),
    "ovk_comm_init": (_I32, [_P, _I32, _I32, C.POINTER(_P)]),
    "ovk_comm_set_timeout_ms": (_I32, [_P, _I32]),
    "ovk_comm_barrier": (_I32, [_P]),
    "ovk_allgather_cols": (_I32, [_P, _P, _I32, _I64, _I64, _I64, _I64, C.POINTER(_P)]),
    "ovk_matmul_nbits_nsplit": (_I32, [_P, _P, _P, _I32, _I64, _I64, _I64, C.POINTER(_P), _I32]),
    "ovk_matmul_nbits_nsplit_multicast": (_I32, [_P, _P, _P, _I32, _I64, _I64, _I64, C.POINTER(_P), _P, _I32]),
    "ovk_allgather_cols_multicast": (_I32, [_P, _P, _I32, _I64, _I64, _I64, _I64, C.POINTER(_P), _P]),
    "ovk_dynamic_quantize": (_I32, [_P, _P, _I64, _P, _P, _P]),
    "ovk_dynamic_quantize_folded": (_I32, [_P, _P, _I64, _P, _P, _P, _P]),
    "ovk_decomposed_gelu": (_I32, [_P, _P, _I64, C.c_float, C.c_float, C.c_float, _I32, _P]),
    "ovk_decomposed_gelu_quantize": (_I32, [_P, _P, _I64, C.c_float, C.c_float, C.c_float, _I32, _P, _P, _P]),
    "ovk_mmi_prepack": (_I32, [_P, _P, _I32, _I64, _I64, C.POINTER(_P)]),
    "ovk_mmi_weight_destroy": (None, [_P, _P]),
    "ovk_matmul_integer": (_I32, [_P, _P, _P, _I32, _I64, _P, _P, _P]),
    "ovk_matmul_integer_static_scratch": (_I32, [_P, _P, _P, _I32, _I64, _P, _P, _P]),
    "ovk_matmul_integer_scale_bias": (_I32, [_P, _P, _P, _I32, _I64, _P, _P, _P, _I32, _P, _I32, _P,
                                             _I32, _U32, _P, _P]),
    "ovk_integer_scale_bias_unfused": (_I32, [_P, _P, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _U32, _P]),
    "ovk_matmul_integer_group": (_I32, [_P, _I32, C.POINTER(_P), _P, _I32, _I64, _P, _P, C.POINTER(_P)]),
    "ovk_matmul_integer_scale_bias_group": (_I32, [_P, _I32, C.POINTER(_P), _P, _I32, _I64, _P, _P, C.POINTER(_P), _I32,
                                                   _P, _I32, C.POINTER(_P), _I32, _U32, C.POINTER(_P)]),
    "ovk_qlinear_matmul": (_I32, [_P, _P, _P, _I32, _I64, _P, _P, _P, _I64, _I32, _I32, _P]),
    "ovk_qconv_prepack": (_I32, [_P, _P, _I32, _I64, _I64, _I64, _I64, _I64, C.POINTER(_P)]),
    "ovk_qconv_weight_destroy": (None, [_P, _P]),
    "ovk_conv_output_shape": (_I32, [_P, C.POINTER(ConvParams), C.POINTER(_I64), C.POINTER(_I64)]),
    "ovk_conv_integer": (_I32, [_P, _P, _P, _I32, C.POINTER(ConvParams), _I32, _I32, _P]),
    "ovk_conv_integer_scale_bias": (_I32, [_P, _P, _P, _I32, C.POINTER(ConvParams), _I32, _I32, _P, _I32, _P, _I32,
                                           _P, _I32, _U32, _P, _P]),
    "ovk_qlinear_conv": (_I32, [_P, _P, _P, _I32, C.POINTER(ConvParams), _I32, _I32, _P, _P, _I32, _I32, _P]),
    "ovk_qlinear_conv_layout": (_I32, [_P, _P, _P, _I32, _I32, C.POINTER(ConvParams), _I32, _I32, _P, _P, _I32, _I32, _P,
                                       _I32, C.POINTER(_I64)]),
    "ovk_nchw_to_padded_nhwc": (_I32, [_P, _P, _I64, _I64, _I64, _I64, C.POINTER(_I64), _I32, _P]),
    "ovk_padded_nhwc_to_nchw": (_I32, [_P, _P, _I64, _I64, _I64, _I64, C.POINTER(_I64), _P]),
    "ovk_requantize": (_I32, [_P, _P, _I64, _I64, _I64, _P, _P, _I32, _I32, _P]),
    "ovk_gather_block_quantized": (_I32, [_P, _P, _P, _I32, _P, _I64, _I64, _I64, _I64, _P, _I32, _I32, _I64, _P, _I32]),
    "ovk_argmax": (_I32, [_P, _P, _I32, _I64, _I64, _I64, _P]),
    "ovk_qlinear_add": (_I32, [_P, _P, C.POINTER(_I64), _I32, C.c_float, _I32, _P, C.POINTER(_I64), _I32, C.c_float, _I32,
                               C.c_float, _I32, _I32, _P, C.POINTER(_I64), C.POINTER(_I32)]),
    "ovk_maxpool_q": (_I32, [_P, _P, _I32, _I64, _I64, _I64, _I64, C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I64),
                             C.POINTER(_I64), _P, C.POINTER(_I64), C.POINTER(_I64)]),
    "ovk_quantize_linear": (_I32, [_P, _P, _I64, _I64, _I64, _P, _P, _I32, _P]),
    "ovk_dequantize_linear": (_I32, [_P, _P, _I32, _I64, _I64, _I64, _P, _P, _P]),
    "ovk_qlinear_global_average_pool": (_I32, [_P, _P, _I32, _I64, _I64, _I64, C.c_float, _I32, C.c_float, _I32, _P]),
}


def lib() -> C.CDLL:
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OvkError(BACKEND, f"{LIB_PATH} is missing: run `python onnx-vulkan-rs_b200/build.py` "
                                    "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def _ptr(t):
    """Device pointer of a torch tensor, an int address, or None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda and t.is_contiguous(), "device tensors must be contiguous CUDA tensors"
    return t.data_ptr()


def _dtype_code(t) -> int:
    import torch
    return {torch.float32: FLOAT, torch.float16: FLOAT16, torch.uint8: UINT8, torch.int8: INT8,
            torch.int32: INT32, torch.int64: INT64}[t.dtype]


class Context:
    """One device, one in-order stream (VkContext, crates/vk-compute/src/context.rs:257)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        import torch
        if not torch.cuda.is_available():
            raise OvkError(BACKEND, "no CUDA device: the quantized-matmul path has no CPU fallback")
        h = _P()
        if stream is None:
            # share torch's current stream so torch allocations, copies and
            # CUDA events are ordered with the kernels
            with torch.cuda.device(device):
                stream = torch.cuda.current_stream().cuda_stream
            if stream == 0:
                stream = 1  # cudaStreamLegacy: the default stream by its explicit handle
        rc = lib().ovk_ctx_create(device, _P(stream) if stream else None, C.byref(h))
        if rc:
            raise OvkError(rc, lib().ovk_last_error(None).decode())
        self.h = h
        self.device = device

    def check(self, rc: int):
        if rc:
            raise OvkError(rc, lib().ovk_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            lib().ovk_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def flush(self):
        self.check(lib().ovk_flush(self.h))

    @property
    def last_kernel(self) -> str:
        return lib().ovk_last_kernel(self.h).decode()

    @property
    def launches(self) -> int:
        return int(lib().ovk_launch_count(self.h))

    @property
    def workspace_bytes(self) -> int:
        return int(lib().ovk_workspace_bytes(self.h))

    def probe_mma_rate(self, dtype=INT8) -> float:
        """Multiply-accumulates per clock per SM of back-to-back tcgen05.mma (kind::i8 or kind::f16)."""
        v = C.c_double()
        self.check(lib().ovk_probe_mma_rate(self.h, dtype, C.byref(v)))
        return v.value

    def selftest_device_timeout(self):
        """Enqueues the wait that is meant to run out; the next flush raises with status TIMEOUT."""
        self.check(lib().ovk_selftest_device_timeout(self.h))

    # ---------------------------------------------------------- MatMulNBits
    def nbits_prepack(self, b, scales, zero_points, n, k, block_size, bits=4, flags=0):
        return NBitsWeight(self, b, scales, zero_points, n, k, block_size, bits, flags)

    def matmul_nbits(self, w: "NBitsWeight", a, out=None, out_dtype=None):
        import torch
        m = a.numel() // w.k
        if a.numel() != m * w.k or (a.dim() and a.shape[-1] != w.k):
            raise OvkError(INVALID_ARGUMENT, f"MatMulNBits: A's last dimension {tuple(a.shape)} disagrees with K={w.k}")
        if out is None:
            out = torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=out_dtype or a.dtype, device=a.device)
        self.check(lib().ovk_matmul_nbits(self.h, w.h, _ptr(a), _dtype_code(a), m, _ptr(out), _dtype_code(out)))
        return out

    def matmul_nbits_group(self, ws, a, outs=None, out_dtype=None):
        """Several weights over the same activations (q|k|v, gate|up): one launch where the decode kernel
        applies and the weights share their tile shape, one call per weight otherwise."""
        import torch
        m = a.numel() // ws[0].k
        if outs is None:
            outs = [torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=out_dtype or a.dtype, device=a.device) for w in ws]
        wp = (_P * len(ws))(*[w.h for w in ws])
        yp = (_P * len(ws))(*[_ptr(o) for o in outs])
        self.check(lib().ovk_matmul_nbits_group(self.h, len(ws), wp, _ptr(a), _dtype_code(a), m, yp, _dtype_code(outs[0])))
        return outs

    # --------------------------------------------- several GPUs of one box
    def comm_alloc(self, nbytes: int) -> int:
        """A zero-filled device buffer that other ranks may map (ovk_comm_alloc); returns its address."""
        p = _P()
        self.check(lib().ovk_comm_alloc(self.h, nbytes, C.byref(p)))
        return p.value

    def comm_export(self, ptr: int) -> bytes:
        buf = C.create_string_buffer(COMM_HANDLE_BYTES)
        self.check(lib().ovk_comm_export(self.h, _P(ptr), buf))
        return buf.raw

    def comm_import(self, handle: bytes) -> int:
        p = _P()
        self.check(lib().ovk_comm_import(self.h, C.c_char_p(handle), C.byref(p)))
        return p.value

    def comm_release(self, ptr: int):
        self.check(lib().ovk_comm_release(self.h, _P(ptr)))

    def comm_init(self, rank: int, world: int, flag_blocks):
        arr = (_P * world)(*[int(b) for b in flag_blocks])
        self.check(lib().ovk_comm_init(self.h, rank, world, arr))
        self.rank, self.world = rank, world

    def comm_set_timeout_ms(self, ms: int):
        self.check(lib().ovk_comm_set_timeout_ms(self.h, int(ms)))

    def comm_barrier(self):
        self.check(lib().ovk_comm_barrier(self.h))

    def allgather_cols(self, y_shard, m, n_shard, col0, n_total, y_peers, dtype=FLOAT16, multicast=None):
        """y_shard: a [m, n_shard] tensor, or None when the block already sits in this rank's matrix.
        multicast: a multicast mapping of the ranks' matrices (one store reaches every rank), or None."""
        arr = (_P * len(y_peers))(*[int(p) for p in y_peers])
        self.check(lib().ovk_allgather_cols_multicast(self.h, _ptr(y_shard),
                                                      dtype if y_shard is None else _dtype_code(y_shard),
                                                      m, n_shard, col0, n_total, arr, _P(multicast) if multicast else None))

    def matmul_nbits_nsplit(self, w: "NBitsWeight", a, col0, n_total, y_peers, y_dtype=FLOAT16, multicast=None):
        """This rank's columns [col0, col0 + w.n) of Y = A x dequant(B), stored into every rank's matrix."""
        m = a.numel() // w.k
        arr = (_P * len(y_peers))(*[int(p) for p in y_peers])
        self.check(lib().ovk_matmul_nbits_nsplit_multicast(self.h, w.h, _ptr(a), _dtype_code(a), m, col0, n_total, arr,
                                                           _P(multicast) if multicast else None, y_dtype))

    # ------------------------------------------------- DynamicQuantizeLinear
    def dynamic_quantize(self, x, folded_range=None, out=None):
        """interp::dynamic_quantize (interp.rs:1945).  `folded_range`: the four-u32 slot the producer of x
        folded its range into (then only the quantize pass runs); `out`: (y, scale, zp) tensors to reuse."""
        import torch
        if out is None:
            out = (torch.empty(x.shape, dtype=torch.uint8, device=x.device),
                   torch.empty((), dtype=torch.float32, device=x.device),
                   torch.empty((), dtype=torch.uint8, device=x.device))
        y, scale, zp = out
        if folded_range is None:
            self.check(lib().ovk_dynamic_quantize(self.h, _ptr(x), x.numel(), _ptr(y), _ptr(scale), _ptr(zp)))
        else:
            self.check(lib().ovk_dynamic_quantize_folded(self.h, _ptr(x), x.numel(), _ptr(folded_range), _ptr(y),
                                                         _ptr(scale), _ptr(zp)))
        return y, scale, zp

    def decomposed_gelu(self, x, divisor, offset, factor, factor_first=False):
        """interp::decomposed_gelu (interp.rs:9060): erf(x / divisor) + offset, times x and factor."""
        import torch
        out = torch.empty_like(x)
        self.check(lib().ovk_decomposed_gelu(self.h, _ptr(x), x.numel(), float(divisor), float(offset), float(factor),
                                             int(factor_first), _ptr(out)))
        return out

    def decomposed_gelu_quantize(self, x, divisor, offset, factor, factor_first=False):
        """interp::decomposed_gelu_quantize (interp.rs:9125): DynamicQuantizeLinear of the GELU, which is never stored."""
        import torch
        y = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        scale = torch.empty((), dtype=torch.float32, device=x.device)
        zp = torch.empty((), dtype=torch.uint8, device=x.device)
        self.check(lib().ovk_decomposed_gelu_quantize(self.h, _ptr(x), x.numel(), float(divisor), float(offset),
                                                      float(factor), int(factor_first), _ptr(y), _ptr(scale), _ptr(zp)))
        return y, scale, zp

    # --------------------------------------------------------- MatMulInteger
    def mmi_prepack(self, b):
        return MmiWeight(self, b)

    def matmul_integer(self, w: "MmiWeight", a, a_zp=None, b_zp=None):
        import torch
        m = a.numel() // max(w.k, 1)
        out = torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=torch.int32, device=a.device)
        self.check(lib().ovk_matmul_integer(self.h, w.h, _ptr(a), int(a.dtype == torch.int8), m,
                                            _ptr(a_zp), _ptr(b_zp), _ptr(out)))
        return out

    def matmul_integer_static_scratch(self, w: "MmiWeight", a, a_zp=None, b_zp=None, out=None):
        """MatMulInteger through the entry point that allocates nothing: for hosts
        that own all device memory themselves.  `out` must be supplied by such a
        caller; it is created here only as a convenience for tests."""
        import torch
        m = a.numel() // max(w.k, 1)
        if out is None:
            out = torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=torch.int32, device=a.device)
        self.check(lib().ovk_matmul_integer_static_scratch(self.h, w.h, _ptr(a), int(a.dtype == torch.int8), m,
                                                           _ptr(a_zp), _ptr(b_zp), _ptr(out)))
        return out

    def matmul_integer_scale_bias(self, w: "MmiWeight", a, a_zp, b_zp, scale, bias, product=None,
                                  relu=False, range_slot=None):
        import torch
        m = a.numel() // max(w.k, 1)
        out = torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=torch.float32, device=a.device)
        step = lambda t: 0 if t is None or t.numel() == 1 else (1 if t.numel() == w.n and t.shape[-1] == w.n else 2)
        flags = (EPILOGUE_RELU if relu else 0) | (EPILOGUE_RANGE if range_slot is not None else 0)
        self.check(lib().ovk_matmul_integer_scale_bias(
            self.h, w.h, _ptr(a), int(a.dtype == torch.int8), m, _ptr(a_zp), _ptr(b_zp),
            _ptr(scale), step(scale), _ptr(product), step(product), _ptr(bias), step(bias), flags,
            _ptr(range_slot), _ptr(out)))
        return out

    def matmul_integer_group(self, ws, a, a_zp=None, b_zp=None):
        """Several weights over the same A (q | k | v): one launch where the tensor-core tiles apply."""
        import torch
        m = a.numel() // max(ws[0].k, 1)
        outs = [torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=torch.int32, device=a.device) for w in ws]
        wp, op = (_P * len(ws))(*[w.h for w in ws]), (_P * len(ws))(*[_ptr(o) for o in outs])
        self.check(lib().ovk_matmul_integer_group(self.h, len(ws), wp, _ptr(a), int(a.dtype == torch.int8), m, _ptr(a_zp),
                                                  _ptr(b_zp), op))
        return outs

    def matmul_integer_scale_bias_group(self, ws, a, a_zp, b_zp, scales, biases, product=None, relu=False):
        """The fused Cast, Mul, Add [, Relu] epilogue for several weights over the same A; scales[j] / biases[j]
        are member j's, all of one value or all of one per column; `product` is one value."""
        import torch
        m = a.numel() // max(ws[0].k, 1)
        outs = [torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=torch.float32, device=a.device) for w in ws]
        n = len(ws)
        step = lambda ts: 0 if all(t.numel() == 1 for t in ts) else (1 if all(t.numel() == w.n for t, w in zip(ts, ws)) else 2)
        arr = lambda ts: (_P * n)(*[_ptr(t) for t in ts])
        self.check(lib().ovk_matmul_integer_scale_bias_group(
            self.h, n, (_P * n)(*[w.h for w in ws]), _ptr(a), int(a.dtype == torch.int8), m, _ptr(a_zp), _ptr(b_zp),
            arr(scales), step(scales), _ptr(product), 0, arr(biases), step(biases), EPILOGUE_RELU if relu else 0, arr(outs)))
        return outs

    def qlinear_matmul(self, w: "MmiWeight", a, a_zp, b_zp, ratio, y_zp, y_signed=False):
        import torch
        m = a.numel() // max(w.k, 1)
        out = torch.empty(tuple(a.shape[:-1]) + (w.n,), dtype=torch.int8 if y_signed else torch.uint8,
                          device=a.device)
        self.check(lib().ovk_qlinear_matmul(self.h, w.h, _ptr(a), int(a.dtype == torch.int8), m,
                                            _ptr(a_zp), _ptr(b_zp), _ptr(ratio), ratio.numel(),
                                            int(y_zp), int(y_signed), _ptr(out)))
        return out

    # ------------------------------------------- ConvInteger / QLinearConv
    def qconv_prepack(self, w, group=1):
        return QConvWeight(self, w, group)

    @staticmethod
    def _conv_params(x, pads, strides, dilations) -> ConvParams:
        n, c, h, wd = x.shape
        return ConvParams(n, c, h, wd, (C.c_int64 * 4)(*pads), (C.c_int64 * 2)(*strides),
                          (C.c_int64 * 2)(*dilations))

    def conv_output_shape(self, w: "QConvWeight", x, pads, strides, dilations):
        p = self._conv_params(x, pads, strides, dilations)
        ho, wo = _I64(), _I64()
        rc = lib().ovk_conv_output_shape(w.h, C.byref(p), C.byref(ho), C.byref(wo))
        if rc:
            raise OvkError(rc, "Conv: degenerate output shape")
        return ho.value, wo.value

    def conv_integer(self, w: "QConvWeight", x, x_zp=0, w_zp=0, pads=(0, 0, 0, 0), strides=(1, 1),
                     dilations=(1, 1)):
        import torch
        ho, wo = self.conv_output_shape(w, x, pads, strides, dilations)
        out = torch.empty((x.shape[0], w.c_out, ho, wo), dtype=torch.int32, device=x.device)
        p = self._conv_params(x, pads, strides, dilations)
        self.check(lib().ovk_conv_integer(self.h, w.h, _ptr(x), int(x.dtype == torch.int8), C.byref(p),
                                          int(x_zp), int(w_zp), _ptr(out)))
        return out

    def conv_integer_scale_bias(self, w: "QConvWeight", x, x_zp, w_zp, scale, bias, product=None, relu=False,
                                range_slot=None, pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1)):
        """scale, bias, product: float32 device tensors of 1 or C_out values."""
        import torch
        ho, wo = self.conv_output_shape(w, x, pads, strides, dilations)
        out = torch.empty((x.shape[0], w.c_out, ho, wo), dtype=torch.float32, device=x.device)
        p = self._conv_params(x, pads, strides, dilations)
        step = lambda t: 0 if t is None or t.numel() == 1 else (1 if t.numel() == w.c_out else 2)
        flags = (EPILOGUE_RELU if relu else 0) | (EPILOGUE_RANGE if range_slot is not None else 0)
        self.check(lib().ovk_conv_integer_scale_bias(
            self.h, w.h, _ptr(x), int(x.dtype == torch.int8), C.byref(p), int(x_zp), int(w_zp),
            _ptr(scale), step(scale), _ptr(product), step(product), _ptr(bias), step(bias), flags,
            _ptr(range_slot), _ptr(out)))
        return out

    def qlinear_conv(self, w: "QConvWeight", x, x_zp, w_zp, ratio, bias, y_zp, y_signed=False,
                     pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1), out=None):
        """ratio: host float32 array of C_out values, (x_scale*w_scale[c])/y_scale."""
        import numpy as np
        import torch
        ho, wo = self.conv_output_shape(w, x, pads, strides, dilations)
        if out is None:
            out = torch.empty((x.shape[0], w.c_out, ho, wo), dtype=torch.int8 if y_signed else torch.uint8,
                              device=x.device)
        ratio = np.ascontiguousarray(ratio, dtype=np.float32)
        if ratio.size == 1:
            ratio = np.repeat(ratio, w.c_out)
        assert ratio.size == w.c_out
        p = self._conv_params(x, pads, strides, dilations)
        self.check(lib().ovk_qlinear_conv(self.h, w.h, _ptr(x), int(x.dtype == torch.int8), C.byref(p),
                                          int(x_zp), int(w_zp), ratio.ctypes.data, _ptr(bias),
                                          int(y_zp), int(y_signed), _ptr(out)))
        return out

    def to_padded_nhwc(self, x, pads, fill, out=None):
        """NCHW u8/i8 -> [n][h + top + bottom][w + left + right][c], the frame set to `fill`; pads = (top, left,
        bottom, right)."""
        import torch
        n, c, h, w = x.shape
        if out is None:
            out = torch.empty((n, h + pads[0] + pads[2], w + pads[1] + pads[3], c), dtype=x.dtype, device=x.device)
        self.check(lib().ovk_nchw_to_padded_nhwc(self.h, _ptr(x.contiguous()), n, c, h, w, (_I64 * 4)(*pads),
                                                 int(fill) & 0xff, _ptr(out)))
        return out

    def from_padded_nhwc(self, xp, pads):
        import torch
        n, hp, wp, c = xp.shape
        h, w = hp - pads[0] - pads[2], wp - pads[1] - pads[3]
        out = torch.empty((n, c, h, w), dtype=xp.dtype, device=xp.device)
        self.check(lib().ovk_padded_nhwc_to_nchw(self.h, _ptr(xp), n, c, h, w, (_I64 * 4)(*pads), _ptr(out)))
        return out

    def qlinear_conv_channels_last(self, w: "QConvWeight", x, x_zp, w_zp, ratio, bias, y_zp, out, out_pads=None,
                                   y_signed=False, pads=(0, 0, 0, 0), dilations=(1, 1), x_nchw=False, strides=(1, 1)):
        """QLinearConv from a padded-NHWC x (frame = `pads`, holding x_zp; or NCHW with x_nchw=True) into the
        interior of the padded-NHWC `out` whose frame is `out_pads` (None: `out` is NCHW)."""
        import numpy as np
        import torch
        if x_nchw:
            n, c, h, wd = x.shape
        else:
            n, hp, wp, c = x.shape
            h, wd = hp - pads[0] - pads[2], wp - pads[1] - pads[3]
        ratio = np.ascontiguousarray(ratio, dtype=np.float32)
        if ratio.size == 1:
            ratio = np.repeat(ratio, w.c_out)
        p = ConvParams(n, c, h, wd, (C.c_int64 * 4)(*pads), (C.c_int64 * 2)(*strides), (C.c_int64 * 2)(*dilations))
        self.check(lib().ovk_qlinear_conv_layout(self.h, w.h, _ptr(x), int(x.dtype == torch.int8), 0 if x_nchw else 1,
                                                 C.byref(p), int(x_zp), int(w_zp), ratio.ctypes.data, _ptr(bias),
                                                 int(y_zp), int(y_signed), _ptr(out), 0 if out_pads is None else 1,
                                                 None if out_pads is None else (_I64 * 4)(*out_pads)))
        return out

    def requantize(self, acc, inner, ratio, y_zp, bias=None, y_signed=False):
        import torch
        out = torch.empty(acc.shape, dtype=torch.int8 if y_signed else torch.uint8, device=acc.device)
        self.check(lib().ovk_requantize(self.h, _ptr(acc), acc.numel(), int(inner), ratio.numel(),
                                        _ptr(bias), _ptr(ratio), int(y_zp), int(y_signed), _ptr(out)))
        return out

    # ------------------------------------- neighbours of the lm_head product
    def gather_block_quantized(self, table, indices, scales, zero_points, block_size, out_dtype=None, out=None):
        """interp::gather_block_quantized (interp.rs:2874).  `indices`: a torch CUDA tensor (read on the
        device), or a CPU tensor / numpy array / list (checked on the host first, as the reference does)."""
        import numpy as np
        import torch
        rows, cols = int(table.shape[0]), int(table.shape[1]) * 2
        on_host = not (isinstance(indices, torch.Tensor) and indices.is_cuda)
        if on_host:
            idx = np.ascontiguousarray(np.asarray(indices, dtype=np.int64))
            shape, count, ptr, code = idx.shape, idx.size, idx.ctypes.data, INT64
        else:
            idx = indices.contiguous()
            shape, count, ptr, code = tuple(idx.shape), idx.numel(), _ptr(idx), _dtype_code(idx)
        if out is None:
            out = torch.empty(tuple(shape) + (cols,), dtype=out_dtype or torch.float32, device=table.device)
        self.check(lib().ovk_gather_block_quantized(self.h, _ptr(table), _ptr(scales), _dtype_code(scales),
                                                    _ptr(zero_points), rows, cols, 4, int(block_size), ptr, code,
                                                    int(on_host), count, _ptr(out), _dtype_code(out)))
        return out

    def argmax(self, x, axis=-1, out=None):
        """interp::arg_extreme_axis (interp.rs:8552): first-occurrence ArgMax over `axis`, int64, on the device."""
        import math
        import torch
        axis = axis % x.dim()
        outer, c, inner = math.prod(x.shape[:axis]), x.shape[axis], math.prod(x.shape[axis + 1:])
        if out is None:
            out = torch.empty(tuple(x.shape[:axis]) + tuple(x.shape[axis + 1:]), dtype=torch.int64, device=x.device)
        self.check(lib().ovk_argmax(self.h, _ptr(x), _dtype_code(x), outer, c, inner, _ptr(out)))
        return out

    # ------------------------------------ the QOperator chain around QLinearConv
    def qlinear_add(self, a, a_scale, a_zp, b, b_scale, b_zp, c_scale, c_zp):
        """interp::qlinear_add (interp.rs:4878); a and b are u8 or i8 tensors that broadcast."""
        import torch
        shape = torch.broadcast_shapes(a.shape, b.shape)
        out = torch.empty(shape, dtype=a.dtype, device=a.device)
        a, b = a.contiguous(), b.contiguous()
        sa, sb = (_I64 * max(a.dim(), 1))(*a.shape), (_I64 * max(b.dim(), 1))(*b.shape)
        self.check(lib().ovk_qlinear_add(self.h, _ptr(a), sa, a.dim(), float(a_scale), int(a_zp), _ptr(b), sb, b.dim(),
                                         float(b_scale), int(b_zp), float(c_scale), int(c_zp),
                                         int(a.dtype == torch.int8), _ptr(out), None, None))
        return out

    def maxpool_q(self, x, kernel, strides=None, pads=(0, 0, 0, 0), dilations=(1, 1)):
        """MaxPool in the quantized domain (shaders/qlinear.rs:145); x is [N, C, H, W] u8 or i8."""
        import torch
        n, c, h, w = x.shape
        strides = strides or (1, 1)
        arr = lambda v: (_I64 * len(v))(*[int(i) for i in v])
        dil = arr(dilations)
        ho = (h + pads[0] + pads[2] - (dilations[0] * (kernel[0] - 1) + 1)) // strides[0] + 1
        wo = (w + pads[1] + pads[3] - (dilations[1] * (kernel[1] - 1) + 1)) // strides[1] + 1
        out = torch.empty((n, c, max(ho, 0), max(wo, 0)), dtype=x.dtype, device=x.device)
        self.check(lib().ovk_maxpool_q(self.h, _ptr(x.contiguous()), int(x.dtype == torch.int8), n, c, h, w, arr(kernel),
                                       arr(strides), arr(pads), dil, _ptr(out), None, None))
        return out

    @staticmethod
    def _qdq_layout(shape, scale, axis):
        import math
        if scale.numel() <= 1:
            return 1, 1
        axis = axis % len(shape)
        return max(math.prod(shape[axis + 1:]), 1), scale.numel()

    def quantize_linear(self, x, scale, zero_point=None, axis=1, signed=False):
        """interp::quantize_linear (interp.rs:5117): saturate(rne(x / scale) + zero_point)."""
        import torch
        signed = signed if zero_point is None else zero_point.dtype == torch.int8
        inner, axis_len = self._qdq_layout(x.shape, scale, axis)
        out = torch.empty(x.shape, dtype=torch.int8 if signed else torch.uint8, device=x.device)
        self.check(lib().ovk_quantize_linear(self.h, _ptr(x.contiguous()), x.numel(), inner, axis_len, _ptr(scale),
                                             _ptr(zero_point), int(signed), _ptr(out)))
        return out

    def dequantize_linear(self, x, scale, zero_point=None, axis=1):
        """interp::dequantize_linear (interp.rs:5055): (x - zero_point) * scale, u8 / i8 / i32 input."""
        import torch
        inner, axis_len = self._qdq_layout(x.shape, scale, axis)
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        self.check(lib().ovk_dequantize_linear(self.h, _ptr(x.contiguous()), _dtype_code(x), x.numel(), inner, axis_len,
                                               _ptr(scale), _ptr(zero_point), _ptr(out)))
        return out

    def qlinear_global_average_pool(self, x, x_scale, x_zp, y_scale, y_zp):
        """interp::qlinear_global_average_pool (interp.rs:4975); x is [N, C, ...] u8 or i8."""
        import math
        import torch
        n, c = x.shape[0], x.shape[1]
        out = torch.empty((n, c) + (1,) * (x.dim() - 2), dtype=x.dtype, device=x.device)
        self.check(lib().ovk_qlinear_global_average_pool(self.h, _ptr(x.contiguous()), int(x.dtype == torch.int8), n, c,
                                                         math.prod(x.shape[2:]), float(x_scale), int(x_zp),
                                                         float(y_scale), int(y_zp), _ptr(out)))
        return out


class NBitsWeight:
    """A MatMulNBits weight prepared once (the role packed_b plays, interp.rs:2712)."""

    def __init__(self, ctx: Context, b, scales, zero_points, n, k, block_size, bits=4, flags=0):
        self.ctx, self.n, self.k, self.block_size = ctx, int(n), int(k), int(block_size)
        self._keep = (b, scales, zero_points)  # the operator-layout buffers must outlive the handle
        h = _P()
        ctx.check(lib().ovk_nbits_prepack(ctx.h, _ptr(b), _ptr(scales), _dtype_code(scales),
                                          _ptr(zero_points), n, k, bits, block_size, flags, C.byref(h)))
        self.h = h

    def __del__(self):
        try:
            if self.h and self.ctx.h:
                lib().ovk_nbits_weight_destroy(self.ctx.h, self.h)
        except Exception:
            pass


class MmiWeight:
    """B [K,N] of MatMulInteger in the tensor-core layout (packed_b, interp.rs:2712)."""

    def __init__(self, ctx: Context, b):
        import torch
        assert b.dim() == 2
        self.ctx, self.k, self.n = ctx, int(b.shape[0]), int(b.shape[1])
        self.signed = b.dtype == torch.int8
        h = _P()
        ctx.check(lib().ovk_mmi_prepack(ctx.h, _ptr(b), int(self.signed), self.k, self.n, C.byref(h)))
        self.h = h

    def __del__(self):
        try:
            if self.h and self.ctx.h:
                lib().ovk_mmi_weight_destroy(self.ctx.h, self.h)
        except Exception:
            pass


class QConvWeight:
    """A ConvInteger / QLinearConv filter bank [C_out, C_in/group, KH, KW]."""

    def __init__(self, ctx: Context, w, group=1):
        import torch
        if w.dim() == 3:  # 1-D convolution: W = 1
            w = w.unsqueeze(-1)
        self.ctx = ctx
        self.c_out, self.cig, self.kh, self.kw = (int(v) for v in w.shape)
        self.group = int(group)
        h = _P()
        ctx.check(lib().ovk_qconv_prepack(ctx.h, _ptr(w.contiguous()), int(w.dtype == torch.int8),
                                          self.c_out, self.cig, self.kh, self.kw, self.group, C.byref(h)))
        self.h = h

    def __del__(self):
        try:
            if self.h and self.ctx.h:
                lib().ovk_qconv_weight_destroy(self.ctx.h, self.h)
        except Exception:
            pass
