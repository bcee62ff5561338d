"""Pins the CPU oracle against the reference's own known-answer tests.

Each test restates one device test of automataIA/onnx-vulkan-rs (file:line in
the docstring, paths under crates/onnx-vulkan-core/): the same inputs, and the
expected values computed here independently of the C oracle (numpy / plain
Python, by the test's own scalar formula).  Integer results must be equal;
float results use the tolerance the reference's test uses.
"""
import json
import os

import numpy as np
import pytest

import cases
import oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


# ------------------------------------------------------------ MatMulNBits

@pytest.mark.parametrize("m,k,n,bs", cases.NBITS_REFERENCE_CASES)
def test_matmul_nbits_reference_cases(m, k, n, bs):
    """tests/matmul_nbits.rs:167-252, tolerance 1e-4*max(|w|,1) (:159-164)."""
    a, nib, zp, scale = cases.nbits_reference_case(m, k, n, bs)
    want = cases.nbits_expected_f64(a, nib, zp, scale, bs)
    got = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert got.shape == (m, n)
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))
    # the reference's shader order (f32 fma chain) agrees within the same bound
    sh = orc.matmul_nbits_f32_shader_order(a, orc.pack_nibbles(nib, bs), scale,
                                           orc.pack_zero_points(zp), k, n, bs)
    assert np.all(np.abs(sh - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))


def test_matmul_nbits_packing_is_low_nibble_first():
    """src/shaders/matmul_nbits.rs:15-19: element 2i in the low nibble."""
    nib = np.array([[1, 2, 3, 4, 5, 6, 7, 8] * 2], dtype=np.uint8)
    packed = orc.pack_nibbles(nib, 16)
    assert packed.reshape(-1)[0] == 0x21 and packed.reshape(-1)[3] == 0x87
    zp = np.array([[3, 9, 5]], dtype=np.uint8)
    assert orc.pack_zero_points(zp).tolist() == [[0x93, 0x05]]


def test_matmul_nbits_missing_zero_point_is_eight():
    """Operator definition (the reference refuses this form, src/interp.rs:447-463)."""
    a, nib, _, scale = cases.nbits_synthetic(1, 1, 64, 8, 32, real=np.float32, with_zp=False)
    eight = np.full((8, 2), 8, dtype=np.uint8)
    y0 = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, None, 64, 8, 32)
    y1 = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(eight), 64, 8, 32)
    assert np.array_equal(y0, y1)


def test_matmul_nbits_fp16_rounds_once():
    a, nib, zp, scale = cases.nbits_synthetic(2, 3, 96, 40, 32, real=np.float16)
    want = cases.nbits_expected_f64(a, nib, zp, scale, 32).astype(np.float16)
    got = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(zp), 96, 40, 32)
    assert got.dtype == np.float16
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_f16_conversion_matches_numpy():
    rng = np.random.default_rng(7)
    d = np.concatenate([rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000),
                        [0.0, -0.0, 65504.0, 65520.0, 65519.99, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -25,
                         1e-9, 1e9, -1e9, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11]])
    out = np.empty(d.size, dtype=np.uint16)
    orc.lib().orc_f64_to_f16(d.ctypes.data, out.ctypes.data, d.size)
    with np.errstate(over="ignore"):
        assert np.array_equal(out, d.astype(np.float16).view(np.uint16))
    back = np.empty(65536, dtype=np.float32)
    allh = np.arange(65536, dtype=np.uint16)
    orc.lib().orc_f16_to_f32(allh.ctypes.data, back.ctypes.data, 65536)
    ref = allh.view(np.float16).astype(np.float32)
    assert np.array_equal(back.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])


# ------------------------------------------------- DynamicQuantizeLinear

@pytest.mark.parametrize("r", [0.6, 1.0, 0.5, 2.0, 3.7])
def test_dql_symmetric_ramps(r):
    """tests/dynamic_quantize.rs:78-87: the zero point sits on a tie."""
    x = cases.dql_ramp(r)
    y, scale, zp = orc.dynamic_quantize(x)
    wy, wscale, wzp = cases.dql_numpy(x)
    assert np.float32(scale).view(np.uint32) == np.float32(wscale).view(np.uint32)
    assert zp == wzp and zp in (127, 128)
    assert np.array_equal(y, wy)


def test_dql_xorshift_million():
    """tests/dynamic_quantize.rs:90-102: 2^20 values, quotients near every .5."""
    x = cases.xorshift_dql_input(1 << 20)
    y, scale, zp = orc.dynamic_quantize(x)
    wy, wscale, wzp = cases.dql_numpy(x)
    assert np.float32(scale).view(np.uint32) == np.float32(wscale).view(np.uint32)
    assert zp == wzp
    assert int(np.count_nonzero(y != wy)) == 0


def test_dql_degenerate_inputs():
    """src/interp.rs:1949-1966 (empty), shader :143-145 (-0.0), range includes 0."""
    y, scale, zp = orc.dynamic_quantize(np.zeros(0, dtype=np.float32))
    assert (scale, zp, y.size) == (1.0, 0, 0)
    y, scale, zp = orc.dynamic_quantize(np.array([-0.0, 0.0], dtype=np.float32))
    assert (scale, zp) == (1.0, 0) and y.tolist() == [0, 0]
    for vals in ([2.0, 4.0], [-3.0, -1.0], [0.25], [-7.5]):
        x = np.array(vals, dtype=np.float32)
        y, scale, zp = orc.dynamic_quantize(x)
        wy, wscale, wzp = cases.dql_numpy(x)
        assert (float(scale), zp) == (float(wscale), wzp) and np.array_equal(y, wy)
        assert zp == (0 if vals[0] > 0 else 255)


# --------------------------------------------------------- MatMulInteger

def _mmi_numpy(a, b, azp, bzp):
    return ((a.astype(np.int64) - azp) @ (b.astype(np.int64) - bzp)).astype(np.int64)


def test_matmul_integer_small_case_with_both_zero_points():
    """tests/matmul_integer_variants.rs:110-145: (7,12,5), zp 37 / 211."""
    a = cases.lcg_bytes(7 * 12, 11).reshape(7, 12)
    b = cases.lcg_bytes(12 * 5, 29).reshape(12, 5)
    got = orc.matmul_integer(a, b, 37, 211)
    assert np.array_equal(got, _mmi_numpy(a, b, 37, 211))


@pytest.mark.parametrize("m,k,n", [(20, 64, 18), (150, 96, 90)])
def test_matmul_integer_tile_straddling_shapes(m, k, n):
    """tests/matmul_integer_variants.rs:161-244."""
    a = cases.lcg_bytes(m * k, 3).reshape(m, k)
    b = cases.lcg_bytes(k * n, 41).reshape(k, n)
    assert np.array_equal(orc.matmul_integer(a, b, 37, 211), _mmi_numpy(a, b, 37, 211))


def test_matmul_integer_signed_b_negative_zero_point():
    """tests/matmul_integer_variants.rs:255-352: int8 B, zp -73."""
    a = cases.lcg_bytes(20 * 64, 3).reshape(20, 64)
    b = cases.lcg_bytes(64 * 18, 41).reshape(64, 18).view(np.int8)
    assert np.array_equal(orc.matmul_integer(a, b, 37, -73), _mmi_numpy(a, b, 37, -73))


@pytest.mark.parametrize("k", [1, 2, 3, 5, 7])
@pytest.mark.parametrize("a_signed,b_signed", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_matmul_integer_any_k(k, a_signed, b_signed):
    """tests/matmul_integer_any_k.rs:141-150: K off the 4-byte grid, all signs."""
    a = cases.lcg_bytes(100 * k, 7).reshape(100, k)
    b = cases.lcg_bytes(k * 37, 13).reshape(k, 37)
    a = a.view(np.int8) if a_signed else a
    b = b.view(np.int8) if b_signed else b
    azp, bzp = (-5 if a_signed else 131), (-7 if b_signed else 121)
    assert np.array_equal(orc.matmul_integer(a, b, azp, bzp), _mmi_numpy(a, b, azp, bzp))


def test_matmul_integer_overflow_is_an_error():
    """src/host_ops.rs:1186-1190."""
    k = 40000
    a = np.full((1, k), 255, dtype=np.uint8)
    b = np.full((k, 1), 255, dtype=np.uint8)
    with pytest.raises(OverflowError):
        orc.matmul_integer(a, b, 0, 0)


def test_scale_bias_epilogue_rounds_each_step():
    """src/shaders/glsl/matmul_integer_coop.comp:162-181: x*s then +bias, no FMA."""
    rng = np.random.default_rng(3)
    acc = rng.integers(-2 ** 26, 2 ** 26, size=(9, 13)).astype(np.int32)
    scale = rng.uniform(1e-4, 1e-2, size=13).astype(np.float32)
    prod = rng.uniform(0.5, 2.0, size=1).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, size=13).astype(np.float32)
    got, rg = orc.scale_bias_epilogue(acc, scale, 1, bias, 1, product=prod, product_step=0,
                                      relu=True, want_range=True)
    s = (scale * prod[0]).astype(np.float32)
    want = np.maximum(((acc.astype(np.float32) * s).astype(np.float32) + bias).astype(np.float32), 0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert rg[1] == want.max() and rg[0] == max(0.0, float((-want).max()))


# ------------------------------------------------ QLinearConv / QLinearMatMul

def _requant_py(acc, ratio, y_zp, signed=False):
    q = int(np.rint(np.float32(np.float32(acc) * np.float32(ratio)))) + y_zp
    return max(-128, min(127, q)) if signed else max(0, min(255, q))


def _load_qlinear_vectors():
    with open(os.path.join(GOLDEN, "qlinear_literal_vectors.json")) as f:
        return json.load(f)


def test_qlinear_conv_per_channel_scales():
    """tests/qlinear.rs:106-153."""
    v = _load_qlinear_vectors()["conv_per_channel"]
    x = np.array(v["x"], dtype=np.uint8).reshape(1, 1, 3, 3)
    w = np.array(v["w"], dtype=np.int8).reshape(2, 1, 2, 2)
    got = orc.qlinear_conv(x, v["x_scale"], v["x_zp"], w, np.array(v["w_scale"], np.float32), 0,
                           v["y_scale"], v["y_zp"], bias=np.array(v["bias"], np.int32))
    want = []
    for c in range(2):
        ratio = np.float32(np.float32(np.float32(v["x_scale"]) * np.float32(v["w_scale"][c])) / np.float32(v["y_scale"]))
        for oh in range(2):
            for ow in range(2):
                acc = v["bias"][c]
                for r in range(2):
                    for s in range(2):
                        acc += (v["x"][(oh + r) * 3 + ow + s] - v["x_zp"]) * v["w"][c * 4 + r * 2 + s]
                want.append(_requant_py(acc, ratio, v["y_zp"]))
    assert got.reshape(-1).tolist() == want


def test_qlinear_conv_per_tensor_scale_keeps_per_channel_bias():
    """tests/qlinear.rs:155-206."""
    v = _load_qlinear_vectors()["conv_per_tensor"]
    x = np.array(v["x"], dtype=np.uint8).reshape(1, 1, 3, 3)
    w = np.array(v["w"], dtype=np.int8).reshape(2, 1, 2, 2)
    got = orc.qlinear_conv(x, v["x_scale"], v["x_zp"], w, np.array([v["w_scale"]], np.float32), 0,
                           v["y_scale"], v["y_zp"], bias=np.array(v["bias"], np.int32))
    ratio = np.float32(np.float32(np.float32(v["x_scale"]) * np.float32(v["w_scale"])) / np.float32(v["y_scale"]))
    want = []
    for c in range(2):
        for oh in range(2):
            for ow in range(2):
                acc = v["bias"][c]
                for r in range(2):
                    for s in range(2):
                        acc += (v["x"][(oh + r) * 3 + ow + s] - v["x_zp"]) * v["w"][c * 4 + r * 2 + s]
                want.append(_requant_py(acc, ratio, v["y_zp"]))
    assert got.reshape(-1).tolist() == want


def test_qlinear_conv_without_bias():
    """tests/qlinear.rs:208-236."""
    v = _load_qlinear_vectors()["conv_no_bias"]
    x = np.array(v["x"], dtype=np.uint8).reshape(1, 1, 2, 2)
    w = np.array(v["w"], dtype=np.int8).reshape(1, 1, 2, 2)
    got = orc.qlinear_conv(x, v["x_scale"], v["x_zp"], w, np.array([v["w_scale"]], np.float32), 0,
                           v["y_scale"], v["y_zp"])
    acc = sum((xv - v["x_zp"]) * wv for xv, wv in zip(v["x"], v["w"]))
    ratio = np.float32(np.float32(np.float32(v["x_scale"]) * np.float32(v["w_scale"])) / np.float32(v["y_scale"]))
    assert got.reshape(-1).tolist() == [_requant_py(acc, ratio, v["y_zp"])]


def test_qlinear_matmul_scales_per_column():
    """tests/qlinear.rs:240-275: MatMulInteger + requantize(inner=1, axis_len=N)."""
    v = _load_qlinear_vectors()["matmul_per_column"]
    a = np.array(v["a"], dtype=np.uint8).reshape(1, 4)
    b = np.array(v["b"], dtype=np.int8).reshape(4, 2)
    acc = orc.matmul_integer(a, b, v["a_zp"], 0)
    ratio = orc.requantize_ratio(v["a_scale"], np.array(v["b_scale"], np.float32), v["y_scale"])
    got = orc.requantize(acc, 1, ratio, v["y_zp"])
    want = []
    for col in range(2):
        s = sum((v["a"][k] - v["a_zp"]) * v["b"][k * 2 + col] for k in range(4))
        r = np.float32(np.float32(np.float32(v["a_scale"]) * np.float32(v["b_scale"][col])) / np.float32(v["y_scale"]))
        want.append(_requant_py(s, r, v["y_zp"]))
    assert got.reshape(-1).tolist() == want


def _conv_numpy(x, w, x_zp, w_zp, stride, dil, pads):
    """tests/conv_integer_im2col.rs:56-87, vectorised over output positions."""
    _, c_in, h, wd = x.shape
    c_out, _, kh, kw = w.shape
    t, l, b, r = pads
    ho = (h + t + b - (dil * (kh - 1) + 1)) // stride + 1
    wo = (wd + l + r - (dil * (kw - 1) + 1)) // stride + 1
    xs = x.astype(np.int64) - x_zp
    ws = w.astype(np.int64) - w_zp
    out = np.zeros((x.shape[0], c_out, ho, wo), dtype=np.int64)
    for rr in range(kh):
        for ss in range(kw):
            for oh in range(ho):
                ih = oh * stride + rr * dil - t
                if ih < 0 or ih >= h:
                    continue
                for ow in range(wo):
                    iw = ow * stride + ss * dil - l
                    if iw < 0 or iw >= wd:
                        continue
                    out[:, :, oh, ow] += xs[:, :, ih, iw] @ ws[:, :, rr, ss].T
    return out


@pytest.mark.parametrize("c_in,c_out,h,w,stride,dil,pads,xs,ws", [
    (64, 32, 20, 20, 1, 1, (1, 1, 1, 1), False, False),
    (32, 48, 18, 22, 2, 2, (2, 0, 1, 3), True, True),
    (32, 16, 15, 15, 1, 1, (1, 1, 1, 1), False, True),
])
def test_conv_integer_reference_geometries(c_in, c_out, h, w, stride, dil, pads, xs, ws):
    """tests/conv_integer_im2col.rs:185-247; x_zp 129 (u8) / -5 (i8), w_zp 7 (:98)."""
    x = cases.lcg_bytes_fast(c_in * h * w, 11).reshape(1, c_in, h, w)
    wt = cases.lcg_bytes_fast(c_out * c_in * 9, 5).reshape(c_out, c_in, 3, 3)
    x = x.view(np.int8) if xs else x
    wt = wt.view(np.int8) if ws else wt
    x_zp = -5 if xs else 129
    got = orc.conv_integer(x, wt, x_zp, 7, strides=(stride, stride), dilations=(dil, dil), pads=pads)
    assert np.array_equal(got, _conv_numpy(x, wt, x_zp, 7, stride, dil, pads))


def test_conv_geometry_auto_pad():
    """src/interp.rs:3425-3437: SAME_UPPER puts the excess at the end."""
    g = orc.conv_geometry((1, 4, 7, 7), (8, 4, 3, 3), strides=(2, 2), auto_pad="SAME_UPPER")
    assert (g.h_out, g.w_out, g.phb, g.phe) == (4, 4, 1, 1)
    g = orc.conv_geometry((1, 4, 8, 8), (8, 4, 3, 3), strides=(2, 2), auto_pad="SAME_UPPER")
    assert (g.h_out, g.phb, g.phe) == (4, 0, 1)
    g = orc.conv_geometry((1, 4, 8, 8), (8, 4, 3, 3), strides=(2, 2), auto_pad="SAME_LOWER")
    assert (g.h_out, g.phb, g.phe) == (4, 1, 0)
    g = orc.conv_geometry((1, 4, 8, 8), (8, 4, 3, 3), pads=(1, 1, 1, 1), auto_pad="VALID")
    assert (g.h_out, g.phb, g.pwe) == (6, 0, 0)


def test_lcg_fast_equals_scalar():
    assert np.array_equal(cases.lcg_bytes_fast(10000, 11), cases.lcg_bytes(10000, 11))


# ------------------------------------------------ GatherBlockQuantized / ArgMax

def gbq_case(rows, cols, block_size):
    """The closed-form table of tests/gather_block_quantized.rs:57-66."""
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    nb = cols // block_size
    b = np.arange(nb)[None, :]
    nib = ((r * 5 + c * 3) % 16).astype(np.uint8)
    zp = ((r + b * 7) % 16).astype(np.uint8)
    scale = (((r * 3 + b) % 11).astype(np.float32) / np.float32(32.0) - np.float32(0.15)).astype(np.float32)
    table = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    zpad = np.zeros((rows, nb + (nb & 1)), dtype=np.uint8)
    zpad[:, :nb] = zp
    zpk = (zpad[:, 0::2] | (zpad[:, 1::2] << 4)).astype(np.uint8)
    return nib, zp, scale, table, zpk


@pytest.mark.parametrize("rows,cols,bs,indices", [
    (64, 1152, 32, [[37]]),                 # tests/gather_block_quantized.rs:163-172
    (32, 128, 32, [[0, 31, 7, 7, 1]]),      # :175-183
    (16, 64, 16, [-1, -16, 3]),             # :186-194
    (9, 80, 16, [8, 0, 5]),                 # :197-207
])
def test_gather_block_quantized_reference_cases(rows, cols, bs, indices):
    nib, zp, scale, table, zpk = gbq_case(rows, cols, bs)
    idx = np.array(indices, dtype=np.int64)
    got = orc.gather_block_quantized(table, idx, scale, zpk, bs)
    assert got.shape == idx.shape + (cols,)
    rr = np.where(idx < 0, idx + rows, idx).reshape(-1)
    blk = np.arange(cols) // bs
    want = (nib[rr].astype(np.float32) - zp[rr][:, blk].astype(np.float32)) * scale[rr][:, blk]
    assert np.array_equal(got.reshape(-1, cols), want)


def test_gather_block_quantized_refuses_an_index_outside_the_table():
    _, _, scale, table, zpk = gbq_case(16, 64, 16)
    with pytest.raises(IndexError):
        orc.gather_block_quantized(table, np.array([16]), scale, zpk, 16)
    with pytest.raises(IndexError):
        orc.gather_block_quantized(table, np.array([-17]), scale, zpk, 16)


def test_argmax_first_occurrence_and_candidates():
    """tests/argmax.rs:126-147 (ties) and the kernels' candidate rule (shaders/reduction.rs:101-107)."""
    assert orc.argmax(np.full(4096, 0.5, dtype=np.float32), 0) == 0
    twice = np.zeros(4096, dtype=np.float32)
    twice[700] = twice[3000] = 2.0
    assert orc.argmax(twice, 0) == 700
    x = np.random.Generator(np.random.PCG64(5)).standard_normal((2, 5, 3, 3)).astype(np.float32)
    assert np.array_equal(orc.argmax(x, 1), np.argmax(x, axis=1))
    odd = np.array([[np.nan, -np.inf, -3.0], [-np.inf, -np.inf, np.nan]], dtype=np.float32)
    assert orc.argmax(odd, 1).tolist() == [2, 0]


# ------------------------------------------ the QOperator chain around QLinearConv

def mlas_add(a, b, scales, zps):
    """tests/qlinear.rs:317-322, in float32 with explicit fused multiply-adds (via float64, which
    holds the exact product of two float32 values and rounds the sum once)."""
    sa, sb, sc = (np.float32(v) for v in scales)
    za, zb, zc = zps
    ra, rb = np.float32(sa / sc), np.float32(sb / sc)
    fma = lambda x, y, z: np.float32(np.float64(x) * np.float64(y) + np.float64(z))
    fixed = np.float32(np.float32(zc) - fma(ra, np.float32(za), np.float32(rb * np.float32(zb))))
    y = fma(np.float32(a), ra, fma(np.float32(b), rb, fixed))
    return int(np.clip(np.rint(y), 0, 255))


def test_qlinear_add_broadcast_literal():
    """tests/qlinear.rs:279-314."""
    a = np.array([[200, 10, 50], [128, 255, 0]], dtype=np.uint8)
    b = np.array([100, 130, 20], dtype=np.uint8)
    got = orc.qlinear_add(a, 0.02, 128, b, 0.05, 100, 0.03, 30)
    want = [mlas_add(int(a.reshape(-1)[i]), int(b[i % 3]), (0.02, 0.05, 0.03), (128, 100, 30)) for i in range(6)]
    assert got.reshape(-1).tolist() == want


def test_qlinear_add_rounds_like_the_cpu_reference_on_every_input_pair():
    """tests/qlinear.rs:356-373: the three pairs ORT maps to 82, 148, 214."""
    scales, zps = (0.03207505, 0.061237868, 0.067996934), (116, 145, 125)
    a = (np.arange(65536) % 256).astype(np.uint8)
    b = (np.arange(65536) // 256).astype(np.uint8)
    got = orc.qlinear_add(a, scales[0], zps[0], b, scales[1], zps[1], scales[2], zps[2])
    for av, bv, cpu in [(129, 91, 82), (162, 147, 148), (195, 203, 214)]:
        assert got[bv * 256 + av] == cpu
    idx = np.arange(0, 65536, 97)
    assert got[idx].tolist() == [mlas_add(int(a[i]), int(b[i]), scales, zps) for i in idx]


def test_qlinear_add_exchanges_a_broadcast_first_operand():
    """tests/qlinear.rs:376-392: at B = 195 the unexchanged formula gives 41, ORT 40."""
    scales, zps = (0.264079, 0.081802, 0.010314), (128, 205, 43)
    b = np.arange(256, dtype=np.uint8)
    got = orc.qlinear_add(np.array([131], dtype=np.uint8), scales[0], zps[0], b, scales[1], zps[1], scales[2], zps[2])
    assert got[195] == 40
    sa, sb, sc = scales
    za, zb, zc = zps
    assert got.tolist() == [mlas_add(v, 131, (sb, sa, sc), (zb, za, zc)) for v in range(256)]


def test_maxpool_q_literal():
    """tests/qlinear.rs:395-416."""
    x = np.array([10, 200, 30, 40, 50, 60, 250, 80, 90, 100, 110, 120, 130, 140, 150, 160], dtype=np.uint8)
    got = orc.maxpool_q(x.reshape(1, 1, 4, 4), (2, 2), strides=(2, 2))
    assert got.reshape(-1).tolist() == [200, 250, 140, 160]


def test_qlinear_global_average_pool_literal():
    """tests/qlinear.rs:419-452."""
    x = np.array([10, 20, 30, 40, 200, 210, 220, 230], dtype=np.uint8).reshape(1, 2, 2, 2)
    got = orc.qlinear_global_average_pool(x, 0.02, 15, 0.05, 7)
    want = []
    for plane in x.reshape(2, 4):
        acc = np.float32(0)
        for v in plane:
            acc = np.float32(acc + np.float32(np.float32(int(v) - 15) * np.float32(0.02)))
        mean = np.float32(acc / np.float32(4.0))
        want.append(int(np.clip(int(np.rint(np.float32(mean / np.float32(0.05)))) + 7, 0, 255)))
    assert got.reshape(-1).tolist() == want


def test_quantize_dequantize_linear_per_tensor_and_per_axis():
    """shaders/quantize_linear.rs: ties to even, saturation, per-axis channel = (i / inner) % axis_len."""
    x = np.array([-13.5, -12.5, 0.49, 0.5, 1.5, 2.5, 300.0, -300.0], dtype=np.float32)
    q = orc.quantize_linear(x, np.array([1.0], dtype=np.float32), np.array([10], dtype=np.uint8))
    assert q.tolist() == [0, 0, 10, 10, 12, 12, 255, 0]
    qs = orc.quantize_linear(x, np.array([1.0], dtype=np.float32), np.array([-3], dtype=np.int8))
    assert qs.tolist() == [-17, -15, -3, -3, -1, -1, 127, -128]
    xa = np.arange(24, dtype=np.float32).reshape(2, 3, 4) - 11.0
    scale = np.array([0.5, 1.0, 2.0], dtype=np.float32)
    zp = np.array([1, 2, 3], dtype=np.uint8)
    qa = orc.quantize_linear(xa, scale, zp, axis=1)
    want = np.clip(np.rint(xa / scale[None, :, None]) + zp[None, :, None], 0, 255).astype(np.uint8)
    assert np.array_equal(qa, want)
    back = orc.dequantize_linear(qa, scale, zp, axis=1)
    assert np.array_equal(back, (qa.astype(np.float32) - zp[None, :, None].astype(np.float32)) * scale[None, :, None])
    bias = np.array([-70000, 5, 123456], dtype=np.int32)
    assert np.array_equal(orc.dequantize_linear(bias, np.array([0.25], dtype=np.float32)),
                          bias.astype(np.float32) * np.float32(0.25))


# ------------------------------------------------------------------ DecomposedGelu

def test_decomposed_gelu_port_follows_the_shader_arithmetic():
    """shaders/elementwise.rs:71-118, restated independently in numpy float32 step by step (with the
    port's own exp, the one function the shader leaves to the device), and close to the exact GELU:
    the five-term erf is good to 1.5e-7."""
    import math
    x = np.concatenate([np.linspace(-9, 9, 3001), [0.0, -0.0, 1e-20, 30.0, -30.0]]).astype(np.float32)
    f = np.float32
    for factor_first in (False, True):
        got = orc.decomposed_gelu(x, float(f(math.sqrt(2.0))), 1.0, 0.5, factor_first)
        v = x / f(math.sqrt(2.0))
        s, a = np.sign(v).astype(f), np.abs(v)
        t = f(1.0) / (f(1.0) + f(0.3275911) * a)
        poly = t * f(1.061405429)
        for c in (-1.453152027, 1.421413741, -0.284496736, 0.254829592):
            poly = t * (f(c) + poly)
        ex = np.array([orc.exp_ieee(float(-ai * ai)) for ai in a], dtype=f)
        e = s * (f(1.0) - poly * ex) + f(1.0)
        want = x * (e * f(0.5)) if factor_first else (x * e) * f(0.5)
        assert np.array_equal(got.view(np.uint32), want.astype(f).view(np.uint32))
        exact = np.array([0.5 * float(xi) * (1.0 + math.erf(float(xi) / math.sqrt(2.0))) for xi in x])
        assert np.abs(got - exact).max() < 5e-6
    for xv in np.linspace(-103.0, 2.0, 2001):  # exp in IEEE operations: about one ulp
        want = math.exp(float(f(xv)))
        assert abs(orc.exp_ieee(float(f(xv))) - want) <= 1.5 * 1.2e-7 * want + 1e-45
    y, scale, zp = orc.decomposed_gelu_quantize(x, float(f(math.sqrt(2.0))), 1.0, 0.5)
    y2, scale2, zp2 = orc.dynamic_quantize(orc.decomposed_gelu(x, float(f(math.sqrt(2.0))), 1.0, 0.5))
    assert np.array_equal(y, y2) and scale == scale2 and zp == zp2
