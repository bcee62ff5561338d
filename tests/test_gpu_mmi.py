"""MatMulInteger and its fused epilogues: exact int32, bit-equal fp32."""
import numpy as np
import pytest
import torch

import cases
import oracle as orc
from gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def zp_dev(v, signed):
    return dev(np.array([v], dtype=np.int8 if signed else np.uint8))


def run_mmi(a, b, azp, bzp):
    w = ctx().mmi_prepack(dev(b))
    out = ctx().matmul_integer(w, dev(a), zp_dev(azp, a.dtype == np.int8), zp_dev(bzp, b.dtype == np.int8))
    return host(out), ctx().last_kernel


def test_small_case_both_zero_points():
    """tests/matmul_integer_variants.rs:110-145."""
    a = cases.lcg_bytes(7 * 12, 11).reshape(7, 12)
    b = cases.lcg_bytes(12 * 5, 29).reshape(12, 5)
    got, _ = run_mmi(a, b, 37, 211)
    assert np.array_equal(got, orc.matmul_integer(a, b, 37, 211))


@pytest.mark.parametrize("m", [1, 3, 15])
@pytest.mark.parametrize("a_signed,b_signed", [(False, True), (True, False)])
def test_a_few_rows_over_a_large_weight_take_the_tensor_core_kernel(m, a_signed, b_signed):
    """An int8 decode step (1 to 15 rows against a weight of a million elements and more) streams the weight through
    the tensor-core kernel, whose bulk loads fill the rows of A that do not exist with zeros; both zero points, exact."""
    k, n = 1024, 1100
    a = cases.lcg_bytes_fast(m * k, 31).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 37).reshape(k, n)
    a = a.view(np.int8) if a_signed else a
    b = b.view(np.int8) if b_signed else b
    azp, bzp = (-5 if a_signed else 131), (-7 if b_signed else 121)
    got, kernel = run_mmi(a, b, azp, bzp)
    assert kernel.startswith("mmi_tc"), kernel
    assert np.array_equal(got, orc.matmul_integer(a, b, azp, bzp))


@pytest.mark.parametrize("m,k,n", [(20, 64, 18), (150, 96, 90), (129, 128, 257), (300, 256, 130)])
def test_tile_straddling_shapes(m, k, n):
    """tests/matmul_integer_variants.rs:161-244 plus shapes around the 128-wide tiles."""
    a = cases.lcg_bytes_fast(m * k, 3).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 41).reshape(k, n)
    got, _ = run_mmi(a, b, 37, 211)
    assert np.array_equal(got, orc.matmul_integer(a, b, 37, 211))


def test_signed_b_negative_zero_point():
    """tests/matmul_integer_variants.rs:255-352."""
    a = cases.lcg_bytes(20 * 64, 3).reshape(20, 64)
    b = cases.lcg_bytes(64 * 18, 41).reshape(64, 18).view(np.int8)
    got, _ = run_mmi(a, b, 37, -73)
    assert np.array_equal(got, orc.matmul_integer(a, b, 37, -73))


@pytest.mark.parametrize("k", [1, 2, 3, 5, 7])
@pytest.mark.parametrize("a_signed,b_signed", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_any_k(k, a_signed, b_signed):
    """tests/matmul_integer_any_k.rs:141-150: (1000, K, 37), all sign pairs."""
    a = cases.lcg_bytes_fast(1000 * k, 7).reshape(1000, k)
    b = cases.lcg_bytes(k * 37, 13).reshape(k, 37)
    a = a.view(np.int8) if a_signed else a
    b = b.view(np.int8) if b_signed else b
    azp, bzp = (-5 if a_signed else 131), (-7 if b_signed else 121)
    got, _ = run_mmi(a, b, azp, bzp)
    assert np.array_equal(got, orc.matmul_integer(a, b, azp, bzp))


def test_box_projection_shape():
    """tests/matmul_integer_any_k.rs:141: (14400, 2, 256) u8 x i8."""
    a = cases.lcg_bytes_fast(14400 * 2, 7).reshape(14400, 2)
    b = cases.lcg_bytes(2 * 256, 13).reshape(2, 256).view(np.int8)
    got, _ = run_mmi(a, b, 131, -7)
    assert np.array_equal(got, orc.matmul_integer(a, b, 131, -7))


@pytest.mark.parametrize("k,n", [(1024, 1024), (1024, 4096), (4096, 1024)])
def test_parakeet_layer_gemms(k, n):
    """Config 3: DQL(u8, per-tensor) x int8 per-channel symmetric weights, T=1000;
    int32 exact, then float(acc)*(a_scale*w_scale[n]) bit-equal."""
    x = cases.rng_for(3, 0).standard_normal((1000, k), dtype=np.float32)
    wq = cases.rng_for(3, 1).integers(-127, 128, size=(k, n), dtype=np.int8)
    w_scale = cases.rng_for(3, 2).uniform(0.001, 0.01, size=n).astype(np.float32)
    xq, a_scale, a_zp = ctx().dynamic_quantize(dev(x))
    oq, o_scale, o_zp = orc.dynamic_quantize(x)
    w = ctx().mmi_prepack(dev(wq))
    acc = ctx().matmul_integer(w, xq, a_zp, None)
    want = orc.matmul_integer(oq, wq, o_zp, 0)
    assert np.array_equal(host(acc), want)
    bias = np.zeros(n, dtype=np.float32)
    out = ctx().matmul_integer_scale_bias(w, xq, a_zp, None, dev(w_scale), dev(bias),
                                          product=a_scale.reshape(1))
    want_f = orc.scale_bias_epilogue(want, w_scale, 1, bias, 1, product=np.array([o_scale], np.float32),
                                     product_step=0)
    assert np.array_equal(host(out).view(np.uint32), want_f.view(np.uint32))


# (A shape, N, W int8, scale kind, relu, range, w_scale per column): the fused
# rows of crates/onnx-vulkan-core/tests/matmul_integer_epilogue.rs:352-736
EPILOGUE_CASES = [
    ((2, 50, 64), 200, False, "product", False, False, False),
    ((700, 96), 330, True, "product", False, False, False),
    ((1100, 64), 1040, True, "product", False, False, False),
    ((1, 128, 32), 48, False, "column", False, False, False),
    ((1, 20, 72, 2), 256, False, "product", False, False, False),
    ((37, 7), 50, True, "column", False, False, False),
    ((700, 96), 330, True, "product", True, False, False),
    ((37, 7), 50, True, "column", True, False, False),
    ((700, 96), 330, True, "product", True, True, False),
    ((1100, 64), 1040, False, "column", False, True, False),
    ((2, 50, 64), 200, False, "product", False, True, False),
    ((1, 32, 256), 320, True, "product", False, True, True),
    ((700, 96), 330, True, "product", True, False, True),
    ((37, 7), 50, True, "product", False, False, True),
    ((1, 1, 256), 48, False, "product", True, True, True),
    ((3, 200, 64), 8, True, "product", False, True, True),
    ((1, 1, 256), 1, True, "scalar", False, False, False),
    ((2, 150, 96), 4, True, "column", False, True, False),
]


@pytest.mark.parametrize("a_shape,n,w_int8,scale_kind,relu,fold_range,per_col", EPILOGUE_CASES)
def test_fused_epilogue_is_bit_identical_to_the_unfused_steps(a_shape, n, w_int8, scale_kind, relu,
                                                              fold_range, per_col):
    k = a_shape[-1]
    m = int(np.prod(a_shape[:-1]))
    a = cases.lcg_bytes_fast(m * k, 1).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 2).reshape(k, n)
    b = b.view(np.int8) if w_int8 else b
    w_zp = -7 if w_int8 else 121
    a_zp = 131
    rng = cases.rng_for(9, n)
    bias = rng.uniform(-0.5, 0.5, size=n).astype(np.float32)
    if scale_kind == "product":
        scale = rng.uniform(1e-3, 5e-3, size=n).astype(np.float32) if per_col else np.array([3.1e-3], np.float32)
        product = np.array([0.0123], np.float32)
    elif scale_kind == "column":
        scale, product = rng.uniform(1e-5, 1e-4, size=n).astype(np.float32), None
    else:
        scale, product = np.array([3.8e-5], np.float32), None
    acc = orc.matmul_integer(a, b, a_zp, w_zp)
    want, want_rng = orc.scale_bias_epilogue(acc, scale, int(scale.size > 1), bias, int(bias.size > 1),
                                             product=product, product_step=0, relu=relu, want_range=True)
    w = ctx().mmi_prepack(dev(b))
    slot = torch.zeros(2, dtype=torch.int32, device="cuda") if fold_range else None
    got = ctx().matmul_integer_scale_bias(
        w, dev(a), zp_dev(a_zp, False), zp_dev(w_zp, w_int8), dev(scale), dev(bias),
        product=None if product is None else dev(product), relu=relu, range_slot=slot)
    assert np.array_equal(host(got).reshape(m, n).view(np.uint32), want.view(np.uint32))
    if fold_range:
        got_rng = host(slot).view(np.float32)
        assert got_rng[0] == want_rng[0] and got_rng[1] == want_rng[1]


def test_scale_over_rows_is_refused_like_the_reference_falls_back():
    """tests/matmul_integer_epilogue.rs:423 ('scale over rows' is not fused)."""
    import ovk_b200
    a = cases.lcg_bytes(64 * 32, 1).reshape(64, 32)
    b = cases.lcg_bytes(32 * 32, 2).reshape(32, 32)
    w = ctx().mmi_prepack(dev(b))
    with pytest.raises(ovk_b200.OvkError) as e:
        ctx().matmul_integer_scale_bias(w, dev(a), None, None, dev(np.ones((64, 1), np.float32)),
                                        dev(np.zeros(32, np.float32)))
    assert e.value.status == ovk_b200.UNSUPPORTED


def test_qlinear_matmul_literal_vectors():
    """tests/qlinear.rs:240-275."""
    a = np.array([[130, 120, 140, 128]], dtype=np.uint8)
    b = np.array([1, -2, 3, 4, -5, 6, 7, -8], dtype=np.int8).reshape(4, 2)
    ratio = orc.requantize_ratio(0.02, np.array([0.01, 0.03], np.float32), 0.05)
    w = ctx().mmi_prepack(dev(b))
    got = ctx().qlinear_matmul(w, dev(a), zp_dev(128, False), None, dev(ratio), 10)
    want = orc.requantize(orc.matmul_integer(a, b, 128, 0), 1, ratio, 10)
    assert np.array_equal(host(got), want)


def test_accumulator_overflow_guard():
    """interp.rs:2216-2218: K above 33025 could overflow i32 and is refused."""
    import ovk_b200
    b = torch.zeros((33026, 1), dtype=torch.uint8, device="cuda")
    w = ctx().mmi_prepack(b)
    with pytest.raises(ovk_b200.OvkError):
        ctx().matmul_integer(w, torch.zeros((1, 33026), dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("m,k,n,a_signed,b_signed", [(1000, 2064, 9470, 0, 1), (1024, 2048, 9472, 1, 0),
                                                     (2300, 2048, 7500, 0, 1)])
def test_large_product_takes_256_tiles(m, k, n, a_signed, b_signed):
    """Long K and whole waves of 256-row blocks: ragged edges in M, N and K, both zero points.  Where the GPU runs
    clusters, two CTAs share each 512 x 256 tile (tcgen05.mma.cta_group::2, half of the B stage loaded by each): the
    last tile's second CTA has rows past M (1000 = 512 + 488) or none at all (2300 = 4 x 512 + 252)."""
    a = cases.lcg_bytes_fast(m * k, 19).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 23).reshape(k, n)
    a = a.view(np.int8) if a_signed else a
    b = b.view(np.int8) if b_signed else b
    azp, bzp = (-5 if a_signed else 131), (-7 if b_signed else 121)
    got, kernel = run_mmi(a, b, azp, bzp)
    assert kernel in ("mmi_tc_256x256", "mmi_tc_pair_512x256")
    assert np.array_equal(got, orc.matmul_integer(a, b, azp, bzp))


@pytest.mark.parametrize("m,k,n", [(2048, 256, 2048), (3000, 384, 1500), (2100, 192, 4224), (4096, 128, 4096)])
def test_short_k_many_tiles_two_issuers(m, k, n):
    """Two threads issue alternate K stages of a tile, and only the tile's first MMA
    overwrites the accumulator: with two or three stages per tile and several tiles
    per CTA every tile start is a hand-over between them (and with one stage per
    tile the other thread only signs the tile off).  Exact against the CPU port."""
    rng = np.random.default_rng(m + k + n)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-127, 128, (k, n), dtype=np.int8)
    w = ctx().mmi_prepack(dev(b))
    zp = zp_dev(131, False)
    want = torch.from_numpy(orc.matmul_integer(a, b, 131, 0)).cuda()
    for _ in range(3):  # the interleaving of the two streams differs from launch to launch
        got = ctx().matmul_integer(w, dev(a), zp, None)
        assert ctx().last_kernel.startswith("mmi_tc"), ctx().last_kernel
        ctx().flush()
        assert torch.equal(got, want)


@pytest.mark.parametrize("m,k,ns,b_zp", [(1000, 1024, (1024, 1024, 1024), None), (300, 256, (130, 64, 200), -7),
                                          (40, 96, (48, 330), None), (7, 12, (5, 9), 3)])
def test_group_of_weights_over_the_same_a(m, k, ns, b_zp):
    """q | k | v over one quantised tensor: one launch where the tensor-core tiles apply (ragged member widths
    included), one call per member otherwise; int32 results and the fused f32 epilogue are those of separate calls."""
    a = cases.lcg_bytes_fast(m * k, 31).reshape(m, k)
    bs = [cases.lcg_bytes_fast(k * n, 40 + j).reshape(k, n).view(np.int8) for j, n in enumerate(ns)]
    ws = [ctx().mmi_prepack(dev(b)) for b in bs]
    azp = zp_dev(131, False)
    bzp = None if b_zp is None else zp_dev(b_zp, True)
    before = ctx().launches
    outs = ctx().matmul_integer_group(ws, dev(a), azp, bzp)
    launched = ctx().launches - before
    if m >= 16 and min(ns) >= 16:
        assert launched == (1 if b_zp is None else 2) and ctx().last_kernel.startswith("mmi_tc")
    for b, o in zip(bs, outs):
        assert np.array_equal(host(o), orc.matmul_integer(a, b, 131, b_zp or 0))
    scales = [dev(np.random.default_rng(j).uniform(1e-3, 1e-2, n).astype(np.float32)) for j, n in enumerate(ns)]
    biases = [dev(np.random.default_rng(9 + j).standard_normal(n).astype(np.float32)) for j, n in enumerate(ns)]
    prod = dev(np.array([0.0123], dtype=np.float32))
    fused = ctx().matmul_integer_scale_bias_group(ws, dev(a), azp, bzp, scales, biases, product=prod, relu=True)
    for w, s, bi, o in zip(ws, scales, biases, fused):
        alone = ctx().matmul_integer_scale_bias(w, dev(a), azp, bzp, s, bi, product=prod, relu=True)
        assert np.array_equal(host(o).view(np.uint32), host(alone).view(np.uint32))
