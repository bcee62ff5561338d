"""DynamicQuantizeLinear parity: bit-equal scale, equal zero point, 0 differing
bytes (crates/onnx-vulkan-core/tests/dynamic_quantize.rs:60-76)."""
import math

import numpy as np
import pytest
import torch

import cases
import oracle as orc
from gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def check(x):
    y, scale, zp = ctx().dynamic_quantize(dev(x))
    wy, wscale, wzp = orc.dynamic_quantize(x)
    y, scale, zp = host(y), host(scale), host(zp)
    assert np.float32(scale).view(np.uint32) == np.float32(wscale).view(np.uint32), "scale"
    assert int(zp) == wzp, "zero point"
    assert int(np.count_nonzero(y != wy)) == 0


@pytest.mark.parametrize("r", [0.6, 1.0, 0.5, 2.0, 3.7])
def test_symmetric_ramps(r):
    """tests/dynamic_quantize.rs:78-87."""
    check(cases.dql_ramp(r))


def test_xorshift_million():
    """tests/dynamic_quantize.rs:90-102."""
    check(cases.xorshift_dql_input(1 << 20))


@pytest.mark.parametrize("n", [1, 2, 3, 5, 255, 1023, 1025, 4099])
def test_ragged_lengths_and_unaligned_views(n):
    x = cases.rng_for(3, n).standard_normal(n + 3, dtype=np.float32) * 3
    check(x[:n])
    # a view starting 4 bytes into the allocation: the vector path must not be taken
    t = dev(x)
    y, scale, zp = ctx().dynamic_quantize(t[1:n + 1])
    wy, wscale, wzp = orc.dynamic_quantize(x[1:n + 1])
    assert np.array_equal(host(y), wy) and float(host(scale)) == float(wscale) and int(host(zp)) == wzp


def test_empty_negative_zero_and_one_sided_ranges():
    """interp.rs:1949-1966 (empty); shader :143-145 (-0.0)."""
    y, scale, zp = ctx().dynamic_quantize(torch.empty(0, device="cuda"))
    assert float(host(scale)) == 1.0 and int(host(zp)) == 0
    for vals in ([-0.0, 0.0], [2.0, 4.0], [-3.0, -1.0], [0.25], [-7.5]):
        check(np.array(vals, dtype=np.float32))


@pytest.mark.parametrize("d", [1024, 4096])
def test_parakeet_activations(d):
    """Config 3: fp32 activations ~N(0,1) [T=1000, d_model or FF]."""
    x = cases.rng_for(3, 0).standard_normal((1000, d), dtype=np.float32)
    check(x)


# ------------------------------------------------------------------ one launch or two

def test_one_launch_up_to_the_register_capacity_then_two():
    """A tensor of whole 16-byte vectors that fits eight vectors per thread of one 1024-thread block per SM
    is quantized by ONE launch (the blocks meet at a counter between the passes); one vector more, a
    length that is no multiple of four, or an unaligned view take the two launches.  Same bytes, scale
    and zero point either way, and repeated calls find the counters zero again."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cap = sms * 1024 * 8 * 4
    rng = cases.rng_for(3, 99)
    for n, kernel, launches in ((4, "dql_one_pass", 1), (4096, "dql_one_pass", 1), (1024 * 1000, "dql_one_pass", 1),
                                (cap, "dql_one_pass", 1), (cap + 4, "dql_quantize", 2), (4098, "dql_quantize", 2)):
        x = rng.standard_normal(n, dtype=np.float32) * np.float32(2.5)
        x[n // 2] = -11.0
        want_y, want_s, want_z = orc.dynamic_quantize(x)
        for _ in range(3):
            before = ctx().launches
            y, s, z = ctx().dynamic_quantize(dev(x))
            assert ctx().launches - before == launches and ctx().last_kernel == kernel, n
            assert np.array_equal(host(y), want_y) and float(host(s)) == float(want_s) and int(host(z)) == want_z, n
    ctx().flush()  # raises if a wait ran out


# ------------------------------------------------------------------ folded range, DecomposedGelu

def test_folded_range_skips_the_range_pass_and_gives_the_same_bytes():
    """interp.rs:1979-1983: when the producer of x folded its range into a slot, only the quantize pass
    runs.  Here the producer is the fused MatMulInteger epilogue; the quantization that follows it equals
    the two-pass one byte for byte, and the slot is left zero for the next producer."""
    m, k, n = 700, 96, 330
    a = cases.lcg_bytes_fast(m * k, 11).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, 2).reshape(k, n).view(np.int8)
    w = ctx().mmi_prepack(dev(b))
    scale = dev(np.array([0.0123 * 3.1e-3], dtype=np.float32))
    bias = dev(np.random.default_rng(5).uniform(-0.5, 0.5, n).astype(np.float32))
    slot = torch.zeros(4, dtype=torch.int32, device="cuda")
    x = ctx().matmul_integer_scale_bias(w, dev(a), dev(np.array([131], dtype=np.uint8)), None, scale, bias,
                                        relu=True, range_slot=slot)
    before = ctx().launches
    y, s, z = ctx().dynamic_quantize(x, folded_range=slot)
    assert ctx().launches - before == 1 and ctx().last_kernel == "dql_quantize"
    want_y, want_s, want_z = orc.dynamic_quantize(host(x))
    assert np.array_equal(host(y), want_y) and float(s) == float(want_s) and int(z) == want_z
    assert slot.cpu().tolist() == [0, 0, 0, 0]
    y2, s2, z2 = ctx().dynamic_quantize(x)  # both passes
    assert np.array_equal(host(y2), want_y) and float(s2) == float(want_s)


GELU = (float(np.float32(np.sqrt(2.0))), 1.0, 0.5)  # the constants of the exact GELU: x / sqrt 2, + 1, * 0.5


@pytest.mark.parametrize("factor_first", [False, True])
def test_decomposed_gelu_matches_the_port_bit_for_bit(factor_first):
    """shaders/elementwise.rs:71-118: every step rounded on its own, both orders of the closing products;
    exp spelled in IEEE operations, so the CPU port and the kernel give the same bits."""
    x = cases.rng_for(3, 7).standard_normal((1000, 4096), dtype=np.float32) * np.float32(3.0)
    x.reshape(-1)[:8] = [0.0, -0.0, 1e-30, -1e-30, 12.5, -12.5, 40.0, -40.0]
    # arguments whose exp(-a * a) is a denormal or underflows (a * a from 82 to 110): the scaling by 2^e in two steps
    sweep = np.linspace(12.8, 14.9, 512, dtype=np.float32)
    x.reshape(-1)[8:8 + 512] = sweep
    x.reshape(-1)[520:520 + 512] = -sweep
    got = host(ctx().decomposed_gelu(dev(x), *GELU, factor_first=factor_first))
    want = orc.decomposed_gelu(x, *GELU, factor_first=factor_first)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ref = np.array([0.5 * v * (1.0 + math.erf(v / math.sqrt(2.0))) for v in x.reshape(-1)[:4096].astype(np.float64)])
    assert np.abs(got.reshape(-1)[:4096] - ref).max() < 2e-6  # the five-term erf is good to 1.5e-7, times |x|


@pytest.mark.parametrize("shape", [(1000, 4096), (3, 77), (1,)])
def test_decomposed_gelu_quantize_equals_the_two_nodes(shape):
    """interp.rs:9125-9150: the fused node's bytes, scale and zero point are those of DecomposedGelu followed
    by DynamicQuantizeLinear - on the device, and in the CPU port."""
    x = (cases.rng_for(3, 8).standard_normal(shape, dtype=np.float32) * np.float32(2.0)).astype(np.float32)
    y, s, z = ctx().decomposed_gelu_quantize(dev(x), *GELU)
    # a whole number of 16-byte vectors that fits the registers of one block per SM: one launch
    assert ctx().last_kernel == ("dql_one_pass" if x.size % 4 == 0 else "dql_quantize")
    g = ctx().decomposed_gelu(dev(x), *GELU)
    y2, s2, z2 = ctx().dynamic_quantize(g)
    assert np.array_equal(host(y), host(y2)) and float(s) == float(s2) and int(z) == int(z2)
    want_y, want_s, want_z = orc.decomposed_gelu_quantize(x, *GELU)
    assert np.array_equal(host(y), want_y) and float(s) == float(want_s) and int(z) == want_z


def test_decomposed_gelu_quantize_of_nothing():
    y, s, z = ctx().decomposed_gelu_quantize(torch.empty((0, 8), device="cuda"), *GELU)
    ctx().flush()
    assert float(s) == 1.0 and int(z) == 0 and y.numel() == 0
