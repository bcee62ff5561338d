"""DynamicQuantizeLinear parity: bit-equal scale, equal zero point, 0 differing
bytes (crates/onnx-vulkan-core/tests/dynamic_quantize.rs:60-76)."""
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
