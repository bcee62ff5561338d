"""Edge cases through the C ABI: empty tensors, refusals before any launch, and inputs that make an
operator leave its fast path (unaligned pointers, ragged sizes)."""
import numpy as np
import pytest
import torch

import cases
import oracle as orc
import ovk_b200
from gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu


def nbits_weight(k, n, bs, seed=50):
    a, nib, zp, scale = cases.nbits_synthetic(seed, 1, k, n, bs)
    w = ctx().nbits_prepack(dev(orc.pack_nibbles(nib, bs)), dev(scale.reshape(-1)), dev(orc.pack_zero_points(zp)), n, k, bs)
    return w, (nib, zp, scale)


def test_empty_inputs_launch_nothing():
    """Zero rows, zero indices, zero images: status OK, no kernel, outputs of the right (empty) shape."""
    w, _ = nbits_weight(64, 32, 32)
    mw = ctx().mmi_prepack(dev(cases.lcg_bytes(64 * 8, 3).reshape(64, 8).view(np.int8)))
    cw = ctx().qconv_prepack(dev(cases.lcg_bytes(8 * 4 * 9, 3).reshape(8, 4, 3, 3).view(np.int8)))
    before = ctx().launches
    y = ctx().matmul_nbits(w, torch.empty((0, 64), dtype=torch.float16, device="cuda"))
    acc = ctx().matmul_integer(mw, torch.empty((0, 64), dtype=torch.uint8, device="cuda"))
    conv = ctx().conv_integer(cw, torch.empty((0, 4, 5, 5), dtype=torch.uint8, device="cuda"), pads=(1, 1, 1, 1))
    tok = ctx().argmax(torch.empty((0, 100), dtype=torch.float32, device="cuda"))
    rows = ctx().gather_block_quantized(dev(np.zeros((4, 16), dtype=np.uint8)), np.zeros((0,), dtype=np.int64),
                                        dev(np.ones((4, 1), dtype=np.float32)), None, 32)
    s = ctx().qlinear_add(torch.empty((0, 7), dtype=torch.uint8, device="cuda"), 0.1, 0,
                          torch.empty((7,), dtype=torch.uint8, device="cuda"), 0.1, 0, 0.1, 0)
    ctx().flush()
    assert ctx().launches == before
    assert tuple(y.shape) == (0, 32) and tuple(acc.shape) == (0, 8) and tuple(conv.shape) == (0, 8, 5, 5)
    assert tuple(tok.shape) == (0,) and tuple(rows.shape) == (0, 32) and tuple(s.shape) == (0, 7)


def test_refusals_come_before_any_launch():
    """Status 1 (invalid) / 2 (unsupported) with the operator's name in the message; the context stays usable."""
    b = dev(np.zeros((8, 2, 16), dtype=np.uint8))
    s = dev(np.ones(16, dtype=np.float32))
    before = ctx().launches
    for bits, bs, status in ((8, 32, ovk_b200.UNSUPPORTED), (4, 12, ovk_b200.UNSUPPORTED), (4, 0, ovk_b200.UNSUPPORTED)):
        with pytest.raises(ovk_b200.OvkError, match="MatMulNBits") as err:
            ctx().nbits_prepack(b, s, None, 8, 64, bs, bits=bits)
        assert err.value.status == status
    big_k = ctx().mmi_prepack(dev(np.zeros((33056, 16), dtype=np.int8)))
    with pytest.raises(ovk_b200.OvkError, match="overflow") as err:
        ctx().matmul_integer(big_k, dev(np.zeros((16, 33056), dtype=np.uint8)))
    assert err.value.status == ovk_b200.UNSUPPORTED
    with pytest.raises(ovk_b200.OvkError, match="ArgMax"):
        ctx().argmax(torch.zeros((3, 0), device="cuda"))
    with pytest.raises(ovk_b200.OvkError, match="QLinearAdd"):
        ctx().qlinear_add(dev(np.zeros((2, 3), dtype=np.uint8)), 0.1, 0, dev(np.zeros((2, 3), dtype=np.uint8)), 0.1, 0, 0.0, 0)
    with pytest.raises(ovk_b200.OvkError, match="GatherBlockQuantized"):
        ctx().gather_block_quantized(dev(np.zeros((4, 16), dtype=np.uint8)), np.array([0]), dev(np.ones((4, 1), dtype=np.float32)),
                                     None, 24)   # 32 columns are not a multiple of 24
    # prepack launches are the only ones made above
    assert ctx().last_kernel in ("mmi_pack_b", "nbits_decode_pack", "nbits_gemm_pack", "") or ctx().launches >= before
    ctx().flush()
    w, (nib, zp, scale) = nbits_weight(64, 32, 32)
    a = cases.rng_for(51, 0).standard_normal((1, 64), dtype=np.float32).astype(np.float16)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(zp), 64, 32, 32)
    assert_close(host(ctx().matmul_nbits(w, dev(a))), want, 1e-3, 1e-3, "after the refusals")


def test_unaligned_activations_take_the_general_paths():
    """Pointers that are not 16-byte aligned: scalar staging in the decode kernel, the one-output-per-thread
    MatMulInteger kernel, the byte-wise layout pass of the convolution - same results."""
    k, n, bs = 1152, 256, 32
    w, (nib, zp, scale) = nbits_weight(k, n, bs, seed=52)
    a = cases.rng_for(52, 9).standard_normal((1, k), dtype=np.float32).astype(np.float16)
    buf = torch.zeros(k + 8, dtype=torch.float16, device="cuda")
    buf[1:k + 1] = dev(a).reshape(-1)
    y = ctx().matmul_nbits(w, buf[1:k + 1].reshape(1, k))          # 2-byte aligned only
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert_close(host(y), want, 1e-3, 1e-3, "unaligned A")
    assert ctx().last_kernel == "nbits_decode_mma"

    m, kk, nn = 40, 96, 48
    am = cases.lcg_bytes_fast(m * kk, 5).reshape(m, kk)
    bm = cases.lcg_bytes_fast(kk * nn, 6).reshape(kk, nn).view(np.int8)
    mw = ctx().mmi_prepack(dev(bm))
    abuf = torch.zeros(m * kk + 16, dtype=torch.uint8, device="cuda")
    abuf[3:3 + m * kk] = dev(am).reshape(-1)
    acc = ctx().matmul_integer(mw, abuf[3:3 + m * kk].reshape(m, kk), dev(np.array([7], dtype=np.uint8)), None)
    assert ctx().last_kernel == "mmi_small"
    assert np.array_equal(host(acc), orc.matmul_integer(am, bm, 7, 0))

    x = cases.lcg_bytes_fast(2 * 64 * 20 * 20, 7).reshape(2, 64, 20, 20)
    wt = cases.lcg_bytes_fast(32 * 64 * 9, 8).reshape(32, 64, 3, 3).view(np.int8)
    cw = ctx().qconv_prepack(dev(wt))
    xbuf = torch.zeros(x.size + 16, dtype=torch.uint8, device="cuda")
    xbuf[1:1 + x.size] = dev(x).reshape(-1)
    got = ctx().conv_integer(cw, xbuf[1:1 + x.size].reshape(x.shape), 129, 0, pads=(1, 1, 1, 1))
    assert np.array_equal(host(got), orc.conv_integer(x, wt, 129, 0, pads=(1, 1, 1, 1)))


def test_a_device_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """Every wait inside the kernels has a limit; when one runs out the thread
    records a code in the context's status word and the kernel ends.  Here the
    wait is made to run out on purpose - one thread, a barrier nothing arrives at,
    1000 polls - and the report is followed end to end: the next flush returns
    OVK_TIMEOUT and names the wait, the flush after that is clean, and an operator
    on the same context is still exact."""
    c = ovk_b200.Context(0)
    c.selftest_device_timeout()
    with pytest.raises(ovk_b200.OvkError) as e:
        c.flush()
    assert e.value.status == ovk_b200.TIMEOUT
    assert "self-test" in e.value.message and "code 6" in e.value.message
    c.flush()  # the status word was cleared by the report
    a = cases.lcg_bytes_fast(200 * 256, 41).reshape(200, 256)
    b = cases.lcg_bytes_fast(256 * 96, 43).reshape(256, 96).view(np.int8)
    w = c.mmi_prepack(dev(b))
    got = c.matmul_integer(w, dev(a), dev(np.array([131], dtype=np.uint8)), None)
    c.flush()
    assert c.last_kernel.startswith("mmi_tc")
    assert np.array_equal(got.cpu().numpy(), orc.matmul_integer(a, b, 131, 0))
    del w
    c.close()
