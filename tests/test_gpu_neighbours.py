"""GatherBlockQuantized and ArgMax, the launches either side of the lm_head product."""
import numpy as np
import pytest
import torch

import cases
import oracle as orc
import ovk_b200
from gpu_util import ctx, dev, host
from test_oracle_golden import gbq_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,bs,indices", [
    (64, 1152, 32, [[37]]),                 # tests/gather_block_quantized.rs:163-172
    (32, 128, 32, [[0, 31, 7, 7, 1]]),      # :175-183
    (16, 64, 16, [-1, -16, 3]),             # :186-194
    (9, 80, 16, [8, 0, 5]),                 # :197-207: three bytes of zero points per row
    (12, 36, 6, [11, 0, -2]),               # a block that is not a whole word: the per-element kernel
])
@pytest.mark.parametrize("on_device", [False, True])
def test_gather_reference_cases(rows, cols, bs, indices, on_device):
    _, _, scale, table, zpk = gbq_case(rows, cols, bs)
    idx = np.array(indices, dtype=np.int64)
    want = orc.gather_block_quantized(table, idx, scale, zpk, bs)
    got = ctx().gather_block_quantized(dev(table), dev(idx) if on_device else idx, dev(scale), dev(zpk), bs)
    ctx().flush()
    assert got.dtype == torch.float32 and tuple(got.shape) == want.shape
    assert np.array_equal(host(got), want)
    assert ctx().last_kernel == ("gather_block_quantized" if bs % 8 == 0 else "gather_block_quantized_elem")


def test_gather_embedding_row_fp16_scales_and_output():
    """The decode step's use: one row of a wide table, f16 scales, f16 out, int32 indices on the device."""
    rng = cases.rng_for(31, 0)
    rows, cols, bs = 4096, 1152, 32
    table = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scale = rng.uniform(0.002, 0.02, size=(rows, cols // bs)).astype(np.float16)
    zpk = rng.integers(0, 256, size=(rows, (cols // bs + 1) // 2), dtype=np.uint8)
    idx = np.array([4095, 0, 1234], dtype=np.int32)
    want = orc.gather_block_quantized(table, idx.astype(np.int64), scale, zpk, bs).astype(np.float16)
    got = ctx().gather_block_quantized(dev(table), dev(idx), dev(scale), dev(zpk), bs, out_dtype=torch.float16)
    assert np.array_equal(host(got).view(np.uint16), want.view(np.uint16))
    no_zp = ctx().gather_block_quantized(dev(table), dev(idx), dev(scale), None, bs)
    assert np.array_equal(host(no_zp), orc.gather_block_quantized(table, idx.astype(np.int64), scale, None, bs))


def test_gather_refuses_a_host_index_outside_the_table_before_launching():
    """interp.rs:2908-2911."""
    _, _, scale, table, zpk = gbq_case(16, 64, 16)
    before = ctx().launches
    with pytest.raises(ovk_b200.OvkError, match="outside the 16-row table"):
        ctx().gather_block_quantized(dev(table), np.array([3, 16]), dev(scale), dev(zpk), 16)
    assert ctx().launches == before


def test_gather_reports_a_device_index_outside_the_table_at_the_next_flush():
    _, _, scale, table, zpk = gbq_case(16, 64, 16)
    idx = np.array([3, 16, -17, 5], dtype=np.int64)
    got = ctx().gather_block_quantized(dev(table), dev(idx), dev(scale), dev(zpk), 16)
    with pytest.raises(ovk_b200.OvkError, match="outside the table") as err:
        ctx().flush()
    assert err.value.status == ovk_b200.INVALID_ARGUMENT
    want = orc.gather_block_quantized(table, np.array([3, 5]), scale, zpk, 16)
    g = host(got)
    assert np.array_equal(g[[0, 3]], want) and not g[[1, 2]].any()
    ctx().flush()  # the report is not sticky


def pseudo(n, seed):
    return cases.rng_for(32, seed).standard_normal(n, dtype=np.float32)


def test_argmax_vocabulary_wide_row_is_split():
    """tests/argmax.rs:90-104: one row of 151936, the maximum planted at 140003."""
    x = pseudo(151936, 0)
    x[140003] = 9.5
    got = ctx().argmax(dev(x.reshape(1, 1, -1)))
    assert tuple(got.shape) == (1, 1) and got.dtype == torch.int64
    assert host(got).tolist() == [[140003]]
    assert ctx().last_kernel == "argmax"


@pytest.mark.parametrize("shape,axis", [((4, 1000), 1), ((2, 5, 3, 3), 1), ((1, 2, 8192), 2), ((300, 77), 1),
                                        ((7, 262144), 1), ((3, 1), 1)])
def test_argmax_matches_the_port(shape, axis):
    """tests/argmax.rs:110-118, :153-164, :205-234 and a batch of logit rows."""
    x = pseudo(int(np.prod(shape)), 1).reshape(shape)
    got = ctx().argmax(dev(x), axis)
    assert np.array_equal(host(got), orc.argmax(x, axis))


def test_argmax_ties_and_candidates():
    """tests/argmax.rs:126-147 and the kernels' candidate rule."""
    assert host(ctx().argmax(dev(np.full(4096, 0.5, dtype=np.float32)), 0)) == 0
    twice = np.zeros(200000, dtype=np.float32)
    twice[[70000, 190000]] = 2.0
    assert host(ctx().argmax(dev(twice), 0)) == 70000
    odd = np.array([[np.nan, -np.inf, -3.0], [-np.inf, -np.inf, np.nan]], dtype=np.float32)
    assert host(ctx().argmax(dev(odd), 1)).tolist() == [2, 0]


def test_argmax_of_fp16_logits_and_the_decode_chain():
    """lm_head -> ArgMax -> GatherBlockQuantized without leaving the device."""
    k, n, bs = 256, 4096, 32
    a, nib, zp, scale = cases.nbits_synthetic(33, 1, k, n, bs)
    bp, zpp = orc.pack_nibbles(nib, bs), orc.pack_zero_points(zp)
    w = ctx().nbits_prepack(dev(bp), dev(scale.reshape(-1)), dev(zpp), n, k, bs)
    logits = ctx().matmul_nbits(w, dev(a))
    token = ctx().argmax(logits)
    ref_logits = host(logits).astype(np.float32)
    assert host(token).tolist() == orc.argmax(ref_logits, 1).tolist()
    # the embedding table is the lm_head weight read the other way: [vocab, hidden]
    row = ctx().gather_block_quantized(dev(bp.reshape(n, k // 2)), token, dev(scale), dev(zpp), bs,
                                       out_dtype=torch.float16)
    ctx().flush()
    want = orc.gather_block_quantized(bp.reshape(n, k // 2), host(token), scale, zpp, bs).astype(np.float16)
    assert np.array_equal(host(row).view(np.uint16), want.view(np.uint16))
