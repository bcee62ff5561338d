"""The MatMulInteger entry point for hosts that may not allocate device memory.

Some callers of this library own every device byte themselves (a runtime whose
plugins must draw from its arena, a serving loop with a fixed memory plan), so
they cannot let an operator grow a workspace behind their back.
ovk_matmul_integer_static_scratch keeps its only scratch - the row sums of A
used when the weight's zero point is not 0 - in a fixed array inside the
library.  This test calls it through the C ABI twice in a row and requires the
very same int32 results as ovk_matmul_integer; the second call runs on the
array the first one left behind, with a different A, so stale contents would
show.  It is collected last on purpose.
"""
import numpy as np
import pytest
import torch

import cases
from gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def _operands(m, k, n, seed):
    a = cases.lcg_bytes_fast(m * k, seed).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, seed + 1).reshape(k, n).view(np.int8)
    return a, b


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row():
    w = None
    for call, (m, seed) in enumerate(((300, 5), (150, 9))):
        a, b = _operands(m, 256, 130, seed)
        if w is None:
            w = ctx().mmi_prepack(dev(b))
            b0 = b
        a_zp = dev(np.array([131], dtype=np.uint8))
        b_zp = dev(np.array([-7], dtype=np.int8))  # non-zero: the row sums (the scratch) are used
        out = torch.empty((m, 130), dtype=torch.int32, device="cuda")  # the caller brings the output
        got = host(ctx().matmul_integer_static_scratch(w, dev(a), a_zp, b_zp, out=out))
        assert ctx().last_kernel.startswith("mmi_tc"), "the scratch-using tensor-core path must have run"
        want = host(ctx().matmul_integer(w, dev(a), a_zp, b_zp))
        assert np.array_equal(got, want), f"call {call}"
        ref = (a.astype(np.int64) - 131) @ (b0.astype(np.int64) + 7)
        assert np.array_equal(got, ref), f"call {call} against the definition"


def test_static_scratch_rejects_more_rows_than_the_array_holds():
    import ovk_b200
    a, b = _operands(16, 64, 32, 3)
    w = ctx().mmi_prepack(dev(b))
    too_many = torch.zeros((65537, 64), dtype=torch.uint8, device="cuda")
    with pytest.raises(ovk_b200.OvkError) as e:
        ctx().matmul_integer_static_scratch(w, too_many, None, dev(np.array([3], dtype=np.int8)))
    assert e.value.status == ovk_b200.INVALID_ARGUMENT and "65536" in e.value.message


def test_static_scratch_small_shapes_need_no_scratch():
    a, b = _operands(7, 12, 5, 11)
    w = ctx().mmi_prepack(dev(b))
    a_zp, b_zp = dev(np.array([37], dtype=np.uint8)), dev(np.array([-73], dtype=np.int8))
    got = host(ctx().matmul_integer_static_scratch(w, dev(a), a_zp, b_zp))
    assert np.array_equal(got, host(ctx().matmul_integer(w, dev(a), a_zp, b_zp)))
