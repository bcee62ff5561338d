"""The MatMulInteger entry point for hosts that may not allocate device memory.

Some callers of this library own every device byte themselves (a runtime whose
plugins must draw from its arena, a serving loop with a fixed memory plan), so
they cannot let an operator grow a workspace behind their back.
ovk_matmul_integer_static_scratch keeps its only scratch - the row sums of A
used when the weight's zero point is not 0 - in a fixed array inside the
library.  This test calls it through the C ABI twice in a row and requires the
very same int32 results as ovk_matmul_integer; the second call runs on the
array the first one left behind, with a different A, so stale contents would
show.  It runs on a context of its own, whose workspace must still be empty
afterwards, and the device's free memory must not move across the second
call: a version that quietly went back to the growing workspace, or to any
other allocation, fails here.  It is collected last on purpose.
"""
import numpy as np
import pytest
import torch

import cases
import ovk_b200
from gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def _operands(m, k, n, seed):
    a = cases.lcg_bytes_fast(m * k, seed).reshape(m, k)
    b = cases.lcg_bytes_fast(k * n, seed + 1).reshape(k, n).view(np.int8)
    return a, b


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row():
    fresh = ovk_b200.Context(0)  # nothing has grown this context's workspace
    assert fresh.workspace_bytes == 0
    w = w_shared = None
    for call, (m, seed) in enumerate(((300, 5), (150, 9))):
        a, b = _operands(m, 256, 130, seed)
        if w is None:
            w = fresh.mmi_prepack(dev(b))
            w_shared = ctx().mmi_prepack(dev(b))
            b0 = b
        a_zp = dev(np.array([131], dtype=np.uint8))
        b_zp = dev(np.array([-7], dtype=np.int8))  # non-zero: the row sums (the scratch) are used
        a_dev = dev(a)
        out = torch.empty((m, 130), dtype=torch.int32, device="cuda")  # the caller brings the output
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        fresh.matmul_integer_static_scratch(w, a_dev, a_zp, b_zp, out=out)
        fresh.flush()
        free_after = torch.cuda.mem_get_info()[0]
        assert fresh.last_kernel.startswith("mmi_tc"), "the scratch-using tensor-core path must have run"
        assert fresh.workspace_bytes == 0, "the entry point grew the context's workspace"
        if call == 1:  # the first call may load the kernels' module; the second one finds everything in place
            assert free_after == free_before, "device memory was allocated during the call"
        got = out.cpu().numpy()
        want = host(ctx().matmul_integer(w_shared, a_dev, a_zp, b_zp))
        assert np.array_equal(got, want), f"call {call}"
        ref = (a.astype(np.int64) - 131) @ (b0.astype(np.int64) + 7)
        assert np.array_equal(got, ref), f"call {call} against the definition"
    del w
    fresh.close()


def test_static_scratch_rejects_more_rows_than_the_array_holds():
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
