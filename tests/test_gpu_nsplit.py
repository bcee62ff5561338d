"""The column-split MatMulNBits prefill and its exchange, on ONE GPU.

Each rank of the split is a context of its own on device 0, with its own flag
block and its own copy of Y; the ranks run one after the other on one stream.
Kernels of different ranks never wait for each other on a single GPU, so the
flags a rank would receive from its peers are written by the test before the
rank's call (an epoch far ahead), and what is checked is everything else: that
a rank's kernel stores its column block into EVERY rank's matrix, at the widths
the shards really have (2368 and 448 columns at eight ranks, 18.5 and 3.5
weight tiles), that the assembled matrix equals the CPU port on sampled columns
and the unsplit launch, and that the flags come out as the protocol says.  The
same entry points run across processes and GPUs in bench.py --gpus N.
"""
import numpy as np
import pytest
import torch

import cases
import oracle as orc
import ovk_b200
from gpu_util import assert_close, ctx, dev
from ovk_b200 import shard

pytestmark = pytest.mark.gpu

AHEAD = 1 << 20  # an epoch no rank reaches: "this peer has long arrived"


class Ranks:
    """`world` contexts on device 0 that name each other's buffers directly (one process: no handles)."""

    def __init__(self, world, m, n, dtype=torch.float16):
        self.world, self.m, self.n = world, m, n
        self.ctxs = [ovk_b200.Context(0) for _ in range(world)]
        es = torch.empty((), dtype=dtype).element_size()
        self.flag_ptrs = [c.comm_alloc(256) for c in self.ctxs]
        self.y_ptrs = [c.comm_alloc(m * n * es) for c in self.ctxs]
        typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4"}[dtype]
        self.flags = [shard.DeviceBlock(p, (64,), "<i4").tensor("cuda") for p in self.flag_ptrs]
        self.ys = [shard.DeviceBlock(p, (m, n), typestr).tensor("cuda") for p in self.y_ptrs]
        for r, c in enumerate(self.ctxs):
            c.comm_init(r, world, self.flag_ptrs)

    def peers_have_arrived(self):
        for f in self.flags:
            f[:32] = AHEAD  # ready[16], done[16]; the CTA counter behind them stays 0
        torch.cuda.synchronize()

    def close(self):
        torch.cuda.synchronize()
        for c, fp, yp in zip(self.ctxs, self.flag_ptrs, self.y_ptrs):
            c.check(ovk_b200.lib().ovk_free(c.h, fp))
            c.check(ovk_b200.lib().ovk_free(c.h, yp))
            c.close()


_WEIGHTS = {}


def qwen_weight(k, n, bs=128):
    """Config 5 tensors (seeded), generated once per shape."""
    key = (k, n, bs)
    if key not in _WEIGHTS:
        _, nib, zp, scale = cases.nbits_synthetic(5, 1, k, n, bs, scale_lo=0.001, scale_hi=0.01)
        _WEIGHTS[key] = (nib, zp, scale, orc.pack_nibbles(nib, bs), orc.pack_zero_points(zp))
    return _WEIGHTS[key]


def run_split(world, m, k, n, bs, weight, a, y_dtype=ovk_b200.FLOAT16, dtype=torch.float16):
    nib, zp, scale, bp, zpp = weight
    ranks = Ranks(world, m, n, dtype)
    kernels = []
    a_dev = dev(a)
    n_blocks = -(-k // bs)
    bt, st, zt = torch.from_numpy(bp), torch.from_numpy(scale.reshape(-1)), torch.from_numpy(zpp)
    for r, c in enumerate(ranks.ctxs):
        sh = shard.column_shard(n, world, r)
        b_s, s_s, z_s = shard.slice_nbits_weight(bt, st, zt, n_blocks, sh)
        w = c.nbits_prepack(b_s.contiguous().cuda(), s_s.contiguous().cuda(), z_s.contiguous().cuda(), sh.count, k, bs)
        ranks.peers_have_arrived()
        c.matmul_nbits_nsplit(w, a_dev, sh.start, n, ranks.y_ptrs, y_dtype)
        c.flush()  # a wait that ran out would raise here
        kernels.append(c.last_kernel)
        # what the protocol leaves behind: this rank's epoch in its slot of every block, the CTA counter back at 0
        for f in ranks.flags:
            assert int(f[r]) == 1 and int(f[16 + r]) == 1 and int(f[32]) == 0
        del w
    return ranks, kernels


@pytest.mark.parametrize("world,m,k,n", [(2, 384, 3584, 18944), (4, 384, 3584, 18944), (8, 4096, 3584, 18944),
                                         (2, 384, 18944, 3584), (4, 384, 18944, 3584), (8, 4096, 18944, 3584)])
def test_every_rank_stores_its_columns_into_every_matrix(world, m, k, n):
    """Config 5 shapes at the shard widths of 2, 4 and 8 ranks (9472/4736/2368 and 1792/896/448 columns)."""
    bs = 128
    weight = qwen_weight(k, n, bs)
    nib, zp, scale, bp, zpp = weight
    a = cases.rng_for(5, 0).standard_normal((m, k), dtype=np.float32).astype(np.float16)
    ranks, kernels = run_split(world, m, k, n, bs, weight, a)
    assert all(kn == "comm_wait" for kn in kernels)  # the fused path ends with the wait for the peers
    full = ranks.ys[0]
    for y in ranks.ys[1:]:
        assert torch.equal(y, full), "the ranks' matrices differ"
    rows = np.arange(1, m, max(1, m // 24))
    cols = np.unique(np.r_[np.arange(3, n, 61), [shard.column_shard(n, world, r).start for r in range(world)],
                           [shard.column_shard(n, world, r).stop - 1 for r in range(world)]])
    got = full[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
    want = orc.matmul_nbits(a[rows], orc.pack_nibbles(nib[cols], bs), scale[cols], orc.pack_zero_points(zp[cols]), k,
                            cols.size, bs)
    assert_close(got, want, 1e-3, 1e-3, f"{world} ranks, {k}->{n}")
    # against the unsplit launch: the same kernel on the same columns; the K order inside an output does
    # not depend on the shard, except where a launch shares tiles' K ranges between CTAs (the sums of
    # the parts are then rounded differently), so this is a tolerance check too
    w = ctx().nbits_prepack(dev(bp), dev(scale.reshape(-1)), dev(zpp), n, k, bs)
    whole = ctx().matmul_nbits(w, dev(a))
    ctx().flush()
    diff = (whole.float() - full.float()).abs()
    bound = 1e-3 + 1e-3 * whole.float().abs()
    assert bool((diff <= bound).all())
    ranks.close()


def test_small_blocks_and_decode_rows_go_through_the_exchange_kernel():
    """Forms the fused store does not cover: the two-term-scale kernel (blocks of 32, fp16 scales) computes
    in place in the rank's own matrix, a decode-sized product in a temporary; both end in allgather_cols."""
    for m, k, n, bs in ((200, 1152, 1040, 32), (3, 1152, 1040, 32), (40, 512, 1000, 128)):
        a, nib, zp, scale = cases.nbits_synthetic(2, m, k, n, bs)
        weight = (nib, zp, scale, orc.pack_nibbles(nib, bs), orc.pack_zero_points(zp))
        world = 4
        y_f32 = bs == 128
        ranks, kernels = run_split(world, m, k, n, bs, weight, a,
                                   y_dtype=ovk_b200.FLOAT if y_f32 else ovk_b200.FLOAT16,
                                   dtype=torch.float32 if y_f32 else torch.float16)
        assert all(kn == "comm_wait" for kn in kernels)
        want = orc.matmul_nbits(a, weight[3], scale, weight[4], k, n, bs, out_dtype=np.float32 if y_f32 else None)
        for y in ranks.ys:
            assert_close(y.cpu().numpy(), want, 1e-4 if y_f32 else 1e-3, 1e-4 if y_f32 else 1e-3, f"M={m} bs={bs}")
        ranks.close()


@pytest.mark.parametrize("m,n,widths,dtype", [(37, 96, (40, 56), torch.float16), (5, 26, (7, 19), torch.float16),
                                               (64, 1024, (512, 512), torch.float32), (9, 48, (16, 32), torch.int32)])
def test_allgather_cols_on_its_own(m, n, widths, dtype):
    """Aligned blocks leave as 16-byte stores, ragged ones element by element; a block may also already sit
    in the rank's own matrix (y_shard = None)."""
    world = len(widths)
    ranks = Ranks(world, m, n, dtype)
    rng = np.random.default_rng(m * n)
    want = torch.from_numpy(rng.integers(-1000, 1000, size=(m, n)).astype(np.float32)).to(dtype)
    col = 0
    for r, (c, wd) in enumerate(zip(ranks.ctxs, widths)):
        block = want[:, col:col + wd].contiguous().cuda()
        ranks.peers_have_arrived()
        if r == 0:  # in place
            ranks.ys[0][:, col:col + wd] = block
            c.allgather_cols(None, m, wd, col, n, ranks.y_ptrs, dtype=ovk_b200._dtype_code(block))
        else:
            c.allgather_cols(block, m, wd, col, n, ranks.y_ptrs)
        c.flush()
        col += wd
    for y in ranks.ys:
        assert torch.equal(y.cpu(), want)
    ranks.close()


def test_a_peer_that_never_arrives_ends_in_a_timeout_not_a_hang():
    """The flags of rank 1 are never written.  Rank 0's exchange waits for them for the two milliseconds it
    was given, records the failure, stores nothing into the peer, and the stream goes on: flush returns
    OVK_TIMEOUT naming the peer wait, and the context still computes exactly afterwards."""
    ranks = Ranks(2, 16, 64)
    c = ranks.ctxs[0]
    c.comm_set_timeout_ms(2)
    block = torch.ones((16, 32), dtype=torch.float16, device="cuda")
    c.allgather_cols(block, 16, 32, 0, 64, ranks.y_ptrs)
    with pytest.raises(ovk_b200.OvkError) as e:
        c.flush()
    assert e.value.status == ovk_b200.TIMEOUT and "peer" in e.value.message
    assert float(ranks.ys[1].abs().sum()) == 0.0  # nothing was stored into a peer that had not said it was ready
    c.flush()
    a = cases.lcg_bytes_fast(64 * 128, 3).reshape(64, 128)
    b = cases.lcg_bytes_fast(128 * 32, 4).reshape(128, 32).view(np.int8)
    w = c.mmi_prepack(dev(b))
    got = c.matmul_integer(w, dev(a))
    c.flush()
    assert np.array_equal(got.cpu().numpy(), orc.matmul_integer(a, b, 0, 0))
    del w
    ranks.close()
