"""The multi-GPU host logic on CPU: two gloo ranks partition the N-split
prefill and the batch-split convolution, compute their shards with the CPU
oracle (standing in for the kernels) and reassemble the full result; a rank
that fails before the exchange is detected on the host."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (os.path.join(ROOT, "onnx-vulkan-rs_b200"), os.path.join(ROOT, "oracle"), HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _init(rank, world, port):
    for p in (os.path.join(ROOT, "onnx-vulkan-rs_b200"), os.path.join(ROOT, "oracle"), HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _nsplit_worker(rank, world, port, out):
    _init(rank, world, port)
    import cases
    import oracle as orc
    from ovk_b200 import shard
    orc.set_num_threads(1)
    m, k, n, bs = 5, 256, 1000, 32  # 1000 columns: 63 units of 16, the last one ragged
    a, nib, zp, scale = cases.nbits_synthetic(5, m, k, n, bs, real=np.float32)
    b, z = orc.pack_nibbles(nib, bs), orc.pack_zero_points(zp)
    sh = shard.column_shard(n, world, rank)
    bs_, ss_, zs_ = shard.slice_nbits_weight(torch.from_numpy(b), torch.from_numpy(scale.reshape(-1)),
                                             torch.from_numpy(z), k // bs, sh)
    y_shard = orc.matmul_nbits(a, bs_.numpy(), ss_.numpy(), zs_.numpy(), k, sh.count, bs)
    y, _ = shard.all_gather_columns(torch.from_numpy(y_shard), n, world)
    want = orc.matmul_nbits(a, b, scale, z, k, n, bs)
    out[rank] = bool(np.array_equal(y.numpy(), want))
    dist.destroy_process_group()


def _batch_worker(rank, world, port, out):
    _init(rank, world, port)
    import cases
    import oracle as orc
    from ovk_b200 import shard
    orc.set_num_threads(1)
    x = cases.rng_for(4, 0).integers(0, 256, size=(5, 8, 9, 9), dtype=np.uint8)
    w = cases.rng_for(4, 1).integers(-127, 128, size=(4, 8, 3, 3), dtype=np.int8)
    sh = shard.batch_shard(5, world, rank)
    mine = orc.conv_integer(x[sh.start:sh.stop], w, 128, 0, pads=(1, 1, 1, 1))
    # no collective is part of the operator; the test gathers only to compare
    parts = [None] * world
    dist.all_gather_object(parts, (sh.start, mine))
    full = np.concatenate([p[1] for p in sorted(parts, key=lambda t: t[0])], axis=0)
    out[rank] = bool(np.array_equal(full, orc.conv_integer(x, w, 128, 0, pads=(1, 1, 1, 1))))
    dist.destroy_process_group()


def _failure_worker(rank, world, port, out):
    _init(rank, world, port)
    from ovk_b200 import shard
    store = dist.distributed_c10d._get_default_store()
    shard.ready_handshake(store, world, rank, step=0, timeout_s=20.0)  # both alive
    if rank == 1:
        out[rank] = "raised before the exchange"  # this rank fails upstream and never posts step 1
    else:
        try:
            shard.ready_handshake(store, world, rank, step=1, timeout_s=1.0)
            out[rank] = "no failure seen"
        except shard.RankFailure as e:
            out[rank] = str(e)
    # leave without a collective: nothing may be half entered
    dist.destroy_process_group()


def _peer_table_worker(rank, world, port, out):
    _init(rank, world, port)
    from ovk_b200 import shard
    # a 64-byte handle as cudaIpcGetMemHandle would give it, here just tagged with its rank
    handle = bytes([rank]) * 64
    handles = shard.gather_handles(handle, world)
    table = shard.peer_table(handles, rank, own_ptr=0x1000 + rank, import_handle=lambda h: 0x9000 + h[0])
    out[rank] = (handles == [bytes([r]) * 64 for r in range(world)], table)
    dist.destroy_process_group()


def _run(worker, world=2):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(worker, args=(world, _free_port(), out), nprocs=world, join=True)
    return dict(out)


def test_shards_cover_everything_once():
    from ovk_b200 import shard
    for n in (16, 17, 1000, 3584, 18944, 152064):
        for world in (1, 2, 4, 8):
            parts = [shard.column_shard(n, world, r) for r in range(world)]
            assert parts[0].start == 0 and parts[-1].stop == n
            assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
            assert all(p.start % 16 == 0 or p.count == 0 for p in parts)
            assert max(p.count for p in parts) - min(p.count for p in parts) < 32 or n < 16 * world
    parts = [shard.batch_shard(64, 8, r) for r in range(8)]
    assert [p.count for p in parts] == [8] * 8
    assert [shard.batch_shard(5, 2, r).count for r in range(2)] == [3, 2]


def test_n_split_prefill_reassembles_bit_for_bit():
    assert _run(_nsplit_worker) == {0: True, 1: True}


def test_batch_split_conv_needs_no_exchange():
    assert _run(_batch_worker) == {0: True, 1: True}


def test_a_rank_that_fails_before_the_exchange_is_reported_on_the_host():
    out = _run(_failure_worker)
    assert "ranks [1] did not reach the exchange" in out[0]


def test_handles_travel_in_rank_order_and_a_rank_keeps_its_own_pointer():
    """The host plumbing of the peer-memory exchange: one all-gather of the 64-byte
    handles; a rank's table holds its own pointer at its own index and a mapping of
    each peer's handle elsewhere."""
    out = _run(_peer_table_worker, world=3)
    for rank in range(3):
        in_order, table = out[rank]
        assert in_order
        assert table == [0x1000 + rank if r == rank else 0x9000 + r for r in range(3)]
