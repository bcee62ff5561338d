"""Partitioning of the two shardable operators across the GPUs of one box.

The reference runs on one device (one VkContext per process,
crates/vk-compute/src/context.rs:685-711), so nothing here has a counterpart
there; the operator semantics are unchanged:

* MatMulNBits prefill is split by weight COLUMNS: rank r owns columns
  [n0, n1) of B / scales / zero_points (whole rows of the operator layout, so a
  shard is a plain slice), computes Y[:, n0:n1] and the shards are exchanged by
  ONE all-gather.  Shards are multiples of 16 columns (the decode panel width)
  and differ by at most one unit.
* QLinearConv is split by BATCH: images are independent, weights replicated,
  no exchange at all.
* The decode GEMV is single-GPU by design: with more ranks each runs a replica.

One process per GPU; torch.distributed (NCCL on GPUs, gloo in the CPU tests)
does the exchange.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    start: int
    count: int

    @property
    def stop(self) -> int:
        return self.start + self.count


def split_units(total: int, world: int, rank: int, unit: int = 1) -> Shard:
    """Contiguous shard of `total` items in whole `unit`s; the first
    (units % world) ranks get one unit more; the last shard absorbs a ragged tail."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    units = -(-total // unit)
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    start = min(u0 * unit, total)
    stop = min(u1 * unit, total)
    return Shard(start, stop - start)


def column_shard(n: int, world: int, rank: int) -> Shard:
    """Weight columns of rank `rank` in an N-split MatMulNBits."""
    return split_units(n, world, rank, unit=16)


def batch_shard(batch: int, world: int, rank: int) -> Shard:
    """Images of rank `rank` in a batch-split QLinearConv."""
    return split_units(batch, world, rank, unit=1)


def slice_nbits_weight(b, scales, zero_points, n_blocks: int, shard: Shard):
    """Rows [start, stop) of the operator-layout tensors: B [N, n_blocks, bs/2],
    scales [N * n_blocks], zero_points [N, ceil(n_blocks/2)] (or None)."""
    bs = b.reshape(b.shape[0], -1)[shard.start:shard.stop]
    ss = scales.reshape(-1, n_blocks)[shard.start:shard.stop].reshape(-1)
    zs = None if zero_points is None else zero_points.reshape(b.shape[0], -1)[shard.start:shard.stop]
    return bs, ss, zs


def all_gather_columns(y_shard, n: int, world: int, group=None):
    """Exchange step of the N-split: every rank contributes Y[:, n0:n1] and gets
    the full [M, N].  Shards may differ in width, so they are gathered into a
    [world, M, widest] staging buffer (one collective) and copied into place.
    Returns (y_full, staging) so that callers can reuse the staging buffer."""
    import torch
    import torch.distributed as dist

    m = y_shard.shape[0]
    widths = [column_shard(n, world, r).count for r in range(world)]
    widest = max(widths)
    if world == 1:
        return y_shard, None
    send = y_shard
    if y_shard.shape[1] != widest:
        send = torch.zeros((m, widest), dtype=y_shard.dtype, device=y_shard.device)
        send[:, :y_shard.shape[1]] = y_shard
    staging = torch.empty((world, m, widest), dtype=y_shard.dtype, device=y_shard.device)
    dist.all_gather_into_tensor(staging.view(world * m, widest), send.contiguous(), group=group)
    y = torch.empty((m, n), dtype=y_shard.dtype, device=y_shard.device)
    for r in range(world):
        s = column_shard(n, world, r)
        y[:, s.start:s.stop] = staging[r, :, :s.count]
    return y, staging


class RankFailure(RuntimeError):
    """A peer did not reach the exchange step in time."""


def ready_handshake(store, world: int, rank: int, step: int, timeout_s: float = 5.0) -> None:
    """Host-side check taken BEFORE a collective is enqueued: every rank posts a
    key for this step and waits for the others'.  A rank that died or raised
    upstream is then reported as a RankFailure on the host, and no GPU
    collective is ever left half entered (nothing here touches a device)."""
    import datetime

    store.set(f"ovk/ready/{step}/{rank}", b"1")
    missing = []
    for r in range(world):
        if r == rank:
            continue
        try:
            store.wait([f"ovk/ready/{step}/{r}"], datetime.timedelta(seconds=timeout_s))
        except Exception:
            missing.append(r)
    if missing:
        raise RankFailure(f"step {step}: ranks {missing} did not reach the exchange within {timeout_s} s")


# ---------------------------------------------------------------------------
# Exchange through peer memory: every rank's Y (and one flag block per rank) is
# mapped into every process, and the kernels store into all of them.

class DeviceBlock:
    """A device buffer from ``Context.comm_alloc`` seen as a torch tensor
    (through ``__cuda_array_interface__``; torch neither owns nor frees it)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.ptr = ptr
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}

    def tensor(self, device):
        import torch
        return torch.as_tensor(self, device=device)


def gather_handles(handle: bytes, world: int, group=None):
    """Every rank's 64-byte handle, in rank order (host plumbing: one all-gather of bytes)."""
    import torch.distributed as dist
    if world == 1:
        return [handle]
    out = [None] * world
    dist.all_gather_object(out, handle, group=group)
    return out


def peer_table(handles, rank: int, own_ptr: int, import_handle):
    """Addresses of every rank's buffer as THIS process sees them: its own
    pointer for itself, a mapping of the peer's handle for the others."""
    if not 0 <= rank < len(handles):
        raise ValueError(f"rank {rank} of {len(handles)}")
    return [own_ptr if r == rank else import_handle(h) for r, h in enumerate(handles)]


class PeerGroup:
    """The ranks of one box as one context sees them.  ``symmetric(nbytes)``
    allocates the same buffer on every rank and returns its address on each;
    the constructor does that once for the flag blocks and calls
    ``ovk_comm_init``.  Collective: every rank builds its group, and makes its
    ``symmetric`` calls, in the same order."""

    def __init__(self, ctx, rank: int, world: int, group=None):
        import ovk_b200
        self.ctx, self.rank, self.world, self.group = ctx, rank, world, group
        self._mapped, self._owned = [], []
        flags = self.symmetric(int(ovk_b200.lib().ovk_comm_flag_bytes()))
        ctx.comm_init(rank, world, flags)

    def symmetric(self, nbytes: int):
        own = self.ctx.comm_alloc(nbytes)
        self._owned.append(own)
        handles = gather_handles(self.ctx.comm_export(own), self.world, self.group)

        def mapped(h):
            p = self.ctx.comm_import(h)
            self._mapped.append(p)
            return p
        return peer_table(handles, self.rank, own, mapped)

    def close(self):
        import ovk_b200
        for p in self._mapped:
            self.ctx.comm_release(p)
        self._mapped = []
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)  # nobody frees a buffer a peer still has mapped
        for p in self._owned:
            self.ctx.check(ovk_b200.lib().ovk_free(self.ctx.h, p))
        self._owned = []


class SymmetricGroup:
    """The same as PeerGroup on buffers from ``torch.distributed._symmetric_memory``, which also
    gives a MULTICAST mapping of a buffer where the box has NVLink SHARP: an address whose stores the
    NVSwitch delivers to the same offset of every rank's buffer.  ``symmetric(nbytes)`` returns
    (addresses per rank, multicast address or 0).  torch owns the buffers; the library only gets
    addresses."""

    def __init__(self, ctx, rank: int, world: int, group=None):
        import torch.distributed as dist
        import ovk_b200
        self.ctx, self.rank, self.world = ctx, rank, world
        self.group = group if group is not None else dist.group.WORLD
        self._keep = []
        flags, _ = self.symmetric(int(ovk_b200.lib().ovk_comm_flag_bytes()))
        ctx.comm_init(rank, world, flags)

    def symmetric(self, nbytes: int):
        import torch
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        t.zero_()
        handle = symm_mem.rendezvous(t, self.group)
        self._keep.append((t, handle))
        return [int(p) for p in handle.buffer_ptrs], int(handle.multicast_ptr or 0)  # 0: the box has no NVLink SHARP

    def close(self):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        self._keep = []
