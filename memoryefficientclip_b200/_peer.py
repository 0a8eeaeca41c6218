"""Shard transport of the ring over peer memory: each rank PUBLISHES its own shard in a buffer
the other ranks of the node have mapped (CUDA IPC), and a rank that needs shard j at ring step
s fetches it from its owner with a device-to-device cudaMemcpyAsync on a copy stream.

Why not NCCL send/recv for the shards: an NCCL transfer is a kernel and needs SMs, while the
persistent tile kernels hold every SM of the GPU (227 KiB of shared memory per CTA), so a
send/recv queued next to them starts only when a tile kernel ends, i.e. the transfer is not
hidden under the MMAs but runs in the gaps between kernels.  Measured on 8 GPUs at global
B = 131072, D = 768: 1.8 ms of a 14.5 ms step were spent waiting for shards.  Copy engines need
no SM.

Ordering between the processes comes from collectives the ring issues anyway:
  * a rank's publish is followed by a one-word all-reduce on the copy stream; a fetch is queued
    behind it, so it starts only after EVERY rank has published (the all-reduce completes
    nowhere before all ranks have contributed, and each contributes after its publish);
  * there are two publish slots, used alternately by successive forwards.  A slot is
    overwritten two forwards later; by then every rank has passed the next forward's all-reduce,
    which it enters only after the fetches of its previous forward and backward have completed
    (stream order), and every backward ends with a collective behind its fetches (the all-reduce
    that closes the partial-gradient exchange, or one of its own), so a backward that runs directly
    before the overwriting forward is ordered too.  A backward must run before the second-next
    forward of the same module and shapes (checked: RuntimeError otherwise).
No kernel ever reads a peer's memory: a shard always lands in a local buffer first.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


_opened = {}       # (device index, handle bytes) -> base address of the mapping in this process


def _map_everywhere(local: torch.Tensor, group, rank: int, world: int, device):
    """Export `local` (this rank's buffer) and map every other rank's counterpart into this process.
    Returns (addresses of the buffers of all ranks in this process, ok); collective over `group`."""
    lib = _lib.load()
    handle = ctypes.create_string_buffer(64)
    offset = ctypes.c_uint64(0)
    mine = None
    try:
        with torch.cuda.device(device):
            _lib.check(lib.meclip_ipc_export(local.data_ptr(), handle, ctypes.byref(offset)))
        mine = (bytes(handle.raw), int(offset.value))
    except _lib.MeclipError:
        pass                             # e.g. an allocator whose memory cannot be exported (virtual-memory segments)
    everyone = [None] * world
    dist.all_gather_object(everyone, mine, group=group)
    addr = [0] * world
    ok = all(e is not None for e in everyone)
    try:
        if not ok:
            raise _lib.MeclipError(_lib.EUNSUPPORTED, "a rank could not export its buffer")
        for p, (h, off) in enumerate(everyone):
            if p == rank:
                addr[p] = local.data_ptr()
                continue
            # An allocation can be mapped once per process; torch may carve several of our buffers out of one
            # cudaMalloc block, which then share a handle: map it the first time, reuse the mapping afterwards.
            key = (device.index, h)
            if key not in _opened:
                base = ctypes.c_void_p()
                with torch.cuda.device(device):
                    _lib.check(lib.meclip_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(base)))
                _opened[key] = base.value
            addr[p] = _opened[key] + off
    except _lib.MeclipError:
        ok = False                       # e.g. a rank on another node: its memory cannot be mapped here
    # all ranks must agree on the transport: one that could not map a peer sends everyone back to send/recv
    answers = [None] * world
    dist.all_gather_object(answers, ok, group=group)
    return addr, all(answers)


class PeerShards:
    """Two publish slots of `rows x cols` elements on this rank, mapped by all ranks of `group`."""

    def __init__(self, group, rank: int, world: int, rows: int, cols: int, dtype, device):
        self.group, self.rank, self.world = group, rank, world
        self.shape = (rows, cols)
        self.dtype = dtype
        self.device = device
        self.slot_bytes = rows * cols * torch.empty((), dtype=dtype).element_size()
        # one allocation for both slots: one handle per rank, opened once per process
        self.local = torch.empty(2, rows, cols, dtype=dtype, device=device)
        self.comm = torch.cuda.Stream(device=device)
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.gen = 0                     # forwards published so far
        self.peer_slot0, self.ok = _map_everywhere(self.local, group, rank, world, device)

    def publish(self, shard: torch.Tensor) -> int:
        """Copy this rank's shard into the next slot (current stream).  Returns the generation to fetch from;
        call announce() before the first fetch of that generation."""
        gen = self.gen
        self.gen += 1
        self.local[gen % 2].copy_(shard)
        self._published = torch.cuda.Event()
        self._published.record()
        return gen

    def announce(self) -> None:
        """The all-reduce that tells every rank that all shards are in place, on the copy stream: fetches queued
        after this call start behind it.  Issuing a collective costs the host ~0.1 ms, so the ring calls this
        after it has queued the kernels of its first step (which work on the rank's own shard)."""
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(self._published)
            dist.all_reduce(self.flag, group=self.group)

    def fetches_done_everywhere(self) -> torch.cuda.Event:
        """The event after which every rank's fetches queued so far have completed (an all-reduce behind them)."""
        with torch.cuda.stream(self.comm):
            dist.all_reduce(self.flag, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.comm)
        return ev

    def check_live(self, gen: int) -> None:
        if self.gen > gen + 2:
            raise RuntimeError("ring (peer transport): this backward belongs to a forward whose published shard has "
                               "been overwritten by two later forwards of the same shapes; run the backward earlier "
                               "or set MECLIP_RING_TRANSPORT=nccl")

    def fetch(self, gen: int, owner: int, into: torch.Tensor, after=None) -> torch.cuda.Event:
        """Queue the copy of `owner`'s shard of generation `gen` into the local tensor `into` on the copy
        stream, behind `after` (the event that says `into` is free again); returns the completion event."""
        assert into.is_contiguous() and into.numel() * into.element_size() == self.slot_bytes
        src = self.peer_slot0[owner] + (gen % 2) * self.slot_bytes
        with torch.cuda.device(self.device):
            if after is not None:
                self.comm.wait_event(after)
            _lib.check(_lib.load().meclip_copy_async(into.data_ptr(), src, self.slot_bytes, self.comm.cuda_stream))
            ev = torch.cuda.Event()
            ev.record(self.comm)
        return ev


class PeerInbox:
    """Where the partial gradients of this rank's own shard arrive in the ring backward: world-1 fp32 buffers
    of `rows x cols`, one per ring step, which the ranks that computed the partials fill with copy-engine
    writes (a rank's partial for shard j goes straight into rank j's buffer of that step).

    No per-transfer signal is needed.  After its last push a rank joins ONE one-word all-reduce on the copy
    stream; when that completes on a rank, every rank's pushes - queued before its contribution - have
    landed, and the owner adds the world-1 buffers to its gradient in a fixed order (deterministic).
    A buffer is written again by the NEXT backward: that one starts with a collective of the ring (the
    column-sum all-gather, or an all-reduce for the losses without one) which the owner joins only after
    it has consumed the buffers (stream order), and pushes are queued behind kernels that wait for it."""

    def __init__(self, group, rank: int, world: int, rows: int, cols: int, device):
        self.group, self.rank, self.world, self.device = group, rank, world, device
        self.slot_bytes = rows * cols * 4
        self.local = torch.empty(world - 1, rows, cols, dtype=torch.float32, device=device)
        self.comm = torch.cuda.Stream(device=device)
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.addr, self.ok = _map_everywhere(self.local, group, rank, world, device)

    def push(self, step: int, partial: torch.Tensor, after) -> torch.cuda.Event:
        """Queue the copy of `partial` (computed at ring step `step` >= 1 for shard rank+step) into its owner's
        buffer of that step, behind `after` (the kernels that wrote it); returns the completion event."""
        assert 1 <= step < self.world and partial.is_contiguous() and partial.numel() * 4 == self.slot_bytes
        owner = (self.rank + step) % self.world
        dst = self.addr[owner] + (step - 1) * self.slot_bytes
        with torch.cuda.device(self.device):
            self.comm.wait_event(after)
            _lib.check(_lib.load().meclip_copy_async(dst, partial.data_ptr(), self.slot_bytes, self.comm.cuda_stream))
            ev = torch.cuda.Event()
            ev.record(self.comm)
        return ev

    def arrived(self) -> torch.cuda.Event:
        """The event after which all world-1 buffers of this rank hold this backward's partials."""
        with torch.cuda.stream(self.comm):
            dist.all_reduce(self.flag, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.comm)
        return ev


_cache = {}


def get(group, rank, world, rows, cols, dtype, device):
    """The exchange for this group and shard shape, created (collectively, once) on first use; None when
    some rank could not map a peer's buffer (the ring then falls back to send/recv on every rank)."""
    key = (id(group) if group is not None else 0, world, rows, cols, dtype, device.index)
    if key not in _cache:
        ex = PeerShards(group, rank, world, rows, cols, dtype, device)
        _cache[key] = ex if ex.ok else None
    return _cache[key]


def get_inbox(group, rank, world, rows, cols, device):
    """The partial-gradient inbox for this group and shape (collective on first use); None when peer memory
    cannot be mapped on some rank."""
    key = ("inbox", id(group) if group is not None else 0, world, rows, cols, device.index)
    if key not in _cache:
        box = PeerInbox(group, rank, world, rows, cols, device)
        _cache[key] = box if box.ok else None
    return _cache[key]
