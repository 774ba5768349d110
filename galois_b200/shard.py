"""Row-sharding of a Q4_0 weight across the GPUs of one box.

The reference has no multi-GPU path.  Rows of a mat-mul are independent
(``dst[b][n]`` depends only on ``W[n, :]`` and ``x[b, :]``, src/op.rs:1540-1543 of
galois), so rank r of g owns a contiguous band of weight rows, every rank
holds the (tiny) activations, runs the same kernel on its band and the f32
outputs are all-gathered into ``[B][N]`` on every rank.  One process per GPU,
``torch.distributed`` (NCCL over NVLink on GPUs; gloo in the CPU tests of the
host logic).

Two exchange steps exist.  ``PeerArena`` + ``PeerShardedMatMul``: the mat-mul
kernel itself stores its results into every rank's inbox over NVLink peer
memory as self-flagging packets and its tail collects the peers' bands (one
kernel per mat-mul at decode batches).  ``RowShardedMatMul``: NCCL all-gather, kept as
the baseline and for process groups whose ranks cannot map each other's memory.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import IPC_HANDLE_BYTES, MAX_RANKS, GaloisPeers, lib
from .tensor import Device, Dim, GError, GGmlType, Tensor, _check


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """(row0, nrows) of `rank`'s band; boundaries are multiples of 32 rows."""
    r0, nr = C.c_int64(), C.c_int64()
    rc = lib.galois_b200_shard_rows(n, world, rank, C.byref(r0), C.byref(nr))
    if rc != 0:
        raise GError(f"shard_rows({n}, {world}, {rank}): bad argument", rc)
    return r0.value, nr.value


def shard_q4_0_bytes(w_bytes: np.ndarray, n: int, k: int, world: int, rank: int) -> np.ndarray:
    """The bytes of `rank`'s band of an [N][K/32] Q4_0 weight held on the host."""
    row_bytes = k // 32 * 18
    w = np.ascontiguousarray(w_bytes).view(np.uint8).reshape(n, row_bytes)
    r0, nr = shard_rows(n, world, rank)
    return w[r0 : r0 + nr].reshape(-1)


class _RawDeviceBytes:
    """Lets torch alias memory that galois_b200_alloc returned (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerArena:
    """One device buffer per rank, mapped into every other rank of `group` (CUDA IPC over
    NVLink).  Pieces are carved out at the same offset on every rank, so a piece's address on any
    peer is that peer's base plus the offset.  Every rank must make the same sequence of
    ``alloc`` calls.  The buffer starts zeroed."""

    def __init__(self, dev, nbytes: int, group=None):
        import torch
        import torch.distributed as dist

        self.dev, self.group = dev, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= MAX_RANKS:
            raise GError(f"PeerArena: {self.world} ranks (2..{MAX_RANKS})")
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        base = C.c_void_p()
        _check(dev.ctx, lib.galois_b200_alloc(dev.ctx, self.nbytes, C.byref(base)), "PeerArena alloc")
        self.base = base.value
        self.bytes = torch.as_tensor(_RawDeviceBytes(self.base, self.nbytes), device=dev.torch_device)
        self.bytes.zero_()
        torch.cuda.synchronize(dev.torch_device)
        handle = C.create_string_buffer(IPC_HANDLE_BYTES)
        _check(dev.ctx, lib.galois_b200_ipc_export(dev.ctx, C.c_void_p(self.base), handle), "ipc_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.bases = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self.base)
                continue
            ptr = C.c_void_p()
            _check(dev.ctx, lib.galois_b200_ipc_import(dev.ctx, h, C.byref(ptr)), f"ipc_import (rank {r})")
            self.bases.append(ptr.value)
        dist.barrier(group=group)  # every rank has zeroed its buffer and mapped its peers
        self._top = 0

    def alloc(self, nbytes: int) -> int:
        """Offset in bytes of a new 256-byte aligned piece."""
        off = self._top
        size = (int(nbytes) + 255) // 256 * 256
        if off + size > self.nbytes:
            raise GError(f"PeerArena: out of space ({off + size} > {self.nbytes} bytes)")
        self._top = off + size
        return off

    def close(self):
        if getattr(self, "base", None):
            import torch

            torch.cuda.synchronize(self.dev.torch_device)
            self.bytes = None
            for r, b in enumerate(self.bases):
                if r != self.rank:
                    lib.galois_b200_ipc_close(self.dev.ctx, C.c_void_p(b))
            lib.galois_b200_free(self.dev.ctx, C.c_void_p(self.base))
            self.base = None


class PeerInbox:
    """The receive areas of one fused exchange: on every rank 2 halves x `world` senders x `slots`
    8-byte packets, plus the epoch counter of the calls made on them."""

    def __init__(self, arena: PeerArena, slots: int):
        self.arena, self.slots = arena, int(slots)
        off = arena.alloc(inbox_bytes(arena.world, slots))
        self.peers = GaloisPeers()
        self.peers.rank, self.peers.nranks, self.peers.slots = arena.rank, arena.world, self.slots
        for r in range(arena.world):
            self.peers.inbox[r] = arena.bases[r] + off
        self.epoch = 0

    def next_epoch(self) -> int:
        self.epoch = (self.epoch % 0xFFFFFFFF) + 1  # 1 .. 2^32 - 1, never 0
        return self.epoch


def inbox_bytes(world: int, slots: int) -> int:
    return 2 * world * int(slots) * 8


def packet_slot(epoch: int, world: int, sender: int, slots: int, b: int, sender_rows: int, r: int) -> int:
    """Index, in 8-byte packets from the start of a receiver's inbox, of the packet carrying result
    (activation row b, row r of `sender`'s band) of call `epoch`: the inbox half alternates with the
    epoch's parity, each half has one area of `slots` packets per sender, and inside an area packets
    are ordered by activation row, then by row of the band (the layout `csrc/gather.cuh` uses)."""
    return ((epoch & 1) * world + sender) * slots + b * sender_rows + r


def band_slots(n_total: int, world: int, batch: int) -> int:
    """Packets the largest band of an N-row result sends per call."""
    return batch * max(shard_rows(n_total, world, r)[1] for r in range(world))


class PeerShardedMatMul:
    """`W` [N][K] Q4_0 sharded by rows over the ranks of the arena's group; ``forward(x)``
    returns the full ``[B][N]`` f32 result on every rank.  The exchange is part of the mat-mul
    call (``galois_b200_mul_mat_q4_0_f32_gather``): packets stored into the peers' inboxes over
    NVLink by the kernel that computes them and collected by its tail; no collective library
    call."""

    def __init__(self, w_local: Tensor, n_total: int, arena: PeerArena, max_batch: int = 1):
        self.arena = arena
        self.n_total = n_total
        self.k = w_local.dim().shape[0]
        self.r0, self.nr = shard_rows(n_total, arena.world, arena.rank)
        if w_local.dim().shape[1] != self.nr:
            raise GError(f"rank {arena.rank} holds {w_local.dim().shape[1]} rows, expected {self.nr}")
        self.w_local = w_local
        self.max_batch = max_batch
        self.inbox = PeerInbox(arena, band_slots(n_total, arena.world, max_batch))
        self._full = {}

    def forward(self, x: Tensor) -> Tensor:
        batch = x.dim().shape[1]
        if batch > self.max_batch:
            raise GError(f"batch {batch} > max_batch {self.max_batch}")
        if batch not in self._full:
            self._full[batch] = Tensor.zeros((self.n_total, batch), GGmlType.F32, x.device)
        full = self._full[batch]
        dev = x.device.gpu
        wd, xd, dd = self.w_local.dim().c_struct(), x.dim().c_struct(), full.dim().c_struct()
        rc = lib.galois_b200_mul_mat_q4_0_f32_gather(dev.ctx, C.c_void_p(self.w_local.data_ptr()), C.byref(wd), C.c_void_p(x.data_ptr()),
                                                     C.byref(xd), C.c_void_p(full.data_ptr()), C.byref(dd), self.r0,
                                                     C.byref(self.inbox.peers), self.inbox.next_epoch())
        _check(dev.ctx, rc, "mul_mat_q4_0_f32_gather")
        return full


class RowShardedMatMul:
    """`W` [N][K] Q4_0 sharded by rows over the ranks of `group`; ``forward(x)`` returns the
    full ``[B][N]`` f32 result on every rank."""

    def __init__(self, w_local: Tensor, n_total: int, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_total = n_total
        self.k = w_local.dim().shape[0]
        self.bands = [shard_rows(n_total, self.world, r) for r in range(self.world)]
        if w_local.dim().shape[1] != self.bands[self.rank][1]:
            raise GError(f"rank {self.rank} holds {w_local.dim().shape[1]} rows, expected {self.bands[self.rank][1]}")
        self.w_local = w_local
        self.equal = len({nr for _, nr in self.bands}) == 1
        self._bufs = {}

    def _buffers(self, batch: int, device: Device):
        key = batch
        if key not in self._bufs:
            nmax = max(nr for _, nr in self.bands)
            local = Tensor.zeros((nmax, batch), GGmlType.F32, device)
            gathered = Tensor.zeros((nmax, batch, self.world), GGmlType.F32, device)
            full = Tensor.zeros((self.n_total, batch), GGmlType.F32, device)
            self._bufs[key] = (local, gathered, full)
        return self._bufs[key]

    def forward(self, x: Tensor) -> Tensor:
        from .op import galois_cpy, galois_matmul

        batch = x.dim().shape[1]
        local, gathered, full = self._buffers(batch, x.device)
        r0, nr = self.bands[self.rank]
        nmax = local.dim().shape[0]
        if batch == 1 and self.equal:
            # each band is one contiguous piece of the [N] result: compute in place, gather in place
            dst = full.view((nr, 1), (1, nr, nr, nr), offset=r0)
            galois_matmul(self.w_local, x, dst)
            self.dist.all_gather_into_tensor(full.storage, full.storage[r0 : r0 + nr], group=self.group)
            return full
        dst = local.view((nr, batch), (1, nmax, nmax * batch, nmax * batch))
        galois_matmul(self.w_local, x, dst)
        self.dist.all_gather_into_tensor(gathered.storage, local.storage, group=self.group)
        # [g][B][nmax] -> [B][N]: element k of the source in ggml order goes to element k of the view
        for r, (b0, bn) in enumerate(self.bands):
            if bn == 0:
                continue
            src = gathered.view((bn, batch), (1, nmax, nmax * batch, nmax * batch), offset=r * nmax * batch)
            out = full.view((bn, batch), (1, self.n_total, self.n_total * batch, self.n_total * batch), offset=b0)
            galois_cpy(src, out)
        return full


def assemble_gathered(gathered, bands, batch: int, n_total: int):
    """Host-logic twin of the re-layout in ``RowShardedMatMul.forward`` for any torch
    device: gathered [g][B][nmax] -> [B][N].  Used by the CPU (gloo) tests."""
    import torch

    nmax = max(bn for _, bn in bands)
    g = gathered.reshape(len(bands), batch, nmax)
    out = torch.empty(batch, n_total, dtype=gathered.dtype, device=gathered.device)
    for r, (b0, bn) in enumerate(bands):
        out[:, b0 : b0 + bn] = g[r, :, :bn]
    return out
