"""Row-sharding of a Q4_0 weight across the GPUs of one box.

The reference has no multi-GPU path.  Rows of a mat-mul are independent
(``dst[b][n]`` depends only on ``W[n, :]`` and ``x[b, :]``, src/op.rs:1540-1543 of
galois), so rank r of g owns a contiguous band of weight rows, every rank
holds the (tiny) activations, runs the same kernel on its band and the f32
outputs are all-gathered into ``[B][N]`` on every rank.  One process per GPU,
``torch.distributed`` (NCCL over NVLink on GPUs; gloo in the CPU tests of the
host logic).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import lib
from .tensor import Device, Dim, GError, GGmlType, Tensor


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
