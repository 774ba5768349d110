"""world_size-2 (and 3) CPU test of the row-sharding host logic over gloo: band
partition, per-rank slicing of the Q4_0 bytes, all-gather layout and re-assembly.
The per-band mat-mul itself is stood in for by the oracle (the product has no CPU
kernel); what is under test is everything around it."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, k, batch, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle as O
        from galois_b200.shard import assemble_gathered, shard_q4_0_bytes, shard_rows

        w = O.quantize_q4_0(O.fill_normal(n * k, 5, 0, 0.02).reshape(n, k))
        x = O.fill_normal(batch * k, 6).reshape(batch, k)
        bands = [shard_rows(n, world, r) for r in range(world)]
        r0, nr = bands[rank]
        mine = shard_q4_0_bytes(w, n, k, world, rank).reshape(nr, -1)
        assert np.array_equal(mine, w[r0:r0 + nr])
        local = O.mul_mat_q4_0(mine, x) if nr else np.zeros((batch, 0), np.float32)
        nmax = max(b[1] for b in bands)
        padded = np.zeros((batch, nmax), np.float32)
        padded[:, :nr] = local
        gathered = torch.empty(world * batch * nmax)
        dist.all_gather_into_tensor(gathered, torch.from_numpy(padded.reshape(-1)))
        full = assemble_gathered(gathered, bands, batch, n).numpy()
        want = O.mul_mat_q4_0(w, x)
        q.put((rank, bool(np.array_equal(full, want))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,batch", [(2, 128, 1), (2, 200, 3), (3, 100, 2)])
def test_row_sharded_gather(world, n, batch):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, 64, batch, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(world))
    assert res == [(r, True) for r in range(world)]
