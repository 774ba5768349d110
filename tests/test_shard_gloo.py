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


@pytest.mark.parametrize("world,n,batch", [(2, 4096, 1), (3, 1000, 4), (8, 11008, 8), (8, 96, 2), (4, 32000, 16)])
def test_packet_inbox_layout(world, n, batch):
    """CPU model of the fused exchange's inbox (all ranks in one process): every rank's packets of an
    epoch land in slots that no other (sender, half) uses, fit the area sized by band_slots, and a
    receiver that reads them back by the same arithmetic rebuilds the full [B][N] result; packets of
    the previous epoch stay untouched in the other half."""
    from galois_b200.shard import band_slots, inbox_bytes, packet_slot, shard_rows

    slots = band_slots(n, world, batch)
    assert inbox_bytes(world, slots) == 2 * world * slots * 8
    bands = [shard_rows(n, world, r) for r in range(world)]
    assert sum(nr for _, nr in bands) == n and all(r0 % 32 == 0 for r0, _ in bands)
    rng = np.random.default_rng(world * 1000 + n + batch)
    inbox = np.zeros((world, 2 * world * slots), np.uint64)  # [receiver][packet]
    results = {}
    for epoch in (1, 2, 3):
        full = rng.standard_normal((batch, n)).astype(np.float32)
        results[epoch] = full
        for sender, (r0, nr) in enumerate(bands):
            for b in range(batch):
                idx = np.array([packet_slot(epoch, world, sender, slots, b, nr, r) for r in range(nr)], np.int64)
                if nr:
                    assert idx.max() < ((epoch & 1) * world + sender + 1) * slots  # stays inside its own area
                pk = (np.uint64(epoch) << np.uint64(32)) | full[b, r0 : r0 + nr].view(np.uint32).astype(np.uint64)
                for receiver in range(world):
                    if receiver != sender:
                        inbox[receiver, idx] = pk
        for receiver in range(world):
            got = np.full((batch, n), np.nan, np.float32)
            got[:, bands[receiver][0] : bands[receiver][0] + bands[receiver][1]] = full[:, bands[receiver][0] : bands[receiver][0] + bands[receiver][1]]
            for sender, (r0, nr) in enumerate(bands):
                if sender == receiver:
                    continue
                for b in range(batch):
                    idx = [packet_slot(epoch, world, sender, slots, b, nr, r) for r in range(nr)]
                    pk = inbox[receiver, idx]
                    assert np.all((pk >> np.uint64(32)) == epoch)
                    got[b, r0 : r0 + nr] = (pk & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32)
            assert np.array_equal(got, full)
        if epoch >= 2:
            # the other half still holds the previous epoch's packets: a peer that is one call behind can read them
            prev, (r0, nr) = epoch - 1, bands[0]
            if nr and world > 1:
                idx = [packet_slot(prev, world, 0, slots, 0, nr, r) for r in range(nr)]
                assert np.all((inbox[1, idx] >> np.uint64(32)) == prev)
