"""One rank of the multi-GPU test of the peer-memory exchange (run under torch.distributed.run by
tests/test_gpu_peer_gather.py, one process per GPU).  Every rank builds the same full Q4_0 weight
from a seed, keeps its band, and compares the gathered result of PeerShardedMatMul with the
unsharded mat-mul of the same library on its own GPU (bit for bit: a row's arithmetic does not
depend on which rows its neighbours are) and with the NCCL exchange.  Prints one line per case and
``PEER_GATHER_OK`` at the end on rank 0."""
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import galois_b200 as gb  # noqa: E402
from galois_b200.shard import PeerArena, PeerShardedMatMul, RowShardedMatMul, shard_q4_0_bytes, shard_rows  # noqa: E402


def random_q4_0(n, k, seed):
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(n * (k // 32), 18), dtype=np.uint8)
    scales = (rng.standard_normal(n * (k // 32)) * 0.01).astype(np.float16)
    raw[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    return raw.reshape(-1)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = gb.CudaDevice(local)
    G = gb.Device.Gpu(dev)
    arena = PeerArena(dev, 64 << 20)
    cases = [(11008, 4096, 1), (4096, 11008, 1), (11008, 4096, 4), (4096, 4096, 3), (11008, 4096, 8), (4096, 4096, 16), (1024, 512, 2)]
    ok = True
    for ci, (n, k, b) in enumerate(cases):
        raw = random_q4_0(n, k, 1234 + ci)
        w_full = gb.Tensor.from_raw(raw, (k, n), gb.GGmlType.Q4_0, G)
        r0, nr = shard_rows(n, world, rank)
        w_band = gb.Tensor.from_raw(shard_q4_0_bytes(raw, n, k, world, rank), (k, nr), gb.GGmlType.Q4_0, G)
        mm = PeerShardedMatMul(w_band, n, arena, max_batch=b)
        nccl = RowShardedMatMul(w_band, n)
        for it in range(3):  # several epochs, alternating result buffers
            x_np = np.random.default_rng(99 + 10 * ci + it).standard_normal((b, k)).astype(np.float32)
            x = gb.Tensor.from_numpy(x_np, gb.GGmlType.F32, G)
            ref = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
            gb.galois_matmul(w_full, x, ref)
            got = mm.forward(x).to_numpy()
            via_nccl = nccl.forward(x).to_numpy()
            want = ref.to_numpy()
            same = np.array_equal(got, want) and np.array_equal(via_nccl, want)
            ok = ok and same
            if not same:
                bad = np.argwhere(got != want)
                print(f"rank {rank} case {(n, k, b)} it {it}: MISMATCH at {len(bad)} places, first {bad[:3].tolist()}", flush=True)
        if rank == 0:
            print(f"case N={n} K={k} B={b}: {'ok' if ok else 'FAILED'}", flush=True)

    # time the two exchanges on the decode shape (stream launches, device events, max over ranks)
    n, k, b = 11008, 4096, 1
    raws = [random_q4_0(n, k, 7000 + i) for i in range(6)]
    bands = [gb.Tensor.from_raw(shard_q4_0_bytes(r, n, k, world, rank), (k, shard_rows(n, world, rank)[1]), gb.GGmlType.Q4_0, G) for r in raws]
    x = gb.Tensor.from_numpy(np.random.default_rng(5).standard_normal((b, k)).astype(np.float32), gb.GGmlType.F32, G)
    for name, cls in (("peer", lambda w: PeerShardedMatMul(w, n, arena, max_batch=b)), ("nccl", lambda w: RowShardedMatMul(w, n))):
        mms = [cls(w) for w in bands]
        for _ in range(5):
            for m in mms:
                m.forward(x)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 50
        e0.record()
        for _ in range(reps):
            for m in mms:
                m.forward(x)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            us = float(t.item()) * 1e3 / (reps * len(mms))
            print(f"timing {name}: {us:.2f} us per sharded mat-mul (N={n} K={k} B={b}, {world} GPUs)", flush=True)
    dev.synchronize()  # picks up a device-side wait that ran out
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("PEER_GATHER_OK", flush=True)
    arena.close()
    dist.destroy_process_group()
    time.sleep(0.1)
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
