"""The exchange step of the row-sharded mat-mul over peer memory
(galois_b200_mul_mat_q4_0_f32_gather; the reference has no multi-GPU path).

On one GPU the peers are stand-ins: ordinary buffers on the same device, with the packets a
peer would have sent written by the test beforehand, so no kernel ever waits for another kernel.  With two or more GPUs the real
protocol runs as one process per GPU (tests/peer_gather_worker.py)."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _setup(dev, n, k, b, world, rank, seed):
    import torch

    import galois_b200 as gb
    from galois_b200._lib import GaloisPeers
    from galois_b200.shard import band_slots, shard_q4_0_bytes, shard_rows
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from peer_gather_worker import random_q4_0

    G = gb.Device.Gpu(dev)
    raw = random_q4_0(n, k, seed)
    r0, nr = shard_rows(n, world, rank)
    w_full = gb.Tensor.from_raw(raw, (k, n), gb.GGmlType.Q4_0, G)
    w_band = gb.Tensor.from_raw(shard_q4_0_bytes(raw, n, k, world, rank), (k, nr), gb.GGmlType.Q4_0, G)
    x = gb.Tensor.from_numpy(np.random.default_rng(seed + 1).standard_normal((b, k)).astype(np.float32), gb.GGmlType.F32, G)
    ref = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    gb.galois_matmul(w_full, x, ref)
    slots = band_slots(n, world, b) + 3
    inboxes = [torch.zeros(2 * world * slots, device=dev.torch_device, dtype=torch.int64) for _ in range(world)]
    peers = GaloisPeers()
    peers.rank, peers.nranks, peers.slots = rank, world, slots
    for p in range(world):
        peers.inbox[p] = inboxes[p].data_ptr()
    full = torch.full((b * n,), -7.0, device=dev.torch_device, dtype=torch.float32)
    dd = gb.Dim.ggml((n, b), gb.GGmlType.F32).c_struct()
    return w_band, x, ref, full, inboxes, peers, dd, r0, nr, slots


def _packets(values: np.ndarray, epoch: int) -> np.ndarray:
    """[b][rows] f32 -> int64 packets {f32 bits, epoch} in slot order."""
    bits = np.ascontiguousarray(values, dtype=np.float32).reshape(-1).view(np.uint32).astype(np.uint64)
    return ((np.uint64(epoch) << np.uint64(32)) | bits).view(np.int64)


def _call(dev, w_band, x, full, dd, r0, peers, epoch):
    from galois_b200 import lib

    return lib.galois_b200_mul_mat_q4_0_f32_gather(dev.ctx, C.c_void_p(w_band.data_ptr()), C.byref(w_band.dim().c_struct()),
                                                   C.c_void_p(x.data_ptr()), C.byref(x.dim().c_struct()), C.c_void_p(full.data_ptr()),
                                                   C.byref(dd), r0, C.byref(peers), epoch)


@pytest.mark.parametrize("n,k,b", [(4096, 4096, 1), (11008, 4096, 4), (4096, 11008, 2), (2048, 1024, 8), (4096, 4096, 16), (256, 64, 3)])
@pytest.mark.parametrize("world,rank,epoch", [(2, 1, 5), (4, 2, 6), (8, 0, 1)])
def test_band_goes_out_and_peers_bands_come_in(dev, n, k, b, world, rank, epoch):
    import torch

    from galois_b200 import lib
    from galois_b200.shard import shard_rows

    w_band, x, ref, full, inboxes, peers, dd, r0, nr, slots = _setup(dev, n, k, b, world, rank, 31 * n + k + b)
    want = ref.to_numpy()  # [b][n]
    # the stand-in peers "have sent": their packets of this epoch already sit in the local inbox
    half = epoch & 1
    for p in range(world):
        if p == rank:
            continue
        p0, pn = shard_rows(n, world, p)
        pk = torch.from_numpy(_packets(want[:, p0 : p0 + pn], epoch)).to(dev.torch_device)
        start = (half * world + p) * slots
        inboxes[rank][start : start + pk.numel()] = pk
    torch.cuda.synchronize()
    rc = _call(dev, w_band, x, full, dd, r0, peers, epoch)
    assert rc == 0, lib.galois_b200_last_error(dev.ctx)
    dev.synchronize()
    assert np.array_equal(full.cpu().numpy().reshape(b, n), want), "full result differs"
    mine = _packets(want[:, r0 : r0 + nr], epoch)
    for p in range(world):
        if p == rank:
            continue
        got = inboxes[p].cpu().numpy()
        start = (half * world + rank) * slots
        assert np.array_equal(got[start : start + mine.size], mine), f"packets in rank {p}'s inbox differ"
        got[start : start + mine.size] = 0
        assert not got.any(), "packets outside this rank's area of the inbox"


def test_long_rows_and_a_large_band_stay_one_wave(dev):
    """K = 20480 needs so much shared memory per CTA that only one CTA fits per SM; the sharded launch
    must then shrink to one wave of CTAs, or first-wave CTAs would poll for packets that only a second
    wave sends.  A band of 20480 rows gives every CTA of the first wave receive work."""
    import torch

    from galois_b200 import lib
    from galois_b200.shard import shard_rows

    n, k, b, world, rank, epoch = 40960, 20480, 1, 2, 1, 3
    w_band, x, ref, full, inboxes, peers, dd, r0, nr, slots = _setup(dev, n, k, b, world, rank, 4242)
    want = ref.to_numpy()
    p0, pn = shard_rows(n, world, 0)
    pk = torch.from_numpy(_packets(want[:, p0 : p0 + pn], epoch)).to(dev.torch_device)
    start = ((epoch & 1) * world + 0) * slots
    inboxes[rank][start : start + pk.numel()] = pk
    torch.cuda.synchronize()
    assert _call(dev, w_band, x, full, dd, r0, peers, epoch) == 0, lib.galois_b200_last_error(dev.ctx)
    dev.synchronize()
    assert np.array_equal(full.cpu().numpy().reshape(b, n), want)


def test_wait_runs_out_and_context_survives(dev):
    """Nothing ever fills the inbox: the bounded device wait gives up, the next synchronize
    reports the time-out, and the context keeps working."""
    import galois_b200 as gb

    n, k, b = 256, 256, 1
    w_band, x, ref, full, inboxes, peers, dd, r0, nr, slots = _setup(dev, n, k, b, 2, 0, 777)
    assert _call(dev, w_band, x, full, dd, r0, peers, 1) == 0
    with pytest.raises(gb.GError) as e:
        dev.synchronize()
    assert e.value.code == -9  # GALOIS_B200_E_TIMEOUT
    # this rank's own band was computed all the same, and later calls are unaffected
    want = ref.to_numpy()
    assert np.array_equal(full.cpu().numpy().reshape(b, n)[:, r0 : r0 + nr], want[:, r0 : r0 + nr])
    out = gb.Tensor.zeros((nr, b), gb.GGmlType.F32, x.device)
    gb.galois_matmul(w_band, x, out)  # rank 0 of 2 holds rows [0, n/2)
    dev.synchronize()
    assert np.array_equal(out.to_numpy(), want[:, :nr])


def test_argument_errors(dev):
    w_band, x, ref, full, inboxes, peers, dd, r0, nr, slots = _setup(dev, 256, 256, 1, 2, 0, 3)
    assert _call(dev, w_band, x, full, dd, r0, peers, 0) == -1  # epoch 0
    assert _call(dev, w_band, x, full, dd, 32, peers, 1) == -2  # not this rank's band
    peers.slots = 5
    assert _call(dev, w_band, x, full, dd, r0, peers, 1) == -2  # inbox too small
    peers.slots = slots
    peers.nranks = 9
    assert _call(dev, w_band, x, full, dd, r0, peers, 1) == -1
    peers.nranks = 2
    peers.inbox[1] = None
    assert _call(dev, w_band, x, full, dd, r0, peers, 1) == -1


def test_two_or_more_gpus_real_exchange():
    import torch

    ngpu = torch.cuda.device_count()
    if ngpu < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if ngpu < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29613", os.path.join(ROOT, "tests", "peer_gather_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0 and "PEER_GATHER_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


_IPC_CHILD = r"""
import ctypes as C, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import galois_b200 as gb
from galois_b200 import lib
dev = gb.CudaDevice(0)
handle = bytes.fromhex(sys.argv[2])
n = int(sys.argv[3])
ptr = C.c_void_p()
assert lib.galois_b200_ipc_import(dev.ctx, handle, C.byref(ptr)) == 0, lib.galois_b200_last_error(dev.ctx)
got = np.empty(n, np.float32)
assert lib.galois_b200_dtoh(dev.ctx, got.ctypes.data_as(C.c_void_p), ptr, 4 * n) == 0
assert np.array_equal(got, np.arange(n, dtype=np.float32)), "child read something else"
back = (2.0 * got).astype(np.float32)
assert lib.galois_b200_htod(dev.ctx, ptr, back.ctypes.data_as(C.c_void_p), 4 * n) == 0
assert lib.galois_b200_synchronize(dev.ctx) == 0
assert lib.galois_b200_ipc_close(dev.ctx, ptr) == 0
print("IPC_CHILD_OK")
"""


def test_ipc_export_import_between_processes(dev):
    """A buffer exported by this process is mapped by a second process (same GPU), read and
    rewritten there; the first process sees the new contents."""
    from galois_b200 import lib

    n = 4096
    ptr = C.c_void_p()
    assert lib.galois_b200_alloc(dev.ctx, 4 * n, C.byref(ptr)) == 0
    try:
        src = np.arange(n, dtype=np.float32)
        assert lib.galois_b200_htod(dev.ctx, ptr, src.ctypes.data_as(C.c_void_p), 4 * n) == 0
        dev.synchronize()
        handle = C.create_string_buffer(64)
        assert lib.galois_b200_ipc_export(dev.ctx, ptr, handle) == 0
        res = subprocess.run([sys.executable, "-c", _IPC_CHILD, ROOT, handle.raw.hex(), str(n)], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0 and "IPC_CHILD_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
        got = np.empty(n, np.float32)
        assert lib.galois_b200_dtoh(dev.ctx, got.ctypes.data_as(C.c_void_p), ptr, 4 * n) == 0
        assert np.array_equal(got, 2.0 * src)
        assert lib.galois_b200_ipc_export(dev.ctx, None, handle) == -1
        assert lib.galois_b200_ipc_import(dev.ctx, None, C.byref(C.c_void_p())) == -1
    finally:
        lib.galois_b200_free(dev.ctx, ptr)
