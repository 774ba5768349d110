"""The exchange step of the row-sharded mat-mul over peer memory
(galois_b200_mul_mat_q4_0_f32_gather; the reference has no multi-GPU path).

On one GPU the peers are stand-ins: ordinary buffers on the same device whose arrival words the
test writes itself, so no kernel ever waits for another kernel.  With two or more GPUs the real
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
    from galois_b200.shard import shard_q4_0_bytes, shard_rows
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
    outs = [torch.full((b * n,), -7.0, device=dev.torch_device, dtype=torch.float32) for _ in range(world)]
    flags = [torch.zeros(64, device=dev.torch_device, dtype=torch.int32) for _ in range(world)]
    peers = GaloisPeers()
    peers.rank, peers.nranks = rank, world
    for p in range(world):
        peers.dst[p] = outs[p].data_ptr()
        peers.flags[p] = flags[p].data_ptr()
    dd = gb.Dim.ggml((n, b), gb.GGmlType.F32).c_struct()
    return w_band, x, ref, outs, flags, peers, dd, r0, nr


@pytest.mark.parametrize("n,k,b", [(4096, 4096, 1), (11008, 4096, 4), (4096, 11008, 2), (2048, 1024, 8), (4096, 4096, 16), (256, 64, 3)])
@pytest.mark.parametrize("world,rank", [(2, 1), (4, 2), (8, 0)])
def test_band_reaches_every_rank(dev, n, k, b, world, rank):
    import torch

    from galois_b200 import lib

    w_band, x, ref, outs, flags, peers, dd, r0, nr = _setup(dev, n, k, b, world, rank, 31 * n + k + b)
    epoch = 5
    for p in range(world):
        if p != rank:
            flags[rank][p] = epoch  # the stand-in peers "have arrived"
    torch.cuda.synchronize()
    rc = lib.galois_b200_mul_mat_q4_0_f32_gather(dev.ctx, C.c_void_p(w_band.data_ptr()), C.byref(w_band.dim().c_struct()),
                                                 C.c_void_p(x.data_ptr()), C.byref(x.dim().c_struct()), C.byref(peers), C.byref(dd), r0, epoch)
    assert rc == 0, lib.galois_b200_last_error(dev.ctx)
    dev.synchronize()
    want = ref.to_numpy()  # [b][n]
    for p in range(world):
        got = outs[p].cpu().numpy().reshape(b, n)
        assert np.array_equal(got[:, r0 : r0 + nr], want[:, r0 : r0 + nr]), f"band differs in rank {p}'s buffer"
        rest = np.delete(got, np.s_[r0 : r0 + nr], axis=1)
        assert np.all(rest == -7.0), "rows outside the band were touched"
        if p != rank:
            assert int(flags[p][rank].item()) == epoch, "arrival word not published"
            assert int(flags[p].sum().item()) == epoch, "a foreign arrival word was written"


def test_wait_runs_out_and_context_survives(dev):
    """Nothing sets the peer's arrival word: the bounded device wait gives up, the next
    synchronize reports the time-out, and the context keeps working."""
    import galois_b200 as gb
    from galois_b200 import lib

    n, k, b = 256, 256, 1
    w_band, x, ref, outs, flags, peers, dd, r0, nr = _setup(dev, n, k, b, 2, 0, 777)
    rc = lib.galois_b200_mul_mat_q4_0_f32_gather(dev.ctx, C.c_void_p(w_band.data_ptr()), C.byref(w_band.dim().c_struct()),
                                                 C.c_void_p(x.data_ptr()), C.byref(x.dim().c_struct()), C.byref(peers), C.byref(dd), r0, 1)
    assert rc == 0
    with pytest.raises(gb.GError) as e:
        dev.synchronize()
    assert e.value.code == -9  # GALOIS_B200_E_TIMEOUT
    # the band itself was computed and pushed, and later calls are unaffected
    want = ref.to_numpy()
    assert np.array_equal(outs[1].cpu().numpy().reshape(b, n)[:, r0 : r0 + nr], want[:, r0 : r0 + nr])
    out = gb.Tensor.zeros((n, b), gb.GGmlType.F32, x.device)
    w_full = w_band  # rank 0 of 2 holds rows [0, n/2)
    out2 = gb.Tensor.zeros((nr, b), gb.GGmlType.F32, x.device)
    gb.galois_matmul(w_full, x, out2)
    dev.synchronize()
    assert np.array_equal(out2.to_numpy(), want[:, :nr])
    del out


def test_argument_errors(dev):
    from galois_b200 import lib

    w_band, x, ref, outs, flags, peers, dd, r0, nr = _setup(dev, 256, 256, 1, 2, 0, 3)
    args = lambda pe, row0, ep: lib.galois_b200_mul_mat_q4_0_f32_gather(  # noqa: E731
        dev.ctx, C.c_void_p(w_band.data_ptr()), C.byref(w_band.dim().c_struct()), C.c_void_p(x.data_ptr()), C.byref(x.dim().c_struct()),
        C.byref(pe), C.byref(dd), row0, ep)
    assert args(peers, r0, 0) == -1  # epoch 0
    assert args(peers, 200, 1) == -2  # band outside the result
    peers.nranks = 9
    assert args(peers, r0, 1) == -1
    peers.nranks = 2
    peers.dst[1] = None
    assert args(peers, r0, 1) == -1


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
