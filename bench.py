#!/usr/bin/env python
"""Benchmark of the Q4_0 mat-mul hot path (decode skinny-GEMM at LLaMA-7B FFN shapes).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

Workload (config 2 of the benchmark): gate / up 11008x4096 and down 4096x11008 Q4_0 weights,
seeded N(0, 0.02) synthetic values, f32 N(0, 1) activations at batch B (default 1).
A *step* is one pass over a pool of `--sets` distinct FFN weight sets (3 mat-muls per
set); the pool is larger than the 126 MB L2 several times over, so every weight byte
comes from HBM.  Metric: algorithmic bytes (weights once + f32 activations once + f32
outputs once) per second, in GB/s.

One JSON line is printed by rank 0 (see the keys at the end of run_ours / run_reference).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, FFN = 4096, 11008
METRIC = "q4_0_mul_mat_hbm_gbs"
UNIT = "GB/s"
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(n: int, k: int, b: int) -> int:
    """Weights once + f32 activations once + f32 outputs once."""
    return n * (k // 32) * 18 + b * k * 4 + b * n * 4


def ffn_shapes():
    """(name, N, K) of the three FFN mat-muls."""
    return [("gate", FFN, HIDDEN), ("up", FFN, HIDDEN), ("down", HIDDEN, FFN)]


# ----------------------------------------------------------------------------- synthetic data
# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_q4_0_kernel launch at config 2, batch 1 (ncu capture,
# mean of the gate/up and down instances: 25 441 792 and 25 473 024 bytes read, 0 / 10 240 written).  A citation of the
# capture summarised in profiles/gemv_q4_0_config2_batch1.md, not a live measurement: NCU_CAPTURE_OF names the
# kernel revision it was taken on (the weight streaming of the kernel has not changed since).
NCU_DRAM_BYTES_PER_LAUNCH = (2 * 25441792 + 25473024) / 3.0
NCU_CAPTURE_OF = "gemv_q4_0_kernel with the deferred wait, grid 144 x 128, captured on the revision that introduced the hazard window"


def make_q4_0(n: int, k: int, seed: int, device):
    """Seeded N(0, 0.02) weights quantised to Q4_0 blocks ({f16 d; 16 bytes of nibbles}; element
    j in the low nibble of byte j, element j+16 in the high nibble; value (q - 8) * d) with torch
    ops.  Data generation only — not part of the measured path.  Returns uint8 [n * k/32 * 18]."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randn(n, k // 32, 32, generator=g, device=device, dtype=torch.float32) * 0.02
    idx = w.abs().argmax(dim=-1, keepdim=True)
    mx = torch.gather(w, -1, idx)
    d = mx / -8.0
    idv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp(torch.trunc(w * idv + 8.5), 0, 15).to(torch.uint8)
    packed = q[..., :16] | (q[..., 16:] << 4)
    dh = d.to(torch.float16).view(torch.uint8).reshape(n, k // 32, 2)
    return torch.cat([dh, packed], dim=-1).reshape(-1).contiguous()


class ClockSampler:
    """Polls SM clock, power and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ----------------------------------------------------------------------------- CPU arm
def cpu_pass(O, sets_host, xs, nth: int):
    """One pass of the reference's CPU mat-mul (oracle restatement) over host weight sets."""
    for ws in sets_host:
        for (name, n, k), w in zip(ffn_shapes(), ws):
            O.mul_mat_q4_0(w, xs[k], nth=nth, avx=True)


def make_host_sets(nsets: int, batch: int):
    """Host copies of `nsets` FFN weight sets + activations, generated with torch on the CPU."""
    import numpy as np
    import torch

    sets = []
    for s in range(nsets):
        ws = []
        for mi, (name, n, k) in enumerate(ffn_shapes()):
            ws.append(make_q4_0(n, k, 20261125 + 1000 * s + mi, torch.device("cpu")).numpy().reshape(n, -1))
        sets.append(ws)
    g = torch.Generator()
    g.manual_seed(77)
    xs = {k: torch.randn(batch, k, generator=g).numpy().astype(np.float32) for k in (HIDDEN, FFN)}
    return sets, xs


def time_cpu(O, sets_host, xs, nth: int, min_seconds: float, min_passes: int = 2):
    cpu_pass(O, sets_host, xs, nth)  # warm-up
    t0 = time.perf_counter()
    passes = 0
    while passes < min_passes or time.perf_counter() - t0 < min_seconds:
        cpu_pass(O, sets_host, xs, nth)
        passes += 1
    return (time.perf_counter() - t0) / passes, passes


def run_reference(args):
    """The reference's own CPU implementation of the path, timed on the host cores: the C++
    restatement of MatMul::f_q_f32_f32 + vec_dot_q8_0 (AVX2) with the reference's fixed
    4-task split, because the Rust crate cannot be built in this image."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as O

    O.build()
    build_kind = O.use_native_build()  # -march=native on this host, as the reference's README flags ask
    nsets = 4  # 304 MB of weights: larger than any host L3
    sets_host, xs = make_host_sets(nsets, args.batch)
    bytes_pass = nsets * sum(algorithmic_bytes(n, k, args.batch) for _, n, k in ffn_shapes())
    nth = 4
    for _ in range(args.warmup):
        cpu_pass(O, sets_host, xs, nth)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(O, sets_host, xs, nth)
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = bytes_pass / dt / 1e9
    sample = f"{nsets} FFN weight sets ({nsets * 3} mat-muls, {bytes_pass / 1e6:.0f} MB) per step at batch {args.batch}"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "config2: LLaMA-7B FFN decode skinny-GEMM, gate/up 11008x4096 + down 4096x11008, Q4_0 x Q8_0",
                   "batch": args.batch, "sets_per_step": nsets},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": nth, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count(), "build": f"g++ -O3 -mavx2 -mfma -mf16c ({build_kind})",
                         "parity": "unpinned: the reference cannot be built here (no Rust toolchain); C++ restatement"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import galois_b200 as gb
    from galois_b200 import lib
    from galois_b200.shard import shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    stream = torch.cuda.Stream(device)
    torch.cuda.set_stream(stream)
    dev = gb.CudaDevice(local_rank, stream)
    ctx = dev.ctx
    B, nsets = args.batch, args.sets

    # ---- resident weights: `nsets` FFN sets, row-sharded when world > 1
    shapes = ffn_shapes()
    bands = {name: shard_rows(n, world, rank) for name, n, k in shapes}
    weights = []  # [set][matrix] -> (torch uint8 buffer, galois_dim of the local band)
    for s in range(nsets):
        ws = []
        for mi, (name, n, k) in enumerate(shapes):
            r0, nr = bands[name]
            buf = make_q4_0(nr, k, 20261125 + 1000 * s + mi + 100000 * rank, device)
            ws.append((buf, gb.Dim.ggml((k, nr), gb.GGmlType.Q4_0).c_struct()))
        weights.append(ws)
    g = torch.Generator(device=device)
    g.manual_seed(77)
    xs = {k: torch.randn(B, k, generator=g, device=device, dtype=torch.float32) for k in (HIDDEN, FFN)}
    xdims = {k: gb.Dim.ggml((k, B), gb.GGmlType.F32).c_struct() for k in (HIDDEN, FFN)}
    outs, odims, fulls = {}, {}, {}
    peer_exchange = world > 1 and args.exchange == "peer"
    arena, inbox, full_dims = None, None, {}
    if peer_exchange:
        # the mat-mul kernel stores its results into every peer's inbox (IPC-mapped arena) and collects the peers' bands
        from galois_b200.shard import PeerArena, PeerInbox, band_slots, inbox_bytes

        slots = max(band_slots(n, world, B) for _, n, _ in shapes)
        arena = PeerArena(dev, inbox_bytes(world, slots) + 4096)
        inbox = PeerInbox(arena, slots)
    for name, n, k in shapes:
        nr = bands[name][1]
        outs[name] = torch.zeros(B, nr, device=device, dtype=torch.float32)
        odims[name] = gb.Dim.ggml((nr, B), gb.GGmlType.F32).c_struct()
        if peer_exchange:
            fulls[name] = torch.zeros(B, n, device=device, dtype=torch.float32)
            full_dims[name] = gb.Dim.ggml((n, B), gb.GGmlType.F32).c_struct()
        elif world > 1:
            fulls[name] = torch.zeros(world, B, nr, device=device, dtype=torch.float32)
    weight_bytes = sum(w[0].numel() for ws in weights for w in ws)
    bytes_step = nsets * sum(algorithmic_bytes(n, k, B) for _, n, k in shapes)  # whole job, all ranks
    calls_step = nsets * len(shapes)

    # every ctypes argument of a step is built once: the timed loops only make the foreign calls
    fn_mm, fn_gather = lib.galois_b200_mul_mat_q4_0_f32, lib.galois_b200_mul_mat_q4_0_f32_gather
    vp = lambda t: C.c_void_p(t.data_ptr())
    step_calls = []
    for ws in weights:
        for (name, n, k), (wbuf, wdim) in zip(shapes, ws):
            if peer_exchange:  # the exchange step is inside the mat-mul kernel: peer stores + arrival words
                step_calls.append((vp(wbuf), C.byref(wdim), vp(xs[k]), C.byref(xdims[k]), vp(fulls[name]), C.byref(full_dims[name]),
                                   bands[name][0], C.byref(inbox.peers)))
            else:
                step_calls.append((vp(wbuf), C.byref(wdim), vp(xs[k]), C.byref(xdims[k]), vp(outs[name]), C.byref(odims[name])))
    step_names = [name for ws in weights for (name, n, k) in shapes]

    def step():
        if peer_exchange:
            for a in step_calls:
                rc = fn_gather(ctx, *a, inbox.next_epoch())
                if rc != 0:
                    raise RuntimeError(f"mul_mat_q4_0 gather failed: {lib.galois_b200_last_error(ctx)} ({rc})")
            return
        for a, name in zip(step_calls, step_names):
            rc = fn_mm(ctx, *a)
            if rc != 0:
                raise RuntimeError(f"mul_mat_q4_0 failed: {lib.galois_b200_last_error(ctx)} ({rc})")
            if world > 1:  # the exchange step as an NCCL all-gather of the f32 output bands
                dist.all_gather_into_tensor(fulls[name], outs[name])

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- N > 1, outside the timed region: the sharded call against the same rank's unsharded mat-mul, bit for bit
    exchange_check = None
    if peer_exchange:
        from galois_b200.shard import PeerArena, PeerInbox, band_slots, inbox_bytes

        cases, ok = [], True
        ck_slots = max(band_slots(n, world, 16) for _, n, _ in shapes)
        ck_arena = PeerArena(dev, inbox_bytes(world, ck_slots) + 4096)
        ck_inbox = PeerInbox(ck_arena, ck_slots)
        for ci, (n, k) in enumerate(((FFN, HIDDEN), (HIDDEN, FFN))):
            w_full = make_q4_0(n, k, 515000 + ci, device)  # the same seed on every rank: the same full matrix
            r0, nr = shard_rows(n, world, rank)
            row_bytes = k // 32 * 18
            w_band = w_full[r0 * row_bytes:(r0 + nr) * row_bytes].clone()
            wd_full = gb.Dim.ggml((k, n), gb.GGmlType.Q4_0).c_struct()
            wd_band = gb.Dim.ggml((k, nr), gb.GGmlType.Q4_0).c_struct()
            for bb in (1, 8, 16):
                gx = torch.Generator(device=device)
                gx.manual_seed(516000 + bb)
                xb = torch.randn(bb, k, generator=gx, device=device, dtype=torch.float32)
                xd_, yd_ = gb.Dim.ggml((k, bb), gb.GGmlType.F32).c_struct(), gb.Dim.ggml((n, bb), gb.GGmlType.F32).c_struct()
                want = torch.zeros(bb, n, device=device, dtype=torch.float32)
                got = torch.full((bb, n), -1.0, device=device, dtype=torch.float32)
                rc = lib.galois_b200_mul_mat_q4_0_f32(ctx, C.c_void_p(w_full.data_ptr()), C.byref(wd_full), C.c_void_p(xb.data_ptr()), C.byref(xd_),
                                                      C.c_void_p(want.data_ptr()), C.byref(yd_))
                if rc == 0:
                    rc = lib.galois_b200_mul_mat_q4_0_f32_gather(ctx, C.c_void_p(w_band.data_ptr()), C.byref(wd_band), C.c_void_p(xb.data_ptr()),
                                                                 C.byref(xd_), C.c_void_p(got.data_ptr()), C.byref(yd_), r0, C.byref(ck_inbox.peers),
                                                                 ck_inbox.next_epoch())
                if rc != 0:
                    raise RuntimeError(f"exchange check failed to launch: {lib.galois_b200_last_error(ctx)} ({rc})")
                dev.synchronize()
                same = bool(torch.equal(got.view(torch.int32), want.view(torch.int32)))
                ok = ok and same
                cases.append({"n": n, "k": k, "batch": bb, "bit_identical": same})
            del w_full, w_band
        flag = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        exchange_check = {"ok": bool(flag.item() == 1), "cases": len(cases), "detail_rank0": cases,
                          "what": "gathered [B][N] of the sharded call == the same rank's unsharded mat-mul, compared as bits, on every rank"}
        dev.synchronize()
        ck_arena.close()

    sampler = ClockSampler(local_rank)
    for _ in range(max(3, args.warmup)):
        step()
    sync_all()

    # ---- `value`: whole-job throughput, inputs resident in HBM; one CUDA graph per step at N = 1
    use_graph = world == 1 and not args.no_graph  # the sharded step (with its NCCL all-gathers) runs as plain stream launches
    launches0 = dev.launch_count()
    modes0 = dev.overlap_counts()
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        launches_step = dev.launch_count() - launches0
        run_step = graph.replay
    else:
        step()
        launches_step = dev.launch_count() - launches0
        run_step = step
    modes_step = dict(zip(("wait_at_entry", "deferred_wait", "barrier"), (a - b for a, b in zip(dev.overlap_counts(), modes0))))
    for _ in range(max(3, args.warmup)):
        run_step()
    sync_all()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    h0 = time.perf_counter()
    for _ in range(args.steps):
        run_step()
    host_us_per_call = (time.perf_counter() - h0) * 1e6 / (args.steps * calls_step)  # time the host spends enqueueing, per mat-mul
    e1.record(stream)
    sync_all()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    value = bytes_step / (ms_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel: events around every mat-mul kernel launch (stream launches)
    lib.galois_b200_profile_enable(ctx, 1)
    prof_steps = max(1, min(args.steps, 4096 // calls_step))
    for _ in range(prof_steps):
        step()
    tot, cnt = C.c_double(), C.c_int64()
    lib.galois_b200_profile_read(ctx, C.byref(tot), C.byref(cnt))
    lib.galois_b200_profile_enable(ctx, 0)
    isolated_ms = tot.value / max(1, cnt.value)  # launch latency included: the events serialise consecutive launches
    local_bytes_call = sum(algorithmic_bytes(bands[name][1], k, B) for name, n, k in shapes) / len(shapes)
    peak, peak_kind = measured_peak_gbs()
    # Average launch duration of the mat-mul kernel over the timed region: consecutive launches overlap
    # (programmatic dependent launch), so it is the region's device time divided by its launches of that kernel.
    kernel_ms = ms_step / calls_step
    achieved = local_bytes_call / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else 0.0

    # ---- e2e: host buffers in, host buffers out, through the public C ABI, copies inside the timed region.
    # A step uploads the activations of all its mat-muls from pinned host memory in one galois_b200_htod,
    # runs the mat-muls on the uploaded rows (N > 1: the sharded call with its fused exchange), and reads all
    # results back into pinned host memory with one galois_b200_dtoh (which synchronises the stream).
    call_list = [(name, n, k, wbuf, wdim) for ws in weights for (name, n, k), (wbuf, wdim) in zip(shapes, ws)]
    x_off, o_off, xo, oo = [], [], 0, 0
    for name, n, k, _, _ in call_list:
        x_off.append(xo)
        o_off.append(oo)
        xo += B * k
        oo += B * n
    xh_all = torch.randn(xo, dtype=torch.float32).pin_memory()
    oh_all = torch.zeros(oo, dtype=torch.float32).pin_memory()
    xd_all = torch.zeros(xo, device=device, dtype=torch.float32)
    od_all = torch.zeros(oo, device=device, dtype=torch.float32)
    full_dims_e2e = {name: gb.Dim.ggml((n, B), gb.GGmlType.F32).c_struct() for name, n, k in shapes}

    e2e_calls = []
    for c, (name, n, k, wbuf, wdim) in enumerate(call_list):
        xp, op = C.c_void_p(xd_all.data_ptr() + 4 * x_off[c]), C.c_void_p(od_all.data_ptr() + 4 * o_off[c])
        if peer_exchange:
            e2e_calls.append((vp(wbuf), C.byref(wdim), xp, C.byref(xdims[k]), op, C.byref(full_dims_e2e[name]), bands[name][0], C.byref(inbox.peers)))
        else:
            e2e_calls.append((vp(wbuf), C.byref(wdim), xp, C.byref(xdims[k]), op, C.byref(full_dims_e2e[name])))
    e2e_in, e2e_out = (vp(xd_all), vp(xh_all), xo * 4), (vp(oh_all), vp(od_all), oo * 4)

    def e2e_step():
        rc = lib.galois_b200_htod(ctx, *e2e_in)
        for a in e2e_calls:
            if rc != 0:
                break
            rc = fn_gather(ctx, *a, inbox.next_epoch()) if peer_exchange else fn_mm(ctx, *a)
        if rc == 0:
            rc = lib.galois_b200_dtoh(ctx, *e2e_out)
        if rc != 0:
            raise RuntimeError(f"e2e step failed: {lib.galois_b200_last_error(ctx)} ({rc})")

    # The same step pipelined, as a host that streams tokens writes it: two sets of device and host buffers in turn,
    # the upload (galois_b200_htod_async) and the read-back (galois_b200_dtoh_async) on streams of their own, and the
    # host waits for the results of step i - 1 (galois_b200_dtoh_wait) after it has enqueued step i.  Every step still
    # uploads its inputs from pinned host memory and reads its results back into pinned host memory inside the
    # timed region; the copies of neighbouring steps overlap the kernels.
    xd_alt = torch.zeros(xo, device=device, dtype=torch.float32)
    od_alt = torch.zeros(oo, device=device, dtype=torch.float32)
    oh_alt = torch.zeros(oo, dtype=torch.float32).pin_memory()
    pipe_calls = [e2e_calls, []]
    for c, (name, n, k, wbuf, wdim) in enumerate(call_list):
        xp, op = C.c_void_p(xd_alt.data_ptr() + 4 * x_off[c]), C.c_void_p(od_alt.data_ptr() + 4 * o_off[c])
        if peer_exchange:
            pipe_calls[1].append((vp(wbuf), C.byref(wdim), xp, C.byref(xdims[k]), op, C.byref(full_dims_e2e[name]), bands[name][0], C.byref(inbox.peers)))
        else:
            pipe_calls[1].append((vp(wbuf), C.byref(wdim), xp, C.byref(xdims[k]), op, C.byref(full_dims_e2e[name])))
    pipe_in = [(vp(xd_all), vp(xh_all), xo * 4), (vp(xd_alt), vp(xh_all), xo * 4)]
    pipe_out = [(vp(oh_all), vp(od_all), oo * 4), (vp(oh_alt), vp(od_alt), oo * 4)]
    pipe_ticket = [None, None]
    ticket = C.c_int(0)

    def pipe_wait(p):
        if pipe_ticket[p] is not None:
            rc = lib.galois_b200_dtoh_wait(ctx, pipe_ticket[p])
            pipe_ticket[p] = None
            if rc != 0:
                raise RuntimeError(f"e2e read-back failed: {lib.galois_b200_last_error(ctx)} ({rc})")

    def pipe_step(i):
        p = i & 1
        rc = lib.galois_b200_htod_async(ctx, *pipe_in[p])
        for a in pipe_calls[p]:
            if rc != 0:
                break
            rc = fn_gather(ctx, *a, inbox.next_epoch()) if peer_exchange else fn_mm(ctx, *a)
        if rc == 0:
            rc = lib.galois_b200_dtoh_async(ctx, *pipe_out[p], C.byref(ticket))
        if rc != 0:
            raise RuntimeError(f"e2e step failed: {lib.galois_b200_last_error(ctx)} ({rc})")
        pipe_ticket[p] = ticket.value
        pipe_wait(1 - p)  # the results of the step before this one are on the host

    e2e = None
    if world == 1 or peer_exchange:
        for _ in range(3):
            e2e_step()
        sync_all()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        sync_all()
        sync_ms = e0.elapsed_time(e1)
        for i in range(4):
            pipe_step(i)
        pipe_wait(0), pipe_wait(1)
        sync_all()
        import time as _time
        t_wall0 = _time.perf_counter()
        e0.record(stream)
        for i in range(args.steps):
            pipe_step(i)
        pipe_wait(0), pipe_wait(1)  # the last results are on the host
        e1.record(stream)
        sync_all()
        wall_ms = (_time.perf_counter() - t_wall0) * 1e3
        # the read-back stream outlives the last kernel: take the longer of the device interval and the host's wall clock
        e2e_ms = max(e0.elapsed_time(e1), wall_ms)
        same = bool(torch.equal(oh_all, oh_alt))
        if world > 1:
            t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e_ms /= args.steps
        sync_ms /= args.steps
        e2e = {"value": bytes_step / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": xo * 4, "d2h_bytes_per_step": oo * 4,
               "ms_per_step": e2e_ms,
               "flow": "per step: galois_b200_htod_async of all activations (pinned), the mat-muls, galois_b200_dtoh_async of all results (pinned); "
                       "two buffer sets in turn, the host waits for step i - 1's results after enqueuing step i; timed = max(device interval, host wall clock)",
               "both_buffer_sets_hold_the_same_results": same,
               "synchronous": {"value": bytes_step / (sync_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": sync_ms,
                               "flow": "per step: one htod of all activations (pinned), the mat-muls, one dtoh of all results (pinned, synchronises)"}}
        if world > 1:
            e2e["note"] = "bytes per rank; every rank uploads the activations and reads back the full results"
    if world == 1:
        # the same bytes through the one-call-per-mat-mul host entry (upload, kernel, result, synchronise per call)
        xh = {k: torch.randn(B, k, dtype=torch.float32).pin_memory() for k in (HIDDEN, FFN)}
        oh = {name: torch.zeros(B, n, dtype=torch.float32).pin_memory() for name, n, k in shapes}

        def per_call_step():
            for ws in weights:
                for (name, n, k), (wbuf, wdim) in zip(shapes, ws):
                    rc = lib.galois_b200_mul_mat_q4_0_f32_host(ctx, C.c_void_p(wbuf.data_ptr()), C.byref(wdim),
                                                               C.c_void_p(xh[k].data_ptr()), C.byref(xdims[k]),
                                                               C.c_void_p(oh[name].data_ptr()), C.byref(odims[name]))
                    if rc != 0:
                        raise RuntimeError(f"mul_mat_q4_0_host failed: {lib.galois_b200_last_error(ctx)} ({rc})")

        pc_steps = max(3, min(args.steps, 30))
        for _ in range(3):
            per_call_step()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(pc_steps):
            per_call_step()
        e1.record(stream)
        torch.cuda.synchronize()
        pc_ms = e0.elapsed_time(e1) / pc_steps
        e2e["per_call_host_entry"] = {"value": bytes_step / (pc_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": pc_ms,
                                      "flow": "galois_b200_mul_mat_q4_0_f32_host per mat-mul: upload, kernel, result, synchronise"}
    sampler.stop()

    # ---- the other configurations of the benchmark measured beside the headline (N = 1 only; reported under "extra")
    extra = None
    if world == 1 and not args.no_extra:
        extra = {}
        # config 4: one decode step of a LLaMA-7B-shaped layer built from galois ops, 4 distinct layers in rotation
        from galois_b200.decode import DecodeLayer, LayerShape, weight_shapes
        shp = LayerShape()
        def measure_layer(fused_layer, attention_kernel=False):
            layers = []
            for li in range(4):
                wq4 = {name: make_q4_0(n, k, 31000 + 100 * li + i, device).cpu().numpy()
                       for i, (name, (n, k)) in enumerate(weight_shapes(shp).items())}
                gk = torch.Generator(device=device)
                gk.manual_seed(32000 + li)
                kc = torch.randn(shp.heads, shp.ctx, shp.head_dim, generator=gk, device=device).to(torch.float16).cpu().numpy()
                vc = torch.randn(shp.heads, shp.head_dim, shp.ctx, generator=gk, device=device).to(torch.float16).cpu().numpy()
                layers.append(DecodeLayer(dev, shp, wq4, np.ones(shp.hidden, np.float32), np.ones(shp.hidden, np.float32), kc, vc,
                                          fused=fused_layer, attention_kernel=attention_kernel))
            G = gb.Device.Gpu(dev)
            xin = gb.Tensor.from_numpy(xs[HIDDEN][:1].cpu().numpy(), gb.GGmlType.F32, G)
            post = gb.Tensor.from_numpy(np.array([shp.ctx - 1], np.int32), gb.GGmlType.I32, G)

            def layer_pass():
                for L in layers:
                    L.step(xin, post, shp.ctx - 1)

            for _ in range(3):
                layer_pass()
            torch.cuda.synchronize()
            l0 = dev.launch_count()
            lg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(lg, stream=stream):
                layer_pass()
            layer_launches = (dev.launch_count() - l0) // len(layers)
            for _ in range(3):
                lg.replay()
            torch.cuda.synchronize()
            reps = max(10, args.steps // 4)
            e0.record(stream)
            for _ in range(reps):
                lg.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            us_layer = e0.elapsed_time(e1) * 1e3 / (reps * len(layers))
            lbytes = layers[0].algorithmic_bytes()
            return {"config": "config4: hidden 4096, 32 heads x 128, FFN 11008, f16 KV cache 2048, batch 1, position 2047",
                                     "layer_steps_per_s": 1e6 / us_layer, "us_per_layer": us_layer, "kernels_per_layer": layer_launches,
                                     "algorithmic_bytes": lbytes, "hbm_gbs": lbytes / us_layer / 1e3,
                                     "frac_of_measured_hbm": lbytes / us_layer / 1e3 / peak}

        extra["decode_layer"] = measure_layer(False)       # the op-by-op sequence a galois caller writes
        extra["decode_layer_fused"] = measure_layer(True)  # stacked QKV / gate-up weights + two-op fusions, same numbers
        # ... and with rope + cache appends + scores, and soft_max + context, as two launches (galois_b200_decode_attention_f32)
        extra["decode_layer_attention_kernels"] = measure_layer(True, True)
        # the same 22-op layers as ONE persistent cooperative kernel per token (galois_b200_decode_layers_f32)
        def measure_stack(nl):
            from galois_b200.decode import DecodeStack
            layers = []
            for li in range(nl):
                wq4 = {name: make_q4_0(n, k, 31000 + 100 * li + i, device).cpu().numpy()
                       for i, (name, (n, k)) in enumerate(weight_shapes(shp).items())}
                gk = torch.Generator(device=device)
                gk.manual_seed(32000 + li)
                kc = torch.randn(shp.heads, shp.ctx, shp.head_dim, generator=gk, device=device).to(torch.float16).cpu().numpy()
                vc = torch.randn(shp.heads, shp.head_dim, shp.ctx, generator=gk, device=device).to(torch.float16).cpu().numpy()
                layers.append(DecodeLayer(dev, shp, wq4, np.ones(shp.hidden, np.float32), np.ones(shp.hidden, np.float32), kc, vc))
            stack = DecodeStack(layers)
            G = gb.Device.Gpu(dev)
            xin = gb.Tensor.from_numpy(xs[HIDDEN][:1].cpu().numpy(), gb.GGmlType.F32, G)
            post = gb.Tensor.from_numpy(np.array([shp.ctx - 1], np.int32), gb.GGmlType.I32, G)
            for _ in range(3):
                stack.step(xin, post)
            dev.synchronize()
            reps = max(20, args.steps // 4)
            e0.record(stream)
            for _ in range(reps):
                stack.step(xin, post)
            e1.record(stream)
            torch.cuda.synchronize()
            us_layer = e0.elapsed_time(e1) * 1e3 / (reps * nl)
            lbytes = layers[0].algorithmic_bytes()
            return {"config": f"config4 shapes, {nl} distinct layers per launch, stream launches", "layers_per_launch": nl,
                    "layer_steps_per_s": 1e6 / us_layer, "us_per_layer": us_layer, "kernels_per_layer": 1.0 / nl, "algorithmic_bytes": lbytes,
                    "hbm_gbs": lbytes / us_layer / 1e3, "frac_of_measured_hbm": lbytes / us_layer / 1e3 / peak}

        extra["decode_layer_persistent"] = measure_stack(8)
        extra["decode_layer_persistent_1_layer_per_launch"] = measure_stack(1)
        if not args.no_cpu:
            # the same layer step on the CPU oracle (the reference's op sequence, mat-muls on its 4 fixed tasks)
            import oracle as O2
            from oracle.layer import make_layer_inputs, oracle_layer_step

            O2.build()
            O2.use_native_build()
            li = make_layer_inputs(O2, shp, 4000)
            oracle_layer_step(O2, shp, *li, shp.ctx - 1)  # appends to its caches in place, at the same position every time
            t0, reps = time.perf_counter(), 0
            while reps < 3 or time.perf_counter() - t0 < 2.0:
                oracle_layer_step(O2, shp, *li, shp.ctx - 1)
                reps += 1
            cpu_layer_us = (time.perf_counter() - t0) / reps * 1e6
            for key in ("decode_layer", "decode_layer_fused", "decode_layer_persistent"):
                extra[key]["cpu_us_4thr"] = cpu_layer_us
                extra[key]["host_cpus"] = os.cpu_count()
        # config 3: prefill 4096 x 4096 x 512 tokens on the tcgen05 int8 path; config 2 at batch 4 and 8
        def time_mm(n, k, b, copies, prepare=False):
            ws = [make_q4_0(n, k, 33000 + c, device) for c in range(copies)]
            wdim = gb.Dim.ggml((k, n), gb.GGmlType.Q4_0).c_struct()
            if prepare:  # the one-time repack at upload: outside the timed region, like the upload itself
                for wbuf in ws:
                    if lib.galois_b200_prepare_weight_q4_0(ctx, C.c_void_p(wbuf.data_ptr()), C.byref(wdim)) != 0:
                        raise RuntimeError(f"prepare_weight failed: {lib.galois_b200_last_error(ctx)}")
            xb = torch.randn(b, k, device=device, dtype=torch.float32)
            yb = torch.zeros(b, n, device=device, dtype=torch.float32)
            xd_, yd_ = gb.Dim.ggml((k, b), gb.GGmlType.F32).c_struct(), gb.Dim.ggml((n, b), gb.GGmlType.F32).c_struct()

            def run():
                for wbuf in ws:
                    rc = lib.galois_b200_mul_mat_q4_0_f32(ctx, C.c_void_p(wbuf.data_ptr()), C.byref(wdim), C.c_void_p(xb.data_ptr()),
                                                          C.byref(xd_), C.c_void_p(yb.data_ptr()), C.byref(yd_))
                    if rc != 0:
                        raise RuntimeError(f"mul_mat_q4_0 failed: {lib.galois_b200_last_error(ctx)} ({rc})")
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg, stream=stream):
                run()
            gg.replay()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(10):
                gg.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            if prepare:
                for wbuf in ws:
                    lib.galois_b200_release_weight(ctx, C.c_void_p(wbuf.data_ptr()))
            return e0.elapsed_time(e1) * 1e3 / (10 * copies)

        # CPU arm beside every row: the oracle's restatement of MatMul::f_q_f32_f32, the reference's fixed 4 tasks
        # (src/op.rs:1438) and an all-cores variant, built -march=native on this host (README.md:33), bounded samples
        import oracle as O

        O.build()
        cpu_build = "skipped" if args.no_cpu else O.use_native_build()
        ncpu = os.cpu_count() or 1

        def cpu_mm_us(n, k, b):
            if args.no_cpu:
                return None, None
            wh = make_q4_0(n, k, 34000, torch.device("cpu")).numpy().reshape(n, -1)
            xh = torch.randn(b, k).numpy().astype(np.float32)
            res = []
            for nth in (4, ncpu):
                O.mul_mat_q4_0(wh, xh, nth=nth, avx=True)
                t0, reps = time.perf_counter(), 0
                while reps < 2 or (time.perf_counter() - t0 < 0.5 and reps < 50):
                    O.mul_mat_q4_0(wh, xh, nth=nth, avx=True)
                    reps += 1
                res.append((time.perf_counter() - t0) / reps * 1e6)
            return res[0], res[1]

        def row(config, n, k, b, us, **more):
            ab = algorithmic_bytes(n, k, b)
            c4, call = cpu_mm_us(n, k, b)
            r = {"config": config, "us": us, "hbm_gbs": ab / us / 1e3, "frac_of_measured": ab / us / 1e3 / peak, "algorithmic_bytes": ab,
                 "cpu_us_4thr": c4, "cpu_us_all_cores": call, "host_cpus": ncpu}
            r.update(more)
            return r

        extra["cpu_build"] = f"oracle port, g++ -O3 -mavx2 -mfma -mf16c, {cpu_build}; parity unpinned (the reference cannot be built here)"
        extra["config1_batch1"] = row("config1: 4096 x 4096 Q4_0 mat-vec, one activation row", 4096, 4096, 1, time_mm(4096, 4096, 1, 40))
        us = time_mm(4096, 4096, 512, 16)
        us_prep = time_mm(4096, 4096, 512, 16, prepare=True)
        ops = 2.0 * 512 * 4096 * 4096
        extra["prefill"] = row("config3: 4096 x 4096 Q4_0 weight x 512 tokens, tcgen05 kind::i8, weights prepared once at upload "
                               "(galois_b200_prepare_weight_q4_0)", 4096, 4096, 512, us_prep, int8_tops=ops / us_prep / 1e6,
                               frac_of_4500_nominal_int8_tops=ops / us_prep / 1e6 / 4500.0, us_unprepared=us,
                               int8_tops_unprepared=ops / us / 1e6)
        for bb in (1, 4, 8):
            us_g, us_d = time_mm(FFN, HIDDEN, bb, 16), time_mm(HIDDEN, FFN, bb, 16)
            ab = algorithmic_bytes(FFN, HIDDEN, bb)
            cg4, cga = cpu_mm_us(FFN, HIDDEN, bb)
            cd4, cda = cpu_mm_us(HIDDEN, FFN, bb)
            extra[f"config2_batch{bb}"] = {"config": f"config2: gate/up 11008 x 4096 and down 4096 x 11008 at batch {bb}, each shape alone over 16 weights",
                                           "us_gate_up": us_g, "us_down": us_d, "hbm_gbs": 3 * ab / (2 * us_g + us_d) / 1e3,
                                           "frac_of_measured": 3 * ab / (2 * us_g + us_d) / 1e3 / peak,
                                           "cpu_us_4thr_gate_up": cg4, "cpu_us_4thr_down": cd4, "cpu_us_all_cores_gate_up": cga,
                                           "cpu_us_all_cores_down": cda, "host_cpus": ncpu}
        us_s = time_mm(2 * FFN, HIDDEN, 1, 12)
        extra["config2_stacked_gate_up_batch1"] = {"us": us_s, "hbm_gbs": algorithmic_bytes(2 * FFN, HIDDEN, 1) / us_s / 1e3,
                                                   "note": "gate and up rows stacked into one 22016 x 4096 weight: one launch for both"}
        extra["config5_head_batch16"] = row("config5: output head 32000 x 4096 at batch 16", 32000, 4096, 16, time_mm(32000, 4096, 16, 8))
        extra["config5_ffn70b_batch16"] = row("config5: 70B-shape FFN 28672 x 8192 at batch 16", 28672, 8192, 16, time_mm(28672, 8192, 16, 4))
        # Q6K weights (the next block format on the path): 4096 x 4096 mat-vec, GPU and the CPU port side by side
        def time_q6k(n, k, b, copies):
            O.build()
            rng = np.random.default_rng(37000)
            raw = rng.integers(0, 256, size=(n * (k // 256), 210), dtype=np.uint8)
            raw[:, 208:210] = (rng.standard_normal(n * (k // 256)) * 1e-3).astype(np.float16).view(np.uint8).reshape(-1, 2)
            ws = [torch.from_numpy(np.roll(raw, c, axis=0).copy()).to(device) for c in range(copies)]
            wdim = gb.Dim.ggml((k, n), gb.GGmlType.Q6K).c_struct()
            xb = torch.randn(b, k, device=device, dtype=torch.float32)
            yb = torch.zeros(b, n, device=device, dtype=torch.float32)
            xd_, yd_ = gb.Dim.ggml((k, b), gb.GGmlType.F32).c_struct(), gb.Dim.ggml((n, b), gb.GGmlType.F32).c_struct()

            def run():
                for wbuf in ws:
                    rc = lib.galois_b200_mul_mat_q6k_f32(ctx, C.c_void_p(wbuf.data_ptr()), C.byref(wdim), C.c_void_p(xb.data_ptr()), C.byref(xd_),
                                                         C.c_void_p(yb.data_ptr()), C.byref(yd_))
                    if rc != 0:
                        raise RuntimeError(f"mul_mat_q6k failed: {lib.galois_b200_last_error(ctx)} ({rc})")
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg, stream=stream):
                run()
            gg.replay()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(10):
                gg.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            us_gpu = e0.elapsed_time(e1) * 1e3 / (10 * copies)
            cpu_us = None
            if not args.no_cpu:
                wh, xh = raw.reshape(n, -1), xb.cpu().numpy()
                O.mul_mat_q6k(wh, xh)
                t0, reps = time.perf_counter(), 0
                while reps < 2 or time.perf_counter() - t0 < 0.5:
                    O.mul_mat_q6k(wh, xh)
                    reps += 1
                cpu_us = (time.perf_counter() - t0) / reps * 1e6
            ab = n * (k // 256) * 210 + b * k * 4 + b * n * 4
            return {"config": f"Q6K weights {n} x {k} (210-byte super-blocks), batch {b}: quantiser + warp-per-row kernel", "us": us_gpu,
                    "hbm_gbs": ab / us_gpu / 1e3, "frac_of_measured": ab / us_gpu / 1e3 / peak, "algorithmic_bytes": ab, "cpu_us_4thr": cpu_us,
                    "host_cpus": ncpu}

        extra["q6k_4096x4096_batch1"] = time_q6k(4096, 4096, 1, 32)
        extra["q6k_head_32000x4096_batch1"] = time_q6k(32000, 4096, 1, 4)  # the output head of a Q4_0 GGUF model is stored as Q6K
        # the headline step again with the overlap of independent mat-vecs switched off: every kernel waits for the
        # kernel in front of it at entry, as if each mat-mul consumed its predecessor's result
        lib.galois_b200_set_overlap(ctx, 0)
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs, stream=stream):
            step()
        for _ in range(3):
            gs.replay()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(max(10, args.steps // 4)):
            gs.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        lib.galois_b200_set_overlap(ctx, 1)
        us_strict = e0.elapsed_time(e1) * 1e3 / (max(10, args.steps // 4) * calls_step)
        extra["config2_batch1_strict_stream_order"] = {
            "us_per_mat_mul": us_strict, "hbm_gbs": local_bytes_call / us_strict / 1e3, "frac_of_measured": local_bytes_call / us_strict / 1e3 / peak,
            "note": "galois_b200_set_overlap(0): the same 48 mat-vecs, each waiting at entry for the one before it (a truly dependent chain)"}
        # one launch over more than 1 GB of rows: what the GEMV kernel sustains once launch boundaries are out of the picture
        n_big = 524288  # x 2304 bytes per row of K = 4096 = 1.2 GB
        w_big = make_q4_0(n_big, HIDDEN, 36000, device)
        wd_big = gb.Dim.ggml((HIDDEN, n_big), gb.GGmlType.Q4_0).c_struct()
        y_big = torch.zeros(1, n_big, device=device, dtype=torch.float32)
        yd_big = gb.Dim.ggml((n_big, 1), gb.GGmlType.F32).c_struct()

        def big():
            rc = lib.galois_b200_mul_mat_q4_0_f32(ctx, C.c_void_p(w_big.data_ptr()), C.byref(wd_big), C.c_void_p(xs[HIDDEN].data_ptr()),
                                                  C.byref(xdims[HIDDEN]), C.c_void_p(y_big.data_ptr()), C.byref(yd_big))
            if rc != 0:
                raise RuntimeError(f"mul_mat_q4_0 failed: {lib.galois_b200_last_error(ctx)} ({rc})")
        for _ in range(3):
            big()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(10):
            big()
        e1.record(stream)
        torch.cuda.synchronize()
        us_big = e0.elapsed_time(e1) * 1e3 / 10
        ab_big = algorithmic_bytes(n_big, HIDDEN, 1)
        extra["gemv_steady_state"] = {"config": f"one launch of gemv_q4_0_kernel over {n_big} x 4096 (1.2 GB of Q4_0 rows), one activation row",
                                      "us": us_big, "hbm_gbs": ab_big / us_big / 1e3, "frac_of_measured": ab_big / us_big / 1e3 / peak}
        del w_big, y_big

    # ---- N > 1: the config-5 shapes (output head, 70B FFN; batch 16) row-sharded with the fused exchange
    if peer_exchange and not args.no_extra:
        from galois_b200.shard import PeerArena, PeerInbox, band_slots, inbox_bytes

        extra = {}
        xb16 = 16
        c5 = [("config5_head_batch16", 32000, 4096, 6), ("config5_ffn70b_batch16", 28672, 8192, 4)]
        slots5 = max(band_slots(n, world, xb16) for _, n, _, _ in c5)
        arena5 = PeerArena(dev, inbox_bytes(world, slots5) + 4096)
        inbox5 = PeerInbox(arena5, slots5)
        for key, n, k, copies in c5:
            r0, nr = shard_rows(n, world, rank)
            wsb = [make_q4_0(nr, k, 35000 + c + 100 * rank, device) for c in range(copies)]
            wdim = gb.Dim.ggml((k, nr), gb.GGmlType.Q4_0).c_struct()
            xb = torch.randn(xb16, k, device=device, dtype=torch.float32)
            yb = torch.zeros(xb16, n, device=device, dtype=torch.float32)
            xd_, yd_ = gb.Dim.ggml((k, xb16), gb.GGmlType.F32).c_struct(), gb.Dim.ggml((n, xb16), gb.GGmlType.F32).c_struct()

            calls5 = [(vp(wbuf), C.byref(wdim), vp(xb), C.byref(xd_), vp(yb), C.byref(yd_), r0, C.byref(inbox5.peers)) for wbuf in wsb]

            def run5():
                for a in calls5:
                    rc = fn_gather(ctx, *a, inbox5.next_epoch())
                    if rc != 0:
                        raise RuntimeError(f"mul_mat_q4_0 gather failed: {lib.galois_b200_last_error(ctx)} ({rc})")
            for _ in range(5):
                run5()
            sync_all()
            e0.record(stream)
            for _ in range(20):
                run5()
            e1.record(stream)
            sync_all()
            t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us5 = float(t.item()) * 1e3 / (20 * copies)
            extra[key] = {"us": us5, "hbm_gbs": algorithmic_bytes(n, k, xb16) / us5 / 1e3, "rows_per_rank": nr}
        dev.synchronize()
        arena5.close()

    # ---- CPU baseline (rank 0, N = 1): the oracle's restatement of the reference CPU path, 4 tasks
    cpu = None
    if world == 1 and not args.no_cpu:
        import oracle as O

        O.build()
        cpu_build_kind = O.use_native_build()  # -march=native on this host (README.md:33 of galois)
        csets = 2
        sets_host = [[w[0].cpu().numpy().reshape(shapes[i][1], -1) for i, w in enumerate(ws)] for ws in weights[:csets]]
        xs_host = {k: v.cpu().numpy() for k, v in xs.items()}
        dt, passes = time_cpu(O, sets_host, xs_host, 4, args.cpu_seconds)
        cbytes = csets * sum(algorithmic_bytes(n, k, B) for _, n, k in shapes)
        cpu = {"value": cbytes / dt / 1e9, "unit": UNIT, "cores": 4, "kind": "port",
               "sample": f"{csets} of the {nsets} FFN weight sets ({csets * 3} mat-muls, {cbytes / 1e6:.0f} MB) x {passes} passes, "
                         f"AVX2 vec_dot, the reference's fixed 4-task split", "host_cpus": os.cpu_count(),
               "build": f"g++ -O3 -mavx2 -mfma -mf16c ({cpu_build_kind})",
               "parity": "unpinned: the reference cannot be built here (no Rust toolchain); C++ restatement"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic",
            "config": {"workload": "config2: LLaMA-7B FFN decode skinny-GEMM, gate/up 11008x4096 + down 4096x11008, Q4_0 x Q8_0",
                       "batch": B, "sets_per_step": nsets, "mat_muls_per_step": calls_step,
                       "weight_bytes_resident_per_gpu": weight_bytes,
                       "l2": f"inputs larger than L2: {weight_bytes / L2_BYTES:.1f}x the 126 MB L2 streamed between reuses",
                       "launch": "cuda_graph" if use_graph else "stream", "host_us_per_mat_mul_enqueue": host_us_per_call,
                       "ordering": "stream order kept; one-row mat-vecs whose input no kernel in flight writes defer their wait "
                                   "for the kernels in front of them to their first store (galois_b200_set_overlap, default on); "
                                   "extra.config2_batch1_strict_stream_order has the same step with every kernel waiting at entry",
                       "one_row_kernels_per_step_by_ordering": modes_step,
                       "parallelism": (f"rows/{world} + " + ("packet exchange over NVLink peer memory fused into the mat-mul kernel" if peer_exchange else "nccl all_gather"))
                       if world > 1 else "single gpu"},
            "roofline": {"bound": "hbm", "kernel": "gemv_q4_0_kernel" if B <= 1 else ("mmq_skinny_kernel" if B <= 192 else "mm_q4_0_tc_kernel"), "achieved": achieved, "peak": peak, "unit": UNIT,
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         # DRAM bytes per launch from the ncu capture of this kernel on this workload (profiles/): read + write
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH if (B == 1 and world == 1) else None,
                         "traffic_source": f"ncu --set full capture summarised in profiles/gemv_q4_0_config2_batch1.md ({NCU_CAPTURE_OF})" if (B == 1 and world == 1) else None,
                         "kernel_us": kernel_ms * 1e3, "algorithmic_bytes_per_launch": local_bytes_call,
                         "timed_launches": calls_step * args.steps, "launches_per_mat_mul": launches_step / calls_step,
                         "isolated_kernel_us": isolated_ms * 1e3, "isolated_launches": cnt.value, "frac_of_8000_nominal": achieved / 8000.0},
            "gpu_launches": launches_step * args.steps,
            "clocks": sampler.summary(),
        }
        if e2e is not None:
            line["e2e"] = e2e
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if extra is not None:
            line["extra"] = extra
        if exchange_check is not None:
            line["exchange_check"] = exchange_check
        print(json.dumps(line), flush=True)
    if arena is not None:
        dev.synchronize()  # surfaces a device-side wait that ran out
        arena.close()
    if world > 1:
        dist.destroy_process_group()
    dev.close()
    if exchange_check is not None and not exchange_check["ok"]:
        raise SystemExit("exchange check failed: the sharded result differs from the unsharded mat-mul")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--sets", type=int, default=16, help="distinct FFN weight sets per step (16 -> 1.2 GB of Q4_0)")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="N > 1: how output bands travel (peer = stores over NVLink from the mat-mul kernel; nccl = all-gather)")
    ap.add_argument("--no-graph", action="store_true", help="plain stream launches instead of one CUDA graph per step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the decode-layer / prefill / batch 4-8 side measurements")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
