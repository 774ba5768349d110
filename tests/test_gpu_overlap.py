"""Ordering of one-row Q4_0 mat-vec kernels that overlap their predecessors (galois_b200_set_overlap).

The reference runs every op in stream order (one stream per device, src/cuda.rs:340).  The
streaming GEMV may defer its wait for the kernels in front of it when the context knows that
none of them writes its input; these tests check that the results are those of strict stream
order in every dependency pattern (read-after-write, write-after-write, write-after-read), that
they are bit-identical with the overlap switched off, and that the deferred mode is the one
that actually ran where it should."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gb():
    import galois_b200

    return galois_b200


def _weights(gb, dev, oracle, shapes, seed):
    G = gb.Device.Gpu(dev)
    out = []
    for i, (n, k) in enumerate(shapes):
        raw = oracle.quantize_q4_0(oracle.fill_normal(n * k, seed + i, 0, 0.02).reshape(n, k))
        out.append((raw, gb.Tensor.from_raw(raw, (k, n), gb.GGmlType.Q4_0, G)))
    return out


def _counts_delta(dev, before):
    now = dev.overlap_counts()
    return tuple(a - b for a, b in zip(now, before))


def test_independent_mat_vecs_defer_their_wait_and_match_serial_results(gb, dev, oracle):
    G = gb.Device.Gpu(dev)
    shapes = [(11008, 4096), (11008, 4096), (4096, 11008), (4096, 4096), (1024, 256), (300, 1024)]
    ws = _weights(gb, dev, oracle, shapes, 9100)
    xs = {k: gb.Tensor.from_numpy(oracle.fill_normal(k, 9200 + k).reshape(1, k), gb.GGmlType.F32, G) for k in (4096, 11008, 256, 1024)}

    def run():
        outs = [gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G) for n, _ in shapes]
        for _ in range(3):  # the same destinations again: write-after-write on every buffer
            for (raw, wt), (n, k), o in zip(ws, shapes, outs):
                gb.galois_matmul(wt, xs[k], o)
        return [o.to_numpy() for o in outs]

    dev.set_overlap(False)
    serial = run()
    dev.set_overlap(True)
    dev.synchronize()
    c0 = dev.overlap_counts()
    overlapped = run()
    entry, deferred, barrier = _counts_delta(dev, c0)
    for a, b, (raw, _), (n, k) in zip(serial, overlapped, ws, shapes):
        assert np.array_equal(a, b)
        from conftest import assert_close

        assert_close(b, oracle.mul_mat_q4_0(raw, xs[k].to_numpy()))
    # Tensor.zeros enqueues a torch kernel the library does not see (stream-ordered, harmless); the first
    # mat-vec after the context's last unknown op runs as a barrier, the others defer their wait
    assert deferred >= 3 * len(shapes) - 2 and entry == 0 and barrier <= 2, (entry, deferred, barrier)


def test_read_after_write_chain_waits_before_it_reads(gb, dev, oracle):
    """y1 = W1 x; y2 = W2 y1; y3 = W3 y2: each input is the output of the kernel in front of it."""
    G = gb.Device.Gpu(dev)
    (r1, w1), (r2, w2), (r3, w3) = _weights(gb, dev, oracle, [(4096, 4096), (11008, 4096), (4096, 11008)], 9300)
    x = gb.Tensor.from_numpy(oracle.fill_normal(4096, 9310).reshape(1, 4096), gb.GGmlType.F32, G)
    y1, y2, y3 = (gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G) for n in (4096, 11008, 4096))
    dev.synchronize()
    c0 = dev.overlap_counts()
    for _ in range(20):  # repeated: the chain also overwrites buffers earlier kernels of the loop read
        gb.galois_matmul(w1, x, y1)
        gb.galois_matmul(w2, y1, y2)
        gb.galois_matmul(w3, y2, y3)
    got = [t.to_numpy() for t in (y1, y2, y3)]
    entry, deferred, barrier = _counts_delta(dev, c0)
    assert barrier >= 38 and entry == 0, (entry, deferred, barrier)  # W2 and W3 always read what is being written
    # the same chain, synchronised after every op
    dev.set_overlap(False)
    try:
        z1, z2, z3 = (gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G) for n in (4096, 11008, 4096))
        gb.galois_matmul(w1, x, z1)
        dev.synchronize()
        gb.galois_matmul(w2, z1, z2)
        dev.synchronize()
        gb.galois_matmul(w3, z2, z3)
        want = [t.to_numpy() for t in (z1, z2, z3)]
    finally:
        dev.set_overlap(True)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)
    from conftest import assert_close

    assert_close(got[0], oracle.mul_mat_q4_0(r1, x.to_numpy()))


def test_write_after_write_and_write_after_read(gb, dev, oracle):
    G = gb.Device.Gpu(dev)
    (ra, wa), (rb, wb), (rc, wc) = _weights(gb, dev, oracle, [(4096, 4096), (4096, 4096), (4096, 4096)], 9400)
    x = gb.Tensor.from_numpy(oracle.fill_normal(4096, 9410).reshape(1, 4096), gb.GGmlType.F32, G)
    z = gb.Tensor.from_numpy(oracle.fill_normal(4096, 9411).reshape(1, 4096), gb.GGmlType.F32, G)
    x0 = x.to_numpy()
    y, y_old, y_new = (gb.Tensor.zeros((4096, 1), gb.GGmlType.F32, G) for _ in range(3))
    dev.synchronize()
    # write-after-write: the later kernel's result must be the one that stays
    for _ in range(25):
        gb.galois_matmul(wa, x, y)
        gb.galois_matmul(wb, x, y)
    assert np.array_equal(y.to_numpy(), _serial(gb, dev, wb, x))
    # write-after-read: y_old reads x, then x is overwritten by another mat-vec, then y_new reads the new x
    gb.galois_matmul(wa, x, y_old)
    gb.galois_matmul(wc, z, x)
    gb.galois_matmul(wa, x, y_new)
    got_old, got_new, x1 = y_old.to_numpy(), y_new.to_numpy(), x.to_numpy()
    from conftest import assert_close

    assert_close(got_old, oracle.mul_mat_q4_0(ra, x0))
    assert_close(x1, oracle.mul_mat_q4_0(rc, z.to_numpy()))
    assert_close(got_new, oracle.mul_mat_q4_0(ra, x1))


def _serial(gb, dev, wt, xt):
    dev.synchronize()
    dev.set_overlap(False)
    try:
        o = gb.Tensor.zeros((wt.dim().shape[1], 1), gb.GGmlType.F32, xt.device)
        gb.galois_matmul(wt, xt, o)
        return o.to_numpy()
    finally:
        dev.set_overlap(True)


def test_fused_forms_with_deferred_wait(gb, dev, oracle):
    """rms_norm + gain prologue and a residual that an unfinished kernel writes: the residual is read
    after the wait, the prologue's operands are checked like x."""
    G = gb.Device.Gpu(dev)
    (r1, w1), (r2, w2) = _weights(gb, dev, oracle, [(4096, 4096), (4096, 4096)], 9500)
    x = gb.Tensor.from_numpy(oracle.fill_normal(4096, 9510).reshape(1, 4096), gb.GGmlType.F32, G)
    gain = gb.Tensor.from_numpy((1.0 + 0.1 * oracle.fill_normal(4096, 9511)).reshape(1, 4096), gb.GGmlType.F32, G)
    res, out = gb.Tensor.zeros((4096, 1), gb.GGmlType.F32, G), gb.Tensor.zeros((4096, 1), gb.GGmlType.F32, G)

    def run():
        gb.galois_matmul(w1, x, res)                                        # res is still being written ...
        gb.galois_matmul_fused(w2, x, out, rms_gain=gain, eps=1e-6, res=res)  # ... when this one starts
        return out.to_numpy(), res.to_numpy()

    dev.synchronize()
    c0 = dev.overlap_counts()
    a = [run() for _ in range(10)][-1]
    assert _counts_delta(dev, c0)[1] >= 10
    dev.set_overlap(False)
    try:
        b = run()
    finally:
        dev.set_overlap(True)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    h = oracle.mul(oracle.rms_norm(x.to_numpy(), 1e-6), gain.to_numpy())
    from conftest import assert_close

    assert_close(a[0], oracle.add(a[1], oracle.mul_mat_q4_0(r2, h)))


def test_other_ops_make_the_next_mat_vec_a_barrier(gb, dev, oracle):
    """rms_norm writes h; Q waits (barrier), K and V read the same h and defer (the op-by-op layer's pattern)."""
    G = gb.Device.Gpu(dev)
    ws = _weights(gb, dev, oracle, [(4096, 4096)] * 3, 9600)
    x = gb.Tensor.from_numpy(oracle.fill_normal(4096, 9610).reshape(1, 4096), gb.GGmlType.F32, G)
    h = gb.Tensor.zeros((4096, 1), gb.GGmlType.F32, G)
    outs = [gb.Tensor.zeros((4096, 1), gb.GGmlType.F32, G) for _ in range(3)]
    dev.synchronize()
    c0 = dev.overlap_counts()
    for _ in range(10):
        gb.galois_rms_norm(x, h, 1e-6)
        for (raw, wt), o in zip(ws, outs):
            gb.galois_matmul(wt, h, o)
    got = [o.to_numpy() for o in outs]
    assert _counts_delta(dev, c0) == (0, 20, 10)
    hh = oracle.rms_norm(x.to_numpy(), 1e-6)
    from conftest import assert_close

    for (raw, _), g in zip(ws, got):
        assert_close(g, oracle.mul_mat_q4_0(raw, hh))
