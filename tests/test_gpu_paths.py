"""Checks that go through a particular kernel path of the C ABI rather than through an op:
the per-block integer sums of EVERY Q4_0 mat-mul kernel (dp4a on whole words, dp4a with the high
nibbles in place, mma.sync, tcgen05) bit for bit against the oracle's restatement of
BlockQ4_0::vec_dot_q8_0 / vec_dot_unopt (src/ggml_quants.rs:156-191), and a few status paths."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gb():
    import galois_b200

    return galois_b200


def _isums_ex(gb, dev, w_bytes, xq_bytes, nb, variant):
    import torch

    wd = torch.from_numpy(np.ascontiguousarray(w_bytes).copy()).to(dev.torch_device)
    xd = torch.from_numpy(np.ascontiguousarray(xq_bytes).copy()).to(dev.torch_device)
    out = torch.full((nb,), -123456, dtype=torch.int32, device=dev.torch_device)
    rc = gb.lib.galois_b200_block_isums_q4_0_q8_0_ex(dev.ctx, C.c_void_p(wd.data_ptr()), C.c_void_p(xd.data_ptr()), nb, variant,
                                                     C.c_void_p(out.data_ptr()))
    assert rc == 0, gb.lib.galois_b200_last_error(dev.ctx)
    dev.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("variant", [1, 2, 4])
@pytest.mark.parametrize("k", [64, 4096, 11008])
def test_block_isums_of_each_kernel_path(gb, dev, oracle, variant, k):
    w = oracle.quantize_q4_0(oracle.fill_normal(k, 150 + k, 0, 0.02)[None])[0]
    xq = oracle.quantize_q8_0(oracle.fill_normal(k, 160 + k)[None])[0]
    assert np.array_equal(_isums_ex(gb, dev, w, xq, k // 32, variant), oracle.block_isums(w, xq))


@pytest.mark.parametrize("variant", [1, 2, 4])
def test_block_isums_extremes_of_each_kernel_path(gb, dev, oracle, golden, variant):
    # golden rows: all-0 / all-15 nibbles against +-127 quants (|sum| up to 32512) and mixed blocks
    for xi, xr in enumerate((0, 2)):
        xq = golden["q8_bytes"][xr][: 2 * 34]
        for r in range(5):
            w = golden["dot_w"][r][: 2 * 18]
            assert np.array_equal(_isums_ex(gb, dev, w, xq, 2, variant), golden["dot_isums"][xi, r][:2])
    # hand-made: every nibble 0 (value -8) against every quant -127, and every nibble 15 against +127
    for nib, q8, want in ((0x00, -127, 32 * 8 * 127), (0xFF, 127, 32 * 7 * 127), (0xFF, -127, -32 * 7 * 127)):
        w = np.zeros(2 * 18, np.uint8)
        w[2:18] = nib
        w[20:36] = nib
        xq = np.zeros(2 * 34, np.uint8)
        xq[2:34] = np.uint8(q8 & 0xFF)
        xq[36:68] = np.uint8(q8 & 0xFF)
        assert list(_isums_ex(gb, dev, w, xq, 2, variant)) == [want, want]


def _numpy_isums(w_rows: np.ndarray, xq_rows: np.ndarray) -> np.ndarray:
    """[n][nb*18] Q4_0 bytes x [b][nb*34] Q8_0 bytes -> [nb][n][b] exact integer block sums."""
    n, b = w_rows.shape[0], xq_rows.shape[0]
    wq = w_rows.reshape(n, -1, 18)[:, :, 2:]
    q4 = np.concatenate([wq & 0x0F, wq >> 4], axis=-1).astype(np.int32) - 8          # element j low nibble, j + 16 high
    q8 = xq_rows.reshape(b, -1, 34)[:, :, 2:].view(np.int8).astype(np.int32)
    return np.einsum("nkj,bkj->knb", q4, q8)


@pytest.mark.parametrize("n,k,b", [(128, 512, 64), (100, 256, 33), (128, 4096, 64)])
def test_block_isums_of_the_tcgen05_path(gb, dev, oracle, n, k, b):
    import torch

    G = gb.Device.Gpu(dev)
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 170 + n, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 171 + b).reshape(b, k)
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q4_0, G)
    xt = gb.Tensor.from_numpy(x, gb.GGmlType.F32, G)
    dst = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    nb = k // 32
    out = torch.full((nb * 128 * 64,), -123456, dtype=torch.int32, device=dev.torch_device)
    rc = gb.lib.galois_b200_mul_mat_q4_0_tc_block_isums(dev.ctx, C.c_void_p(wt.data_ptr()), C.byref(wt.dim().c_struct()),
                                                        C.c_void_p(xt.data_ptr()), C.byref(xt.dim().c_struct()),
                                                        C.c_void_p(dst.data_ptr()), C.byref(dst.dim().c_struct()), C.c_void_p(out.data_ptr()))
    assert rc == 0, gb.lib.galois_b200_last_error(dev.ctx)
    dev.synchronize()
    got = out.cpu().numpy().reshape(nb, 128, 64)[:, :n, :b]
    xq = oracle.quantize_q8_0(x)
    assert np.array_equal(got, _numpy_isums(w.reshape(n, -1), xq.reshape(b, -1)))
    # a few (row, activation) pairs against the oracle's own block sums
    for r, c in ((0, 0), (n - 1, b - 1), (n // 2, b // 3)):
        assert np.array_equal(got[:, r, c], oracle.block_isums(w.reshape(n, -1)[r], xq.reshape(b, -1)[c]))
    from conftest import assert_close

    assert_close(dst.to_numpy(), oracle.mul_mat_q4_0(w, x))


def test_soft_max_fully_masked_row_reports_badarg(gb, dev, oracle):
    """The reference asserts sum > 0.0 (src/lib.rs:586); here the row is zeroed and a status is raised."""
    G = gb.Device.Gpu(dev)
    x = oracle.fill_normal(3 * 64, 180).reshape(3, 1, 64)
    x[1] = -np.inf
    y = gb.Tensor.from_numpy(np.full((3, 1, 64), 5.0, np.float32), gb.GGmlType.F32, G)
    gb.galois_soft_max(gb.Tensor.from_numpy(x, gb.GGmlType.F32, G), y)
    with pytest.raises(gb.GError) as e:
        dev.synchronize()
    assert e.value.code == -1
    dev.synchronize()  # reported once
    got = y.to_numpy()
    assert np.array_equal(got[1], np.zeros((1, 64), np.float32))
    want = oracle.soft_max(x[[0, 2]])
    assert np.allclose(got[[0, 2]], want, rtol=0, atol=1e-5)
    # causal mask with a negative position masks every column
    pos = gb.Tensor.from_numpy(np.array([-1, 5, 63], np.int32), gb.GGmlType.I32, G)
    xe = oracle.fill_normal(3 * 64, 181).reshape(3, 1, 64)
    gb.galois_soft_max_ext(gb.Tensor.from_numpy(xe, gb.GGmlType.F32, G), y, 0.5, pos)
    with pytest.raises(gb.GError):
        dev.synchronize()
    assert not y.to_numpy()[0].any()


def test_dtoh_reports_a_wait_that_ran_out(gb, dev):
    """A sharded call whose inbox nothing fills: the read-back of its result returns the time-out."""
    import sys, os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_gpu_peer_gather import _call, _setup

    w_band, x, ref, full, inboxes, peers, dd, r0, nr, slots = _setup(dev, 256, 256, 1, 2, 0, 778)
    assert _call(dev, w_band, x, full, dd, r0, peers, 1) == 0
    host = np.zeros(256, np.float32)
    rc = gb.lib.galois_b200_dtoh(dev.ctx, host.ctypes.data_as(C.c_void_p), C.c_void_p(full.data_ptr()), host.nbytes)
    assert rc == -9
    dev.synchronize()  # cleared; the context works on


def test_reserve_scratch_keeps_later_calls_allocation_free(gb, dev, oracle):
    import torch

    G = gb.Device.Gpu(dev)
    n, k, b = 512, 4096, 4000  # far beyond the 16 MiB the context starts with
    wt = gb.Tensor.zeros((k, n), gb.GGmlType.Q4_0, G)
    xt = gb.Tensor.zeros((k, b), gb.GGmlType.F32, G)
    dst = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    need = C.c_size_t()
    assert gb.lib.galois_b200_mul_mat_q4_0_scratch_bytes(dev.ctx, C.byref(wt.dim().c_struct()), C.byref(xt.dim().c_struct()), C.byref(need)) == 0
    assert need.value > b * k
    assert gb.lib.galois_b200_reserve_scratch(dev.ctx, need.value) == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for variant in (0, 1, 3):
        dev.set_mul_mat_variant(variant)
        try:
            gb.galois_matmul(wt, xt, dst)
        finally:
            dev.set_mul_mat_variant(0)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


@pytest.mark.parametrize("n,k,b", [(128, 256, 64), (200, 768, 33), (77, 256, 130), (4096, 4096, 512), (300, 1024, 200), (11008, 4096, 256)])
def test_prepared_weight_gives_the_bits_of_the_unprepared_path(gb, dev, oracle, n, k, b):
    """galois_b200_prepare_weight_q4_0 (the one-time repack at upload) changes where the tensor-core kernel
    takes its operands from, not a single result bit; and the op API is unchanged."""
    G = gb.Device.Gpu(dev)
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 190 + n, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 191 + b).reshape(b, k)
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q4_0, G)
    xt = gb.Tensor.from_numpy(x, gb.GGmlType.F32, G)
    plain, prepared = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G), gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
    dev.set_mul_mat_variant(3)
    try:
        l0 = dev.launch_count()
        gb.galois_matmul(wt, xt, plain)
        dev.prepare_weight(wt)
        dev.prepare_weight(wt)  # refreshing an existing copy is allowed
        l1 = dev.launch_count()
        gb.galois_matmul(wt, xt, prepared)
        a, p = plain.to_numpy(), prepared.to_numpy()
        dev.release_weight(wt)
        gb.galois_matmul(wt, xt, prepared)  # back on the unprepared kernel
        assert np.array_equal(prepared.to_numpy(), a)
    finally:
        dev.set_mul_mat_variant(0)
    assert l1 - l0 == 4  # quantiser + GEMM, two repacks
    assert np.array_equal(a.view(np.uint32), p.view(np.uint32))
    from conftest import assert_close

    assert_close(p, oracle.mul_mat_q4_0(w, x))
    with pytest.raises(gb.GError):
        dev.release_weight(wt)  # not prepared any more


def test_pipelined_host_copies_give_the_results_of_the_synchronous_ones(gb, dev, oracle):
    """galois_b200_htod_async / dtoh_async / dtoh_wait: two buffer sets in turn, the host waits for step i - 1 after
    enqueuing step i; every step's read-back equals the synchronous call's."""
    import torch

    n, k = 1024, 4096
    w = oracle.quantize_q4_0(oracle.fill_normal(n * k, 210, 0, 0.02).reshape(n, k))
    G = gb.Device.Gpu(dev)
    wt = gb.Tensor.from_raw(w, (k, n), gb.GGmlType.Q4_0, G)
    wd = wt.dim().c_struct()
    xdim = gb.Dim.ggml((k, 1), gb.GGmlType.F32).c_struct()
    ydim = gb.Dim.ggml((n, 1), gb.GGmlType.F32).c_struct()
    steps = 6
    xs = [torch.from_numpy(oracle.fill_normal(k, 220 + i)).pin_memory() for i in range(steps)]
    xd = [torch.zeros(k, device=dev.torch_device) for _ in range(2)]
    yd = [torch.zeros(n, device=dev.torch_device) for _ in range(2)]
    yh = [torch.zeros(n).pin_memory() for _ in range(steps)]
    vp = lambda t: C.c_void_p(t.data_ptr())
    tickets, ticket = [None, None], C.c_int(-1)
    for i in range(steps):
        p = i & 1
        assert gb.lib.galois_b200_htod_async(dev.ctx, vp(xd[p]), vp(xs[i]), k * 4) == 0
        assert gb.lib.galois_b200_mul_mat_q4_0_f32(dev.ctx, C.c_void_p(wt.data_ptr()), C.byref(wd), vp(xd[p]), C.byref(xdim), vp(yd[p]), C.byref(ydim)) == 0
        assert gb.lib.galois_b200_dtoh_async(dev.ctx, vp(yh[i]), vp(yd[p]), n * 4, C.byref(ticket)) == 0
        tickets[p] = ticket.value
        if tickets[1 - p] is not None:
            assert gb.lib.galois_b200_dtoh_wait(dev.ctx, tickets[1 - p]) == 0
            tickets[1 - p] = None
    for t in tickets:
        if t is not None:
            assert gb.lib.galois_b200_dtoh_wait(dev.ctx, t) == 0
    assert gb.lib.galois_b200_dtoh_wait(dev.ctx, 99) == -1
    dev.synchronize()
    from conftest import assert_close

    for i in range(steps):
        xt = gb.Tensor.from_numpy(xs[i].numpy().reshape(1, k), gb.GGmlType.F32, G)
        yt = gb.Tensor.zeros((n, 1), gb.GGmlType.F32, G)
        gb.galois_matmul(wt, xt, yt)
        want = yt.to_numpy().reshape(-1)
        assert np.array_equal(yh[i].numpy().view(np.uint32), want.view(np.uint32)), i
        if i == 0:
            assert_close(want.reshape(1, n), oracle.mul_mat_q4_0(w, xs[i].numpy().reshape(1, k)))


def test_auto_prepare_follows_alloc_upload_and_free(gb, dev, oracle):
    """galois_b200_set_auto_prepare: a weight in memory from galois_b200_alloc is repacked by its first large-batch
    mat-mul, re-uploading it drops the copy (the next call repacks the new contents), freeing the block releases
    it; a weight in memory the context did not allocate is left alone.  Results equal the unprepared kernel's bits."""
    import torch

    n, k, b = 256, 512, 96
    G = gb.Device.Gpu(dev)
    wa = oracle.quantize_q4_0(oracle.fill_normal(n * k, 230, 0, 0.02).reshape(n, k))
    wb = oracle.quantize_q4_0(oracle.fill_normal(n * k, 231, 0, 0.02).reshape(n, k))
    x = oracle.fill_normal(b * k, 232).reshape(b, k)
    xt = gb.Tensor.from_numpy(x, gb.GGmlType.F32, G)
    wd = gb.Dim.ggml((k, n), gb.GGmlType.Q4_0).c_struct()
    nbytes = wa.size

    def reference(wraw):  # the unprepared tensor-core kernel on an ordinary tensor
        out = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
        gb.galois_matmul(gb.Tensor.from_raw(wraw, (k, n), gb.GGmlType.Q4_0, G), xt, out)
        return out.to_numpy()

    def run(ptr):
        out = gb.Tensor.zeros((n, b), gb.GGmlType.F32, G)
        rc = gb.lib.galois_b200_mul_mat_q4_0_f32(dev.ctx, ptr, C.byref(wd), C.c_void_p(xt.data_ptr()), C.byref(xt.dim().c_struct()),
                                                 C.c_void_p(out.data_ptr()), C.byref(out.dim().c_struct()))
        assert rc == 0, gb.lib.galois_b200_last_error(dev.ctx)
        return out.to_numpy()

    dev.set_mul_mat_variant(3)
    assert gb.lib.galois_b200_set_auto_prepare(dev.ctx, 1) == 0
    ptr = C.c_void_p()
    assert gb.lib.galois_b200_alloc(dev.ctx, nbytes, C.byref(ptr)) == 0
    try:
        want_a, want_b = reference(wa), reference(wb)   # ordinary tensors: never prepared
        l0 = dev.launch_count()
        reference(wa)
        assert dev.launch_count() - l0 == 2              # quantiser + unprepared GEMM, no repack
        host = np.ascontiguousarray(wa).view(np.uint8).reshape(-1)
        assert gb.lib.galois_b200_htod(dev.ctx, ptr, host.ctypes.data_as(C.c_void_p), nbytes) == 0
        l0 = dev.launch_count()
        got = run(ptr)
        assert dev.launch_count() - l0 == 3              # repack + quantiser + GEMM
        assert np.array_equal(got.view(np.uint32), want_a.view(np.uint32))
        l0 = dev.launch_count()
        run(ptr)
        assert dev.launch_count() - l0 == 2              # the copy is reused
        host_b = np.ascontiguousarray(wb).view(np.uint8).reshape(-1)
        assert gb.lib.galois_b200_htod(dev.ctx, ptr, host_b.ctypes.data_as(C.c_void_p), nbytes) == 0
        l0 = dev.launch_count()
        got = run(ptr)
        assert dev.launch_count() - l0 == 3              # new contents: repacked again
        assert np.array_equal(got.view(np.uint32), want_b.view(np.uint32))
        assert gb.lib.galois_b200_free(dev.ctx, ptr) == 0
        ptr = C.c_void_p()
        assert gb.lib.galois_b200_release_weight(dev.ctx, C.c_void_p(0x1000)) != 0  # nothing prepared is left behind
    finally:
        gb.lib.galois_b200_set_auto_prepare(dev.ctx, 0)
        dev.set_mul_mat_variant(0)
        if ptr.value:
            gb.lib.galois_b200_free(dev.ctx, ptr)


@pytest.mark.parametrize("n2,k,b", [(2 * 11008, 4096, 1), (2 * 300, 256, 1), (2 * 64, 1024, 1), (2 * 100, 11008, 1), (2 * 96, 512, 3)])
@pytest.mark.parametrize("with_norm", [False, True])
def test_swiglu_mat_vec_equals_the_separate_ops(gb, dev, oracle, n2, k, b, with_norm):
    """galois_matmul_swiglu on a weight with gate / up rows interleaved = two mat-muls, Silu and Mul of the reference
    API, bit for bit: in one launch where a warp holds both rows of a pair, otherwise through the pairing kernel."""
    G = gb.Device.Gpu(dev)
    f = n2 // 2
    wg = oracle.quantize_q4_0(oracle.fill_normal(f * k, 240 + k, 0, 0.02).reshape(f, k))
    wu = oracle.quantize_q4_0(oracle.fill_normal(f * k, 241 + k, 0, 0.02).reshape(f, k))
    rb = k // 32 * 18
    inter = np.stack([wg.reshape(f, rb), wu.reshape(f, rb)], axis=1).reshape(n2, rb)
    x = oracle.fill_normal(b * k, 242).reshape(b, k)
    gain = (1.0 + 0.1 * oracle.fill_normal(k, 243)).reshape(1, k)
    xt = gb.Tensor.from_numpy(x, gb.GGmlType.F32, G)
    gt = gb.Tensor.from_numpy(gain, gb.GGmlType.F32, G)
    # the separate ops
    h = gb.Tensor.zeros((k, b), gb.GGmlType.F32, G)
    if with_norm:
        gb.galois_rms_norm(xt, h, 1e-6)
        gb.galois_mul(h, gt, h)
    else:
        h = xt
    g_out, u_out = gb.Tensor.zeros((f, b), gb.GGmlType.F32, G), gb.Tensor.zeros((f, b), gb.GGmlType.F32, G)
    gb.galois_matmul(gb.Tensor.from_raw(wg, (k, f), gb.GGmlType.Q4_0, G), h, g_out)
    gb.galois_matmul(gb.Tensor.from_raw(wu, (k, f), gb.GGmlType.Q4_0, G), h, u_out)
    a = gb.Tensor.zeros((f, b), gb.GGmlType.F32, G)
    gb.galois_unary(g_out, a, gb.UnaryOp.Silu)
    gb.galois_mul(a, u_out, a)
    want = a.to_numpy()
    got = gb.Tensor.zeros((f, b), gb.GGmlType.F32, G)
    l0 = dev.launch_count()
    gb.galois_matmul_swiglu(gb.Tensor.from_raw(inter, (k, n2), gb.GGmlType.Q4_0, G), xt, got, rms_gain=gt if with_norm else None, eps=1e-6)
    launches = dev.launch_count() - l0
    if b == 1 and k in (256, 512, 1024, 4096):
        assert launches == 1
    assert np.array_equal(got.to_numpy().view(np.uint32), want.view(np.uint32))
