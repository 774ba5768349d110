"""CPU tests of the C-ABI boundary: the library loads, exports every function the
header declares, and the host-only entry points behave (no GPU compute here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "galois_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(galois_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import galois_b200
    from galois_b200._lib import SIGNATURES

    names = _declared()
    assert len(names) >= 25
    raw = C.CDLL(galois_b200.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/galois_b200.h but not exported"
        assert n in SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(SIGNATURES) == names


def test_init_without_gpu_fails_cleanly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is visible")
    import galois_b200 as gb

    h = C.c_void_p()
    rc = gb.lib.galois_b200_init(0, None, C.byref(h))
    assert rc != 0 and not h.value
    assert b"init" in gb.lib.galois_b200_last_error(None)
    with pytest.raises(gb.GError):
        gb.CudaDevice(0)
    # a null context is an error code, never a crash
    assert gb.lib.galois_b200_synchronize(None) < 0
    assert gb.lib.galois_b200_destroy(None) == 0


def test_shard_rows_partition():
    from galois_b200.shard import shard_rows

    for n in (0, 1, 31, 32, 100, 4096, 11008, 32000, 28672):
        for world in (1, 2, 3, 4, 8):
            bands = [shard_rows(n, world, r) for r in range(world)]
            at = 0
            for r0, nr in bands:
                assert r0 == at and nr >= 0
                assert r0 % 32 == 0 or r0 == n
                at += nr
            assert at == n
    assert [nr for _, nr in [shard_rows(11008, 8, r) for r in range(8)]] == [1376] * 8
    from galois_b200 import GError

    with pytest.raises(GError):
        shard_rows(10, 2, 2)


def test_cpu_tensors_are_rejected():
    import numpy as np

    import galois_b200 as gb

    a = gb.Tensor.from_numpy(np.zeros((2, 32), np.float32), gb.GGmlType.F32, gb.Device.Cpu())
    with pytest.raises(gb.GError):
        gb.galois_rms_norm(a, a, 1e-6)


def test_dim_mirror():
    import galois_b200 as gb

    d = gb.Dim.ggml((4096, 11008), gb.GGmlType.Q4_0)
    assert d.stride == (1, 128, 128 * 11008, 128 * 11008) and d.shape == (4096, 11008, 1, 1)
    assert d.ggml_is_contiguous(32) and not d.ggml_is_contiguous()
    d = gb.Dim.ggml((128, 32, 1), gb.GGmlType.F32)
    assert d.stride == (1, 128, 4096, 4096) and d.n_dims == 3 and d.ggml_is_contiguous()


def test_to_numpy_rejects_row_padded_view():
    """A window whose rows are further apart than their length (the band of a sharded result) is not
    contiguous (src/shape.rs:254-259): to_numpy must refuse it instead of returning the wrong elements."""
    import numpy as np

    import galois_b200 as gb

    t = gb.Tensor.from_numpy(np.arange(4 * 16, dtype=np.float32).reshape(4, 16), gb.GGmlType.F32, gb.Device.Cpu())
    band = t.view((8, 4), (1, 16, 64, 64))
    assert not band.dim().ggml_is_contiguous()
    with pytest.raises(gb.GError):
        band.to_numpy()
    assert np.array_equal(t.view((16, 2), (1, 16, 32, 32), offset=16).to_numpy(), np.arange(16, 48, dtype=np.float32).reshape(2, 16))
