"""Host-side container types mirroring the slice of galois's ``Tensor`` API the
GPU hot path touches (src/lib.rs:58-2832, src/shape.rs, src/cuda.rs:35-308).

Only what the ops need is here: dtype, ggml-ordered shape/strides, a CPU
storage (numpy) and a GPU storage (a torch CUDA byte buffer: torch is used for
device memory and streams only), upload and read-back.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from ._lib import GaloisDim, lib

MAX_DIM = 4
QK4_0 = 32


class GError(RuntimeError):
    """Mirror of ``GError`` (src/error.rs:14-92); carries the C-ABI status code."""

    def __init__(self, msg: str, code: int = 0):
        super().__init__(msg)
        self.code = code


class GGmlType(enum.IntEnum):
    """The dtypes the hot path uses (subset of src/lib.rs GGmlType)."""

    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q6K = 14
    I32 = 18


# elements per block and bytes per block (GS_BLCK_SIZE / GS_TYPE_SIZE, src/lib.rs:340-375)
BLCK_SIZE = {GGmlType.F32: 1, GGmlType.F16: 1, GGmlType.Q4_0: QK4_0, GGmlType.Q6K: 256, GGmlType.I32: 1}
TYPE_SIZE = {GGmlType.F32: 4, GGmlType.F16: 2, GGmlType.Q4_0: 18, GGmlType.Q6K: 210, GGmlType.I32: 4}
_NP_DTYPE = {GGmlType.F32: np.float32, GGmlType.F16: np.float16, GGmlType.I32: np.int32}


@dataclass
class Dim:
    """``Dim { n_dims, shape, stride }`` (src/shape.rs:29-34): ggml order, strides in
    elements (blocks for quantised types, src/shape.rs:422-430)."""

    n_dims: int
    shape: tuple
    stride: tuple

    @staticmethod
    def ggml(shape, dtype: GGmlType) -> "Dim":
        shape = tuple(int(s) for s in shape)
        n_dims = len(shape)
        ne = shape + (1,) * (MAX_DIM - n_dims)
        nb = [1, ne[0] // BLCK_SIZE[dtype], 0, 0]
        nb[2] = nb[1] * ne[1]
        nb[3] = nb[2] * ne[2]
        return Dim(n_dims, ne, tuple(nb))

    def dim4(self):
        return self.shape

    def stride_4d(self):
        return self.stride

    def elem_count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def nrows(self) -> int:
        return self.shape[1] * self.shape[2] * self.shape[3]

    def ggml_is_contiguous(self, block: int = 1) -> bool:
        """src/shape.rs:254-259; strides are in blocks of `block` elements (32 for Q4_0), so a row
        of shape[0] elements is contiguous with the next one when stride[1] == shape[0] / block."""
        s, n = self.stride, self.shape
        return s[0] == 1 and s[1] == n[0] // block and s[2] == s[1] * n[1] and s[3] == s[2] * n[2]

    def c_struct(self) -> GaloisDim:
        d = GaloisDim()
        d.n_dims = self.n_dims
        for i in range(4):
            d.ne[i] = self.shape[i]
            d.nb[i] = self.stride[i]
        return d


def _check(ctx, rc: int, what: str):
    if rc != 0:
        msg = lib.galois_b200_last_error(ctx)
        raise GError(f"{what}: {msg.decode() if msg else ''} (status {rc})", rc)


class CudaDevice:
    """Mirror of ``CudaDevice::new(ordinal)`` + ``init_cuda_function`` (src/cuda.rs:221-229,
    src/kernels.rs:4-22): owns the ``galois_b200_ctx`` of one GPU."""

    def __init__(self, ordinal: int = 0, stream=None):
        import torch

        if not torch.cuda.is_available():
            raise GError("CudaDevice: no CUDA device is visible; galois_b200 has no CPU path")
        self.ordinal = ordinal
        torch.cuda.set_device(ordinal)
        self.torch_device = torch.device("cuda", ordinal)
        self._stream = stream if stream is not None else torch.cuda.current_stream(self.torch_device)
        handle = C.c_void_p()
        rc = lib.galois_b200_init(ordinal, C.c_void_p(self._stream.cuda_stream), C.byref(handle))
        if rc != 0:
            msg = lib.galois_b200_last_error(None)
            raise GError(f"galois_b200_init: {msg.decode() if msg else ''} (status {rc})", rc)
        self.ctx = handle

    def set_stream(self, stream):
        self._stream = stream
        _check(self.ctx, lib.galois_b200_set_stream(self.ctx, C.c_void_p(stream.cuda_stream)), "set_stream")

    @property
    def stream(self):
        return self._stream

    def set_mul_mat_variant(self, variant: int):
        _check(self.ctx, lib.galois_b200_set_mul_mat_variant(self.ctx, variant), "set_mul_mat_variant")

    def set_overlap(self, on: bool):
        """Overlap of independent one-row mat-muls (galois_b200_set_overlap; default on)."""
        _check(self.ctx, lib.galois_b200_set_overlap(self.ctx, 1 if on else 0), "set_overlap")

    def prepare_weight(self, w: "Tensor"):
        """One-time repack of a Q4_0 weight for the large-batch mat-mul (galois_b200_prepare_weight_q4_0)."""
        _check(self.ctx, lib.galois_b200_prepare_weight_q4_0(self.ctx, C.c_void_p(w.data_ptr()), C.byref(w.dim().c_struct())), "prepare_weight")

    def release_weight(self, w: "Tensor"):
        _check(self.ctx, lib.galois_b200_release_weight(self.ctx, C.c_void_p(w.data_ptr())), "release_weight")

    def overlap_counts(self):
        """(waited at entry, deferred wait, barrier) counts of one-row mat-vec launches so far."""
        out = (C.c_int64 * 3)()
        _check(self.ctx, lib.galois_b200_overlap_counts(self.ctx, C.byref(out)), "overlap_counts")
        return tuple(int(v) for v in out)

    def launch_count(self) -> int:
        return int(lib.galois_b200_launch_count(self.ctx))

    def synchronize(self):
        _check(self.ctx, lib.galois_b200_synchronize(self.ctx), "synchronize")

    def close(self):
        if getattr(self, "ctx", None):
            lib.galois_b200_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Device:
    """``Device::{Cpu, Gpu(CudaDevice)}`` (src/lib.rs)."""

    def __init__(self, gpu: CudaDevice | None = None):
        self.gpu = gpu

    @staticmethod
    def Cpu() -> "Device":
        return Device(None)

    @staticmethod
    def Gpu(dev: CudaDevice) -> "Device":
        return Device(dev)

    @property
    def is_gpu(self) -> bool:
        return self.gpu is not None


class Tensor:
    """A dtype + ``Dim`` + storage.  CPU storage is a flat numpy array (uint8 for
    Q4_0); GPU storage is a flat torch CUDA tensor of the same element type."""

    def __init__(self, dtype: GGmlType, dim: Dim, storage, device: Device, offset: int = 0):
        self.dtype = dtype
        self._dim = dim
        self.storage = storage
        self.device = device
        self.offset = offset  # in elements (blocks for Q4_0) from the start of `storage`

    # ---- constructors ------------------------------------------------
    @staticmethod
    def from_raw(raw: np.ndarray, shape, dtype: GGmlType, device: Device) -> "Tensor":
        """``Tensor::from_raw`` (src/lib.rs:2477-2491): `raw` holds the tensor's bytes
        (Q4_0 blocks enter galois this way)."""
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        dim = Dim.ggml(shape, dtype)
        want = dim.elem_count() // BLCK_SIZE[dtype] * TYPE_SIZE[dtype]
        if raw.size != want:
            raise GError(f"from_raw: {raw.size} bytes for shape {tuple(shape)} {dtype.name}, expected {want}")
        if dtype in (GGmlType.Q4_0, GGmlType.Q6K):
            host = raw.copy()
        else:
            host = raw.view(_NP_DTYPE[dtype]).copy()
        return Tensor._place(dtype, dim, host, device)

    @staticmethod
    def from_numpy(arr: np.ndarray, dtype: GGmlType, device: Device) -> "Tensor":
        """numpy array of shape (n3, n2, n1, n0) (C order) -> tensor with ne = [n0, n1, n2, n3]
        (``Tensor::from_vec``, src/lib.rs:2467-2475)."""
        if dtype in (GGmlType.Q4_0, GGmlType.Q6K):
            raise GError("from_numpy: quantised tensors are built with from_raw")
        host = np.ascontiguousarray(arr, dtype=_NP_DTYPE[dtype])
        dim = Dim.ggml(tuple(host.shape)[::-1], dtype)
        return Tensor._place(dtype, dim, host.reshape(-1).copy(), device)

    @staticmethod
    def zeros(shape, dtype: GGmlType, device: Device) -> "Tensor":
        dim = Dim.ggml(shape, dtype)
        n = dim.elem_count() // BLCK_SIZE[dtype]
        if device.is_gpu:
            import torch

            tdt = {GGmlType.F32: torch.float32, GGmlType.F16: torch.float16, GGmlType.I32: torch.int32}.get(dtype)
            if dtype in (GGmlType.Q4_0, GGmlType.Q6K):
                st = torch.zeros(n * TYPE_SIZE[dtype], dtype=torch.uint8, device=device.gpu.torch_device)
            else:
                st = torch.zeros(n, dtype=tdt, device=device.gpu.torch_device)
            return Tensor(dtype, dim, st, device)
        if dtype in (GGmlType.Q4_0, GGmlType.Q6K):
            return Tensor(dtype, dim, np.zeros(n * TYPE_SIZE[dtype], dtype=np.uint8), device)
        return Tensor(dtype, dim, np.zeros(n, dtype=_NP_DTYPE[dtype]), device)

    @staticmethod
    def _place(dtype, dim, host: np.ndarray, device: Device) -> "Tensor":
        if not device.is_gpu:
            return Tensor(dtype, dim, host, device)
        import torch

        # htod_sync_copy (src/cuda.rs:231-255)
        st = torch.from_numpy(host).to(device.gpu.torch_device)
        return Tensor(dtype, dim, st, device)

    # ---- accessors -----------------------------------------------------
    def dim(self) -> Dim:
        return self._dim

    def shape(self):
        return self._dim.shape[: self._dim.n_dims]

    @property
    def is_gpu(self) -> bool:
        return self.device.is_gpu

    def data_ptr(self) -> int:
        if not self.is_gpu:
            raise GError("data_ptr: CPU tensor")
        return self.storage.data_ptr() + self.offset * TYPE_SIZE[self.dtype]

    def view(self, shape, stride, offset: int = 0) -> "Tensor":
        """A strided window on the same storage (shape/stride in ggml order, stride and
        offset in elements; blocks for Q4_0)."""
        shape = tuple(shape) + (1,) * (4 - len(shape))
        stride = tuple(stride)
        assert len(stride) == 4
        n_dims = max(1, max(i + 1 for i in range(4) if shape[i] != 1 or i == 0))
        return Tensor(self.dtype, Dim(n_dims, shape, stride), self.storage, self.device, self.offset + offset)

    def to_cpu_tensor(self) -> "Tensor":
        """``Tensor::to_cpu_tensor`` (src/lib.rs:2279-2341): dtoh_sync_copy of the whole storage."""
        if not self.is_gpu:
            return self
        self.device.gpu.synchronize()
        host = self.storage.cpu().numpy()
        return Tensor(self.dtype, self._dim, host, Device.Cpu(), self.offset)

    def to_numpy(self) -> np.ndarray:
        """Contiguous tensors only: numpy array of shape (n3, n2, n1, n0) trimmed to n_dims."""
        t = self.to_cpu_tensor()
        if not t._dim.ggml_is_contiguous(BLCK_SIZE[t.dtype]):
            raise GError("to_numpy: tensor is not contiguous")
        n = t._dim.elem_count() // BLCK_SIZE[t.dtype]
        if t.dtype in (GGmlType.Q4_0, GGmlType.Q6K):
            sz = TYPE_SIZE[t.dtype]
            return np.asarray(t.storage)[t.offset * sz : (t.offset + n) * sz].copy()
        flat = np.asarray(t.storage)[t.offset : t.offset + n]
        return flat.reshape(tuple(t._dim.shape[: t._dim.n_dims])[::-1]).copy()
