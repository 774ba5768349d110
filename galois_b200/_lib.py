"""ctypes binding of ``libgalois_b200.so`` (declared in ``include/galois_b200.h``).

There is no fallback of any kind: if the shared library is missing or a symbol
is absent, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgalois_b200.so")


class GaloisDim(C.Structure):
    """``galois_dim``: copy of galois ``Dim`` (src/shape.rs:29-34)."""

    _fields_ = [("n_dims", C.c_int32), ("ne", C.c_int64 * 4), ("nb", C.c_int64 * 4)]


MAX_RANKS = 8
IPC_HANDLE_BYTES = 64


class GaloisPeers(C.Structure):
    """``galois_b200_peers``: every rank's inbox of the fused exchange, as addresses valid on this
    rank's device."""

    _fields_ = [("rank", C.c_int32), ("nranks", C.c_int32), ("slots", C.c_int64), ("inbox", C.c_void_p * MAX_RANKS)]


class GaloisPrologue(C.Structure):
    """``galois_b200_prologue``: an op pair applied to the activations inside the fused mat-mul call."""

    _fields_ = [("kind", C.c_int32), ("aux", C.c_void_p), ("eps", C.c_float)]


class GaloisDecodeLayer(C.Structure):
    """``galois_b200_decode_layer``: device pointers of one decoder layer for the persistent decode kernel."""

    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down", "attn_norm", "ffn_norm", "k_cache", "v_cache")]


class GaloisDecodeShape(C.Structure):
    """``galois_b200_decode_shape``."""

    _fields_ = [("hidden", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("ctx", C.c_int32),
                ("eps", C.c_float), ("rope_freq_base", C.c_float), ("rope_freq_scale", C.c_float)]


_P, _F, _I, _I64, _SZ = C.c_void_p, C.c_float, C.c_int, C.c_int64, C.c_size_t
_DP = C.POINTER(GaloisDim)

# name -> (argtypes, restype); must list every function include/galois_b200.h declares
SIGNATURES = {
    "galois_b200_init": ([_I, _P, C.POINTER(_P)], _I),
    "galois_b200_destroy": ([_P], _I),
    "galois_b200_set_stream": ([_P, _P], _I),
    "galois_b200_last_error": ([_P], C.c_char_p),
    "galois_b200_launch_count": ([_P], _I64),
    "galois_b200_set_mul_mat_variant": ([_P, _I], _I),
    "galois_b200_set_pdl": ([_P, _I], _I),
    "galois_b200_set_overlap": ([_P, _I], _I),
    "galois_b200_overlap_counts": ([_P, C.POINTER(_I64 * 3)], _I),
    "galois_b200_profile_enable": ([_P, _I], _I),
    "galois_b200_profile_read": ([_P, C.POINTER(C.c_double), C.POINTER(_I64)], _I),
    "galois_b200_alloc": ([_P, _SZ, C.POINTER(_P)], _I),
    "galois_b200_free": ([_P, _P], _I),
    "galois_b200_htod": ([_P, _P, _P, _SZ], _I),
    "galois_b200_dtoh": ([_P, _P, _P, _SZ], _I),
    "galois_b200_htod_async": ([_P, _P, _P, _SZ], _I),
    "galois_b200_dtoh_async": ([_P, _P, _P, _SZ, C.POINTER(_I)], _I),
    "galois_b200_dtoh_wait": ([_P, _I], _I),
    "galois_b200_synchronize": ([_P], _I),
    "galois_b200_reserve_scratch": ([_P, _SZ], _I),
    "galois_b200_mul_mat_q4_0_scratch_bytes": ([_P, _DP, _DP, C.POINTER(_SZ)], _I),
    "galois_b200_quantize_q8_0": ([_P, _P, _I64, _P, _I64, _I64], _I),
    "galois_b200_block_isums_q4_0_q8_0": ([_P, _P, _P, _I64, _P], _I),
    "galois_b200_block_isums_q4_0_q8_0_ex": ([_P, _P, _P, _I64, _I, _P], _I),
    "galois_b200_mul_mat_q4_0_tc_block_isums": ([_P, _P, _DP, _P, _DP, _P, _DP, _P], _I),
    "galois_b200_mul_mat_q4_0_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_prepare_weight_q4_0": ([_P, _P, _DP], _I),
    "galois_b200_release_weight": ([_P, _P], _I),
    "galois_b200_set_auto_prepare": ([_P, _I], _I),
    "galois_b200_mul_mat_q4_0_f32_fused": ([_P, _P, _DP, _P, _DP, C.POINTER(GaloisPrologue), _P, _DP, _P, _DP], _I),
    "galois_b200_mul_mat_q4_0_f32_swiglu": ([_P, _P, _DP, _P, _DP, C.POINTER(GaloisPrologue), _P, _DP], _I),
    "galois_b200_mul_mat_q4_0_f32_add": ([_P, _P, _DP, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_mul_mat_q4_0_f32_host": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_mul_mat_q4_0_f32_static": ([_P, _P, _DP, _P, _DP, _P, _DP, C.c_char_p, _SZ], _I),
    "galois_b200_mul_mat_q6k_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_quantize_q8_k": ([_P, _P, _I64, _P, _I64, _I64], _I),
    "galois_b200_block_isums_q6k_q8k": ([_P, _P, _P, _I64, _P], _I),
    "galois_b200_mul_mat_f16_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_rms_norm_f32": ([_P, _P, _DP, _P, _DP, _F], _I),
    "galois_b200_rms_norm_mul_f32": ([_P, _P, _DP, _P, _DP, _P, _DP, _F], _I),
    "galois_b200_silu_mul_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_rope_f32": ([_P, _P, _DP, _P, _DP, _P, _DP, _I, _I, _I, _F, _F, _F, _I], _I),
    "galois_b200_soft_max_f32": ([_P, _P, _DP, _P, _DP], _I),
    "galois_b200_soft_max_ext_f32": ([_P, _P, _DP, _P, _DP, _F, _P], _I),
    "galois_b200_silu_f32": ([_P, _P, _DP, _P, _DP], _I),
    "galois_b200_mul_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_add_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_scale_f32": ([_P, _P, _DP, _F, _P, _DP], _I),
    "galois_b200_cpy_f32_f32": ([_P, _P, _DP, _P, _DP], _I),
    "galois_b200_cpy_f32_f16": ([_P, _P, _DP, _P, _DP], _I),
    "galois_b200_cpy_f32_f16_pair": ([_P, _P, _DP, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_get_rows_q4_0_f32": ([_P, _P, _DP, _P, _DP, _P, _DP], _I),
    "galois_b200_decode_workspace_bytes": ([_P, C.POINTER(GaloisDecodeShape), C.POINTER(_SZ)], _I),
    "galois_b200_decode_layers_f32": ([_P, C.POINTER(GaloisDecodeShape), C.POINTER(GaloisDecodeLayer), _I, _P, _P, _P, _P, _SZ], _I),
    "galois_b200_decode_attention_f32": ([_P, C.POINTER(GaloisDecodeShape), C.POINTER(GaloisDecodeLayer), _P, _P, _P, _P, _SZ], _I),
    "galois_b200_shard_rows": ([_I64, _I, _I, C.POINTER(_I64), C.POINTER(_I64)], _I),
    "galois_b200_ipc_export": ([_P, _P, C.c_char_p], _I),
    "galois_b200_ipc_import": ([_P, C.c_char_p, C.POINTER(_P)], _I),
    "galois_b200_ipc_close": ([_P, _P], _I),
    "galois_b200_mul_mat_q4_0_f32_gather": ([_P, _P, _DP, _P, _DP, _P, _DP, _I64, C.POINTER(GaloisPeers), C.c_uint32], _I),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python galois_b200/build.py` (nvcc, sm_100a). "
            "galois_b200 has no CPU or eager fallback."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (args, res) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = args
        fn.restype = res
    return lib


lib = _load()
