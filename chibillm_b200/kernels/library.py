"""Loads the compiled CUDA libraries and declares their C entry points."""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Sequence

from ..csrc import build

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}

P, I, L, F = c_void_p, c_int, c_longlong, c_float

# entry point -> argument types (all return int: 0 ok, >0 a CUDA error, <0 ours)
_SIGNATURES = {
    "chibi_kernels": {
        "chibi_embed": [P, P, I, P, I, L, I, I, P, P],
        "chibi_rmsnorm": [P, I, P, I, P, I, L, I, L, L, F, F, P],
        "chibi_qk_norm_rope_append": [P, I, L, P, P, P, I, P, P, I, P, P, P, P, P, I, L, I, I, I, I, I,
                                      I, F, F, I, P, P],
        "chibi_apply_table_updates": [P, I, I, P, I, P, P],
        "chibi_swiglu": [P, I, P, I, L, I, P],
        "chibi_gather_rows": [P, I, P, P, I, L, I, L, P],
        "chibi_cast": [P, I, P, I, L, P],
        "chibi_add_into": [P, P, I, L, P],
        "chibi_gemm_simt": [P, I, P, I, P, I, P, I, I, I, L, L, L, L, P],
        "chibi_gemm_bf16_splits": [I, I, I],
        "chibi_gemm_bf16_splits_capped": [I, I, I, I],
        "chibi_gemm_bf16": [P, P, P, I, P, I, I, I, L, L, L, L, P, L, P, P],
        "chibi_gemm_set_stream_scratch": [P, L],
        "chibi_gemm_set_pair_tiles": [I, I],
        "chibi_gemm_many_rows_plan": [I, I, I],
        "chibi_gemm_reset_stream_counters": [P],
        "chibi_gemm_bf16_norm_parts": [I, I, I],
        "chibi_gemm_few_rows_max": [],
        "chibi_gemm_bf16_rows": [P, P, P, I, P, I, I, I, L, L, L, L, I, P, P, P, P, P],
        "chibi_rope_table": [P, P, L, I, P, P],
        "chibi_cache_slots": [P, P, P, P, I, L, I, I, I, I, P, P, P],
        "chibi_scale_rows": [P, L, I, L, P, I, F, I, P],
        "chibi_gemm_bf16_fused": [P, P, P, I, P, I, I, I, L, L, L, L, I, P, P],
        "chibi_gemm_bf16_partial": [P, P, I, I, I, L, L, P, L, I, P, P],
        "chibi_reduce_residual_rmsnorm": [P, I, I, I, P, L, P, I, P, I, L, F, F, P],
        "chibi_reduce_swiglu": [P, I, I, I, P, I, I, P],
        "chibi_qk_norm_rope_append_partial": [P, I, L, L, P, P, P, P, P, I, P, P, P, P, P, I, I, I, I, I,
                                              I, I, F, F, I, P, P],
        "chibi_attention_generic": [P, I, P, P, I, P, P, I, P, P, P, P, P, L, I, I, I, I, I, F, I, P, P],
        "chibi_sample": [P, L, L, I, P, P, P, P, L, P],
    },
    "chibi_attention_tc": {
        "chibi_attention_tc_head_dim": [],
        "chibi_attention_prefill_tc": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, I, I, I, P, L, L, P, P],
    },
    "chibi_attention_mma": {
        "chibi_attention_mma_head_dim": [],
        "chibi_attention_mma": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, I, I, P, L, P, P],
        "chibi_attention_decode_fused": [P, I, L, L, P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, P, L, P, P, P,
                                         F, F, I, P, P],
    },
}


class RowScale(ctypes.Structure):
    """ChibiRowScale of gemm_tcgen05.cu: the factor of an RMSNorm that x lacks."""
    _fields_ = [("ssq", c_void_p), ("parts", c_int), ("eps", c_float), ("n", c_int)]


class NormOut(ctypes.Structure):
    """ChibiNormOut of gemm_tcgen05.cu: the norm output that a product writes beside the residual."""
    _fields_ = [("w", c_void_p), ("w_type", c_int), ("offset", c_float), ("out", c_void_p),
                ("out_stride", c_longlong), ("ssq", c_void_p), ("ssq_floats", c_longlong)]


class HeadsOut(ctypes.Structure):
    """ChibiHeadsOut of gemm_tcgen05.cu: where the heads of a q | k | v product go."""
    _fields_ = [("cos_sin", c_void_p), ("slots", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p),
                ("v_cache", c_void_p), ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("w_type", c_int),
                ("nq", c_int), ("nkv", c_int), ("page_size", c_int), ("eps", c_float), ("offset", c_float)]


class KernelLibraryError(RuntimeError):
    pass


def load(name: str, defines: Sequence[str] = ()) -> ctypes.CDLL:
    """Return the library, compiling it first if its current version is absent."""
    key = name + "".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is not None:
            return lib
        try:
            path = build.ensure_library(name, defines)
        except build.BuildError as e:
            raise KernelLibraryError(
                f"the CUDA library '{name}' of chibillm_b200 could not be built; there is no other "
                f"path to run the model on.\n{e}") from None
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelLibraryError(f"cannot load {path}: {e}") from None
        for fn, argtypes in _SIGNATURES.get(name, {}).items():
            f = getattr(lib, fn)
            f.argtypes = argtypes
            f.restype = c_int
        _loaded[key] = lib
        return lib
