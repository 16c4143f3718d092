"""Loads libmmh3_attn_b200.so and declares its C ABI (include/mmh3_attention.h) for ctypes.

There is no fallback: if the library has not been built, importing the bindings raises.
"""

from __future__ import annotations

import ctypes
import pathlib

ROOT = pathlib.Path(__file__).resolve().parent
LIBRARY = ROOT / "lib" / "libmmh3_attn_b200.so"
SELFTEST_LIBRARY = ROOT / "lib" / "libmmh3_b200_selftest.so"

c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p

CUDA_ERROR_INVALID_VALUE = 1
CUDA_ERROR_NOT_SUPPORTED = 801


class AttentionLayout(ctypes.Structure):
    """Mmh3AttentionLayout: strides in elements of query, key, value and output."""

    _fields_ = [
        ("token_stride", c_int64 * 4),
        ("head_stride", c_int64 * 4),
        ("batch_stride", c_int64 * 4),
        ("heads_per_key_value", ctypes.c_int32),
        ("causal", ctypes.c_int32),
    ]


class SparseWorkspace(ctypes.Structure):
    _fields_ = [
        (name, c_void_p)
        for name in (
            "centroids",
            "block_keys",
            "value_sums",
            "key_mean",
            "key_variance",
            "row_offsets",
            "routes",
            "route_counts",
            "tail_max",
            "tail_sum",
            "tail_values",
        )
    ]


class QuantizedWorkspaceStruct(ctypes.Structure):
    _fields_ = [
        (name, c_void_p)
        for name in (
            "query",
            "key",
            "value",
            "query_scales",
            "key_scales",
            "value_scales",
            "value_maxima",
        )
    ]


class VsaWorkspaceStruct(ctypes.Structure):
    _fields_ = [
        (name, c_void_p)
        for name in (
            "tile_starts",
            "tile_lengths",
            "pooled_query",
            "pooled_key",
            "pooled_value",
            "routes",
            "route_counts",
            "coarse",
        )
    ]


P = ctypes.POINTER

# name -> argument types, in the order of include/mmh3_attention.h and
# include/mmh3_int8_gemm.h. Every function returns int.
SIGNATURES = {
    "mmh3_attention": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                       P(AttentionLayout), c_float, c_void_p],
    "mmh3_attention_roped": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, P(AttentionLayout), c_float, c_void_p, c_int, c_float,
                             c_void_p],
    "mmh3_attention_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                            c_int64, c_int64, c_int64, c_float, c_void_p],
    "mmh3_qk_norm_rope": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_float, c_void_p],
    "mmh3_attention_inputs": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_float, P(SparseWorkspace), P(QuantizedWorkspaceStruct), c_void_p,
                              c_void_p, c_int, c_void_p, c_void_p],
    "mmh3_attention_quantized": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 P(AttentionLayout), c_float, P(SparseWorkspace),
                                 P(QuantizedWorkspaceStruct), c_int, c_void_p],
    "mmh3_vsa_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int,
                           c_int, P(AttentionLayout), c_float, c_int, c_int, c_int,
                           P(VsaWorkspaceStruct), P(QuantizedWorkspaceStruct), c_int, c_void_p],
    "mmh3_vsa_attention_quantized": [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int,
                                     P(AttentionLayout), c_float, c_int, P(VsaWorkspaceStruct),
                                     P(QuantizedWorkspaceStruct), c_int, c_void_p],
    "mmh3_sparse_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                              P(AttentionLayout), c_float, c_float, c_int, c_int, c_int, c_int,
                              P(SparseWorkspace), P(QuantizedWorkspaceStruct), c_int, c_void_p],
    "mmh3_dit_shard_pack": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p],
    "mmh3_dit_shard_unpack": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    # include/mmh3_int8_gemm.h
    "mmh3_int8_gemm_config_count": [],
    "mmh3_int8_gemm_group_heights": [c_void_p, c_int],
    "mmh3_int8_gemm_bf16": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_void_p],
    "mmh3_int8_gemm": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                       c_float, c_void_p, c_int, c_void_p],
    "mmh3_interleave_swiglu_rows": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "mmh3_int8_gemm_tilings": [c_void_p, c_int],
    "mmh3_int8_gemm_tiling_key": [ctypes.c_char_p, c_int],
    "mmh3_b200_attention_quantized_static": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             P(AttentionLayout), c_float, c_void_p],
    "mmh3_b200_take_status": [],
}


def declare(library: ctypes.CDLL) -> ctypes.CDLL:
    for name, arguments in SIGNATURES.items():
        function = getattr(library, name)
        function.argtypes = arguments
        function.restype = c_int
    return library


_library: ctypes.CDLL | None = None


def library() -> ctypes.CDLL:
    """The loaded library. Raises when it has not been built (python -m mmh3_b200.build)."""
    global _library
    if _library is None:
        if not LIBRARY.exists():
            raise RuntimeError(
                f"{LIBRARY} is missing: build it with `python -m mmh3_b200.build`; "
                "there is no fallback path"
            )
        _library = declare(ctypes.CDLL(str(LIBRARY)))
    return _library
