"""ctypes access to the oracles, for tests, the smoke check and the benchmark's CPU baseline only.

`load()` is the CPU restatement (oracle/liboracle.so). `load_reference()` is the reference's own
CUDA kernels compiled from its sources into oracle/_ref/libmmh3_ref.so, which exports the same C
ABI as the product library and therefore takes the same ctypes declarations.
"""

from __future__ import annotations

import ctypes
import pathlib
import subprocess

import numpy as np

REPO = pathlib.Path(__file__).resolve().parent.parent
ORACLE_DIR = REPO / "oracle"
ORACLE = ORACLE_DIR / "liboracle.so"
REFERENCE = ORACLE_DIR / "_ref" / "libmmh3_ref.so"

c_int, c_int64, c_float, c_double = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_double
c_void_p = ctypes.c_void_p


def build() -> None:
    """Builds the CPU oracle and, where the reference checkout is present, oracle/_ref."""
    subprocess.run(["make", "-C", str(ORACLE_DIR), "-j8"], check=True, capture_output=True)


def load() -> ctypes.CDLL:
    source = ORACLE_DIR / "oracle.cpp"
    if not ORACLE.exists() or ORACLE.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "liboracle.so"], check=True,
                       capture_output=True)
    library = ctypes.CDLL(str(ORACLE))
    library.oracle_max_threads.restype = c_int
    library.oracle_f32_to_bf16.argtypes = [c_float]
    library.oracle_f32_to_bf16.restype = ctypes.c_uint16
    library.oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
    library.oracle_bf16_to_f32.restype = c_float
    library.oracle_f32_to_e4m3.argtypes = [c_float]
    library.oracle_f32_to_e4m3.restype = ctypes.c_uint8
    library.oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
    library.oracle_e4m3_to_f32.restype = c_float
    library.oracle_lcg_uniform.argtypes = [ctypes.c_uint64, c_float, c_float, c_void_p, c_int64]
    library.oracle_lcg_uniform.restype = ctypes.c_uint64
    library.oracle_attention_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                             c_int, c_int, c_double, c_int]
    library.oracle_attention_f32.restype = None
    library.oracle_attention_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                              c_void_p, c_void_p, c_int, c_double, c_int64,
                                              c_int64, c_int, c_int, c_int]
    library.oracle_attention_bf16.restype = None
    library.oracle_quantize_rows.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p,
                                             c_void_p, c_int, c_void_p, c_void_p]
    library.oracle_quantize_rows.restype = None
    library.oracle_quantize_value.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int,
                                              c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p]
    library.oracle_quantize_value.restype = None
    library.oracle_quantized_attention.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float,
        c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
        c_int64, c_int64]
    library.oracle_quantized_attention.restype = None
    library.oracle_vsa_plan.argtypes = [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p]
    library.oracle_vsa_plan.restype = c_int
    library.oracle_vsa_kept.argtypes = [c_int, c_double]
    library.oracle_vsa_kept.restype = c_int
    library.oracle_select_tiles.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    library.oracle_select_tiles.restype = c_int
    library.oracle_vsa_pool.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
    library.oracle_vsa_pool.restype = None
    library.oracle_vsa_score.argtypes = [c_void_p, c_void_p, c_float]
    library.oracle_vsa_score.restype = c_float
    library.oracle_vsa_select.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                          c_void_p, c_void_p, c_void_p]
    library.oracle_vsa_select.restype = None
    library.oracle_vsa_reference.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int, c_float, c_int,
                                             c_void_p]
    library.oracle_vsa_reference.restype = None
    library.oracle_shard_even.argtypes = [c_int64, c_int, c_int64, c_void_p]
    library.oracle_shard_even.restype = None
    library.oracle_sol_route.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                         c_int, c_float, c_float, c_void_p] + [c_void_p] * 11
    library.oracle_sol_route.restype = None
    library.oracle_sol_reference.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_float, c_float, c_void_p, c_void_p]
    library.oracle_sol_reference.restype = c_double
    library.oracle_int8_gemm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_int]
    library.oracle_int8_gemm.restype = None
    return library


def load_reference():
    """The reference's CUDA kernels, or None when oracle/_ref has not been built."""
    if not REFERENCE.exists():
        return None
    from mmh3_b200 import _lib

    library = ctypes.CDLL(str(REFERENCE))
    for name, arguments in _lib.SIGNATURES.items():
        if name.startswith("mmh3_b200_"):
            continue
        function = getattr(library, name)
        function.argtypes = arguments
        function.restype = c_int
    return library


def ptr(array: np.ndarray | None) -> c_void_p:
    if array is None:
        return c_void_p(0)
    assert array.flags["C_CONTIGUOUS"]
    return c_void_p(array.ctypes.data)


def lcg(library, state: int, count: int, low: float, high: float):
    values = np.empty(count, dtype=np.float32)
    state = library.oracle_lcg_uniform(state, low, high, ptr(values), count)
    return values, state


def attention_bf16(library, qkv_bits: np.ndarray, tokens: int, heads: int, scale: float,
                   query_begin: int = 0, query_end: int | None = None, head_begin: int = 0,
                   head_end: int | None = None, threads: int = 0) -> np.ndarray:
    """f64 dense attention on BF16 qkv [tokens, 3, heads, 128] (bit patterns); f32 output
    [queries, heads, 128]."""
    inner = heads * 128
    query_end = tokens if query_end is None else query_end
    head_end = heads if head_end is None else head_end
    flat = np.ascontiguousarray(qkv_bits.reshape(-1))
    token_stride = np.array([3 * inner] * 3, dtype=np.int64)
    head_stride = np.array([128] * 3, dtype=np.int64)
    output = np.empty((query_end - query_begin, head_end - head_begin, 128), dtype=np.float32)
    base = flat.ctypes.data
    library.oracle_attention_bf16(
        c_void_p(base), c_void_p(base + 2 * inner), c_void_p(base + 4 * inner), ptr(output),
        tokens, ptr(token_stride), ptr(head_stride), 1, scale, query_begin, query_end, head_begin,
        head_end, threads)
    return output


def sol_route(library, qkv_bits: np.ndarray, tokens: int, heads: int, tau: float, scale: float,
              sinks=(0, 0, 0, 0)) -> dict:
    """Sol-Attn's routing workspace in FP32 kernel order from BF16 qkv [tokens, 3, heads, 128]
    (bit patterns): a dict of the workspace's arrays, shaped."""
    inner = heads * 128
    blocks = -(-tokens // 64)
    flat = np.ascontiguousarray(qkv_bits.reshape(-1))
    token_stride = np.array([3 * inner] * 3, dtype=np.int64)
    head_stride = np.array([128] * 3, dtype=np.int64)
    sink_array = np.array(sinks, dtype=np.int32)
    result = {
        "centroids": np.empty((heads, blocks, 128), dtype=np.float32),
        "block_keys": np.empty((heads, blocks, 128), dtype=np.float32),
        "value_sums": np.empty((heads, blocks, 128), dtype=np.float32),
        "key_mean": np.empty((heads, 128), dtype=np.float32),
        "key_variance": np.empty((heads, 128), dtype=np.float32),
        "row_offsets": np.empty((heads, tokens), dtype=np.float32),
        "routes": np.zeros((heads, blocks, blocks), dtype=np.uint16),
        "route_counts": np.empty((heads, blocks), dtype=np.int32),
        "tail_max": np.empty((heads, blocks), dtype=np.float32),
        "tail_sum": np.empty((heads, blocks), dtype=np.float32),
        "tail_values": np.empty((heads, blocks, 128), dtype=np.float32),
    }
    base = flat.ctypes.data
    library.oracle_sol_route(
        c_void_p(base), c_void_p(base + 2 * inner), c_void_p(base + 4 * inner),
        ptr(token_stride), ptr(head_stride), tokens, heads, tau, scale, ptr(sink_array),
        *(ptr(result[name]) for name in (
            "centroids", "block_keys", "value_sums", "key_mean", "key_variance", "row_offsets",
            "routes", "route_counts", "tail_max", "tail_sum", "tail_values")))
    return result


def sol_reference(library, query: np.ndarray, key: np.ndarray, value: np.ndarray, tau: float,
                  scale: float, sinks=(0, 0, 0, 0)):
    """f64 Sol-Attn on f32 [tokens, heads, dim] operands: (output f32, routed fraction)."""
    tokens, heads, dim = query.shape
    output = np.empty((tokens, heads, dim), dtype=np.float32)
    sink_array = np.array(sinks, dtype=np.int32)
    operands = [np.ascontiguousarray(operand, dtype=np.float32) for operand in (query, key, value)]
    fraction = library.oracle_sol_reference(
        ptr(operands[0]), ptr(operands[1]), ptr(operands[2]), tokens, heads, dim, tau, scale,
        ptr(sink_array), ptr(output))
    return output, fraction


def int8_gemm(library, activations: np.ndarray, weights: np.ndarray, activation_scales: np.ndarray,
              weight_scales: np.ndarray, bias: np.ndarray | None = None, f16: bool = False,
              swiglu: bool = False, maxima_first_column: int | None = None):
    """The scaled INT8 GEMM in the kernels' FP32 order: (output bit patterns [m, n] or [m, n / 2],
    column maxima as FP32 or None)."""
    m, k = activations.shape
    n = weights.shape[0]
    output = np.zeros((m, n // 2 if swiglu else n), dtype=np.uint16)
    maxima = None
    if maxima_first_column is not None:
        maxima = np.zeros(max((n - maxima_first_column) // 128, 1), dtype=np.uint32)
    kept = [np.ascontiguousarray(activations, dtype=np.int8),
            np.ascontiguousarray(weights, dtype=np.int8),
            np.ascontiguousarray(activation_scales, dtype=np.float32),
            np.ascontiguousarray(weight_scales, dtype=np.float32),
            None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)]
    library.oracle_int8_gemm(ptr(kept[0]), ptr(kept[1]), ptr(kept[2]), ptr(kept[3]), ptr(kept[4]),
                             ptr(output), int(f16), int(swiglu), m, n, k, output.shape[1],
                             ptr(maxima), maxima_first_column or 0)
    return output, None if maxima is None else maxima.view(np.float32)
