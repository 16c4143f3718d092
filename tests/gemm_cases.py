"""Seeded operands of the scaled INT8 GEMM, with the value ranges of the reference's own tests
(crates/mmh3-cuda/tests/int8_gemm.rs:87-112, 276-281), and its definition in float64."""

from __future__ import annotations

import numpy as np


def operands(m: int, n: int, k: int, seed: int, bias: bool = False, swiglu: bool = False):
    random = np.random.RandomState(seed)
    activations = random.randint(-127, 128, size=(m, k)).astype(np.int8)
    weights = random.randint(-127, 128, size=(n, k)).astype(np.int8)
    activation_scales = random.uniform(0.5, 1.5, size=m).astype(np.float32)
    low, high = (0.00002, 0.0001) if swiglu else (0.0001, 0.001)
    weight_scales = random.uniform(low, high, size=n).astype(np.float32)
    bias_values = None
    if bias:
        span = 2.0 if swiglu else 20.0
        bias_values = random.uniform(-span, span, size=n).astype(np.float32)
    return activations, weights, activation_scales, weight_scales, bias_values


def definition(activations, weights, activation_scales, weight_scales, bias=None,
               adapter=None) -> np.ndarray:
    """sum_k a[m, k] w[n, k] * scale[m] * scale[n] + adapter_scale * down . up^T + bias[n] in
    float64, [m, n]. `adapter` is (down BF16 bits [m, stride], up BF16 bits [n, rank], rank,
    scale)."""
    # float64 holds these integer sums exactly.
    sums = activations.astype(np.float64) @ weights.astype(np.float64).T
    result = sums * activation_scales.astype(np.float64)[:, None] * \
        weight_scales.astype(np.float64)[None, :]
    if adapter is not None:
        down, up, rank, scale = adapter
        result = result + scale * (widen(down[:, :rank], False) @ widen(up, False).T)
    if bias is not None:
        result = result + bias.astype(np.float64)[None, :]
    return result


def adapter_operands(m: int, n: int, rank: int, stride: int, seed: int, span: float = 2.0):
    """BF16 down [m, stride] (columns past the rank hold 1000, which must not be read) and up
    [n, rank], as crates/mmh3-cuda/tests/int8_gemm.rs:93-103 draws them."""
    random = np.random.RandomState(seed)

    def bf16(values):
        bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)

    down = random.uniform(-span, span, size=(m, stride)).astype(np.float32)
    down[:, rank:] = 1000.0
    up = random.uniform(-span, span, size=(n, rank)).astype(np.float32)
    return bf16(down), bf16(up)


def interleave(rows: np.ndarray) -> np.ndarray:
    """Rows in the order mmh3_interleave_swiglu_rows leaves them: groups of eight, the gates of
    four features and then their up projections, from gates in the first half and up projections
    in the second."""
    count = rows.shape[0]
    features = count // 2
    order = np.empty(count, dtype=np.int64)
    for row in range(count):
        group, position = divmod(row, 8)
        order[row] = group * 4 + position if position < 4 else features + group * 4 + position - 4
    return rows[order]


def widen(bits: np.ndarray, f16: bool) -> np.ndarray:
    if f16:
        return bits.view(np.float16).astype(np.float64)
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def column_maxima(bits: np.ndarray, first_column: int) -> np.ndarray:
    """The largest BF16 magnitude of each group of 128 columns from `first_column` on."""
    magnitudes = (((bits & 0x7fff).astype(np.uint32)) << 16).view(np.float32)
    groups = (bits.shape[1] - first_column) // 128
    return magnitudes[:, first_column:].reshape(bits.shape[0], groups, 128).max(axis=(0, 2))
