"""The scaled INT8 GEMM of the DiT's linear layers, through the library's C ABI.

Mirrors the safe wrapper of niw/mmh3's CUDA crate (crates/mmh3-cuda/src/gemm.rs:345-462): the same
names, argument meaning and bounds checks, with `torch` tensors standing where the crate has
`DeviceBuffer`s.
"""

from __future__ import annotations

import ctypes
import dataclasses

import torch

from . import _lib
from .attention import _pointer, _stream, check


@dataclasses.dataclass
class Int8Tiling:
    """A tile shape (0: N in multiples of 128, 1: of 256) and the height of the bands of tiles
    (gemm.rs:296-299). Every tiling gives the same bits, and here the same speed."""

    config: int
    group_m: int


@dataclasses.dataclass
class Adapter:
    """A low-rank adapter scale * down . up^T (gemm.rs:140-156): `down` BF16 [m, rank] with rows
    `down_stride` elements apart, `up` BF16 [n, rank]; the rank a multiple of 64."""

    down: torch.Tensor
    up: torch.Tensor
    rank: int
    down_stride: int
    scale: float


@dataclasses.dataclass
class ColumnMaxima:
    """Zeroed FP32 values that receive the maximum |output| of each 128 columns from
    `first_column`, a multiple of 128, on (gemm.rs:361-364)."""

    values: torch.Tensor
    first_column: int


@dataclasses.dataclass
class Output:
    """Where `int8` writes its result (gemm.rs:351-359): [m, n] in BF16 or FP16 after adding an
    optional f32 bias [n], or silu(gate) * up as [m, n / 2] with `swiglu`."""

    buffer: torch.Tensor
    f16: bool = False
    bias: torch.Tensor | None = None
    swiglu: bool = False
    column_maxima: ColumnMaxima | None = None
    stride: int = 0


def configs() -> int:
    return _lib.library().mmh3_int8_gemm_config_count()


def group_heights() -> list[int]:
    heights = (ctypes.c_int * 8)()
    count = _lib.library().mmh3_int8_gemm_group_heights(heights, 8)
    return list(heights[:count])


def int8(tiling: Int8Tiling | None, activations: torch.Tensor, weights: torch.Tensor,
         activation_scales: torch.Tensor, weight_scales: torch.Tensor, output: Output, m: int,
         n: int, k: int, adapter: Adapter | None = None) -> None:
    """output[m, n] = round(sum_k activations[m, k] * weights[n, k] * activation_scales[m] *
    weight_scales[n] + the adapter + the bias). K must be a multiple of 128 and N of the tile
    width."""
    assert activations.numel() * activations.element_size() >= m * k, \
        "activations are smaller than m x k"
    assert weights.numel() * weights.element_size() >= n * k, "weights are smaller than n x k"
    assert activation_scales.numel() >= m, "activation scales are smaller than m"
    assert weight_scales.numel() >= n, "weight scales are smaller than n"
    row = output.stride if output.stride else (n // 2 if output.swiglu else n)
    assert output.buffer.numel() >= (m - 1) * row + (n // 2 if output.swiglu else n), \
        "output is smaller than its m rows"
    if output.bias is not None:
        assert output.bias.numel() >= n, "bias is smaller than n"
    maxima = output.column_maxima
    if maxima is not None:
        assert maxima.first_column <= n and \
            maxima.values.numel() >= (n - maxima.first_column) // 128, \
            "column maxima are smaller than the groups of 128 columns from first_column"
    if adapter is not None:
        assert adapter.down_stride >= adapter.rank and \
            adapter.down.numel() >= m * adapter.down_stride, \
            "adapter down activations are smaller than m x down_stride"
        assert adapter.up.numel() >= n * adapter.rank, "adapter up weights are smaller than n x rank"
        down, up, rank, down_stride, scale = (adapter.down, adapter.up, adapter.rank,
                                              adapter.down_stride, adapter.scale)
    else:
        down, up, rank, down_stride, scale = None, None, 0, 0, 0.0
    check(_lib.library().mmh3_int8_gemm(
        -1 if tiling is None else tiling.config, 0 if tiling is None else tiling.group_m,
        _pointer(activations), _pointer(weights), _pointer(activation_scales),
        _pointer(weight_scales), _pointer(output.bias), _pointer(output.buffer), int(output.f16),
        int(output.swiglu), m, n, k, output.stride, _pointer(down), _pointer(up), rank,
        down_stride, scale, _pointer(None if maxima is None else maxima.values),
        0 if maxima is None else maxima.first_column, _stream()), "mmh3_int8_gemm")


def interleave_swiglu_rows(source: torch.Tensor, destination: torch.Tensor, rows: int,
                           row_bytes: int) -> None:
    """Reorders [rows, row_bytes] whose first half are SwiGLU gates and second half the matching
    up projections into groups of eight rows: four gates, then their up projections."""
    assert source.numel() * source.element_size() >= rows * row_bytes
    assert destination.numel() * destination.element_size() >= rows * row_bytes
    check(_lib.library().mmh3_interleave_swiglu_rows(
        _pointer(source), _pointer(destination), rows, row_bytes, _stream()),
        "mmh3_interleave_swiglu_rows")
