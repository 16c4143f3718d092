"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

They stand in for the DiT's activations: q and v ~ N(0, 1); k ~ N(0, 1) plus a per-channel offset
drawn once from N(0, variance 2); for the video configurations a smooth 3-D correlated component
(a trilinearly upsampled low-resolution N(0, 1) field, weight 0.5) so that tile scores differ.
Everything is generated on the CPU generator, so that host and device runs share the data, and
rounded to BF16.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .vsa import PackedLayout, VsaPlan

HEAD_DIM = 128

CONFIGS = {
    # name: (tokens, heads)
    "C0": (4096, 8),
    "C1": (65536 + 512, 32),
    "C3": (124992 + 512, 32),
}


def softmax_scale() -> float:
    return 1.0 / math.sqrt(HEAD_DIM)


def dense_qkv(tokens: int, heads: int, seed: int, pinned: bool = False) -> torch.Tensor:
    """BF16 qkv [tokens, 3, heads, 128] with the distribution of configurations C0-C2."""
    generator = torch.Generator(device="cpu").manual_seed(seed)
    qkv = torch.empty((tokens, 3, heads, HEAD_DIM), dtype=torch.bfloat16, pin_memory=pinned)
    offsets = torch.randn((heads, HEAD_DIM), generator=generator) * math.sqrt(2.0)
    chunk = max(1, (1 << 24) // (3 * heads * HEAD_DIM))
    for start in range(0, tokens, chunk):
        rows = min(chunk, tokens - start)
        block = torch.randn((rows, 3, heads, HEAD_DIM), generator=generator)
        block[:, 1] += offsets
        qkv[start:start + rows] = block.to(torch.bfloat16)
    return qkv


def lcg_uniform(state: int, count: int, low: float, high: float) -> tuple[np.ndarray, int]:
    """`count` FP32 values uniform in [low, high) from the generator of the reference's kernel
    tests (crates/mmh3-cuda/tests/attention.rs:8-16), and the advanced state."""
    mask = (1 << 64) - 1
    values = np.empty(count, dtype=np.float32)
    span = np.float32(high) - np.float32(low)
    for index in range(count):
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        values[index] = np.float32(low) + span * (np.float32(state >> 40) / np.float32(1 << 24))
    return values, state


def to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """FP32 -> BF16 bit patterns, round to nearest even (crates/mmh3-core/src/numeric.rs:7-13)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def bf16_tensor(bits: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def video_plan(text_tokens: int = 512, frames: int = 31, latent_height: int = 96,
               latent_width: int = 168) -> tuple[PackedLayout, VsaPlan]:
    """The layout and tile plan of configuration C3: a 31 x 48 x 84 patch grid after the text."""
    layout = PackedLayout.text_to_video(text_tokens, frames, latent_height, latent_width, 0)
    return layout, VsaPlan.for_layout(layout)


def video_qkv(layout: PackedLayout, plan: VsaPlan, heads: int, seed: int,
              coarse_grid=(4, 6, 11), weight: float = 0.5, pinned: bool = False) -> torch.Tensor:
    """BF16 qkv [tokens, 3, heads, 128] in the plan's cube order: N(0, 1) plus `weight` times a
    smooth field over (frame, row, column) for the video tokens, a different field per tensor,
    head and channel, evaluated at each token's own grid position."""
    generator = torch.Generator(device="cpu").manual_seed(seed)
    tokens = len(layout)
    grid = (layout.latent_frames, layout.latent_height // 2, layout.latent_width // 2)
    order = torch.tensor(plan.video_order, dtype=torch.int64)
    qkv = torch.empty((tokens, 3, heads, HEAD_DIM), dtype=torch.bfloat16, pin_memory=pinned)
    video = slice(plan.video_start, plan.video_start + len(plan.video_order))
    for head in range(heads):
        noise = torch.randn((tokens, 3, HEAD_DIM), generator=generator)
        low = torch.randn((1, 3 * HEAD_DIM, *coarse_grid), generator=generator)
        smooth = torch.nn.functional.interpolate(low, size=grid, mode="trilinear",
                                                 align_corners=True)
        smooth = smooth.reshape(3 * HEAD_DIM, -1).t().reshape(-1, 3, HEAD_DIM)
        noise[video] += weight * smooth[order]
        qkv[:, :, head, :] = noise.to(torch.bfloat16)
    return qkv


def video_qkv_device(layout: PackedLayout, plan: VsaPlan, heads: int, seed: int,
                     coarse_grid=(4, 6, 11), weight: float = 0.5, device="cuda") -> torch.Tensor:
    """`video_qkv` drawn on the device's own generator: the same distribution, and the same values
    on every GPU of one kind for one seed, without the minute the CPU generator takes at 125,504
    tokens x 32 heads. Every rank of a sharded run draws the whole tensor and keeps its rows, so
    the data does not depend on the rank count."""
    generator = torch.Generator(device=device).manual_seed(seed)
    tokens = len(layout)
    grid = (layout.latent_frames, layout.latent_height // 2, layout.latent_width // 2)
    order = torch.tensor(plan.video_order, dtype=torch.int64, device=device)
    qkv = torch.randn((tokens, 3, heads, HEAD_DIM), generator=generator, device=device,
                      dtype=torch.float32).bfloat16()
    video = slice(plan.video_start, plan.video_start + len(plan.video_order))
    for head in range(heads):
        low = torch.randn((1, 3 * HEAD_DIM, *coarse_grid), generator=generator, device=device)
        smooth = torch.nn.functional.interpolate(low, size=grid, mode="trilinear",
                                                 align_corners=True)
        smooth = smooth.reshape(3 * HEAD_DIM, -1).t().reshape(-1, 3, HEAD_DIM)[order]
        qkv[video, :, head, :] = (qkv[video, :, head, :].float() + weight * smooth).bfloat16()
    return qkv
