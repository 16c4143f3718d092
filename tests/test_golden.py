"""Holds the CPU oracle to outputs of the REFERENCE's own CUDA kernels.

tests/golden/reference_kernels.npz was written on a B200 by tests/golden/make_golden.py from the
reference's attention kernels compiled from its sources. Inputs are regenerated here from the same
seeds. INT8 q and k, scales, FP8 V, pooled tiles and routes must match bit for bit; outputs within
the tolerance of the reference's own tests. Runs without a GPU.
"""

import ctypes
import pathlib

import numpy as np
import pytest

import oracle_lib
from mmh3_b200 import synthetic
from mmh3_b200.vsa import PackedLayout, VsaPlan

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden" / "reference_kernels.npz"
SCALE = synthetic.softmax_scale()


@pytest.fixture(scope="module")
def golden():
    if not GOLDEN.exists():
        pytest.skip("no golden fixture")
    return np.load(GOLDEN)


def lcg_qkv(oracle, tokens, heads, seed):
    values, _ = oracle_lib.lcg(oracle, seed, tokens * 3 * heads * 128, -2.0, 2.0)
    return synthetic.to_bf16_bits(values).reshape(tokens, 3, heads, 128)


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


@pytest.mark.parametrize("tokens,heads", [(1, 1), (64, 2), (200, 3)])
def test_dense_oracle_against_the_reference_kernel(oracle, golden, tokens, heads):
    bits = lcg_qkv(oracle, tokens, heads, tokens * 31 + heads)
    expected = oracle_lib.attention_bf16(oracle, bits, tokens, heads, SCALE)
    actual = synthetic.bf16_bits_to_f32(golden[f"dense_{tokens}_{heads}"]).reshape(expected.shape)
    assert np.all(np.abs(actual - expected) <= 0.02 + 0.01 * np.abs(expected))


@pytest.mark.parametrize("tokens,heads", [(65, 2), (200, 3)])
def test_quantizer_oracle_against_the_reference_kernels(oracle, golden, tokens, heads):
    inner = heads * 128
    blocks = -(-tokens // 64)
    bits = lcg_qkv(oracle, tokens, heads, tokens * 17 + heads)
    flat = np.ascontiguousarray(bits.reshape(-1))
    key = f"quantized_{tokens}_{heads}"
    quantized, scales = {}, {}
    for part, name in ((0, "query"), (1, "key")):
        quantized[name] = np.zeros(tokens * inner, dtype=np.int8)
        scales[name] = np.zeros(heads * blocks, dtype=np.float32)
        oracle.oracle_quantize_rows(ctypes.c_void_p(flat.ctypes.data + part * inner * 2),
                                    3 * inner, 128, tokens, heads, None, None, 0,
                                    oracle_lib.ptr(quantized[name]), oracle_lib.ptr(scales[name]))
        assert np.array_equal(quantized[name].view(np.uint8), golden[f"{key}_{name}"])
        assert np.array_equal(scales[name].view(np.uint32),
                              golden[f"{key}_{name}_scales"].view(np.uint32))
    value8 = np.zeros(heads * 128 * blocks * 64, dtype=np.uint8)
    value_scales = np.zeros(heads, dtype=np.float32)
    value_maxima = np.zeros(heads * blocks, dtype=np.float32)
    oracle.oracle_quantize_value(ctypes.c_void_p(flat.ctypes.data + 2 * inner * 2), 3 * inner, 128,
                                 tokens, heads, None, None, 0, oracle_lib.ptr(value8),
                                 oracle_lib.ptr(value_scales), oracle_lib.ptr(value_maxima))
    assert np.array_equal(value8, golden[f"{key}_value"])
    assert np.array_equal(value_scales.view(np.uint32),
                          golden[f"{key}_value_scales"].view(np.uint32))
    assert np.array_equal(value_maxima.view(np.uint32),
                          golden[f"{key}_value_maxima"].view(np.uint32))
    output = np.zeros(tokens * inner, dtype=np.uint16)
    oracle.oracle_quantized_attention(
        oracle_lib.ptr(quantized["query"]), oracle_lib.ptr(quantized["key"]),
        oracle_lib.ptr(value8), oracle_lib.ptr(scales["query"]), oracle_lib.ptr(scales["key"]),
        oracle_lib.ptr(value_scales), tokens, heads, SCALE, None, None, 0, None, None, None, 0,
        None, oracle_lib.ptr(output), inner, 128)
    ours = synthetic.bf16_bits_to_f32(output)
    theirs = synthetic.bf16_bits_to_f32(golden[f"{key}_output"]).reshape(-1)
    assert cosine(ours, theirs) >= 0.9995
    assert np.max(np.abs(ours - theirs)) <= 0.05


def test_vsa_oracle_against_the_reference_kernels(oracle, golden):
    layout = PackedLayout.text_to_video(70, 9, 16, 24, 40)
    plan = VsaPlan.for_layout(layout)
    tokens, heads = len(layout), 2
    inner = heads * 128
    kept = plan.kept_video_tiles(0.7)
    state = tokens + heads
    directions, state = oracle_lib.lcg(oracle, state, plan.tiles * 3 * inner, -1.0, 1.0)
    tile_of = np.zeros(tokens, dtype=np.int64)
    for tile, (start, length) in enumerate(zip(plan.tile_starts, plan.tile_lengths)):
        tile_of[start:start + length] = tile
    noise, state = oracle_lib.lcg(oracle, state, tokens * 3 * inner, -1.0, 1.0)
    qkv = directions.reshape(plan.tiles, 3 * inner)[tile_of] + noise.reshape(tokens, 3 * inner)
    bits = synthetic.to_bf16_bits(qkv.reshape(-1)).reshape(tokens, 3, heads, 128)
    flat = np.ascontiguousarray(bits.reshape(-1))
    base = flat.ctypes.data
    token_stride = np.array([3 * inner] * 3, dtype=np.int64)
    head_stride = np.array([128] * 3, dtype=np.int64)
    starts = np.array(plan.tile_starts, dtype=np.int32)
    lengths = np.array(plan.tile_lengths, dtype=np.int32)
    pooled = [np.empty((heads, plan.tiles, 128), dtype=np.float32) for _ in range(3)]
    oracle.oracle_vsa_pool(ctypes.c_void_p(base), ctypes.c_void_p(base + 2 * inner),
                           ctypes.c_void_p(base + 4 * inner), oracle_lib.ptr(token_stride),
                           oracle_lib.ptr(head_stride), heads, oracle_lib.ptr(starts),
                           oracle_lib.ptr(lengths), plan.tiles,
                           *(oracle_lib.ptr(buffer) for buffer in pooled))
    for buffer, name in zip(pooled, ("pooled_query", "pooled_key", "pooled_value")):
        assert np.array_equal(buffer.reshape(-1).view(np.uint32),
                              golden[f"vsa_{name}"].view(np.uint32)), name
    routes = np.zeros((heads, plan.tiles, plan.tiles), dtype=np.uint16)
    counts = np.zeros((heads, plan.tiles), dtype=np.int32)
    oracle.oracle_vsa_select(oracle_lib.ptr(pooled[0]), oracle_lib.ptr(pooled[1]), heads,
                             plan.tiles, plan.prefix_tiles, kept, SCALE, oracle_lib.ptr(routes),
                             oracle_lib.ptr(counts), None)
    assert np.array_equal(counts, golden["vsa_route_counts"])
    packed = np.concatenate([routes[head, tile, :counts[head, tile]]
                             for head in range(heads) for tile in range(plan.tiles)])
    assert np.array_equal(packed, golden["vsa_routes"])
    values = synthetic.bf16_bits_to_f32(bits)
    parts = [np.ascontiguousarray(values[:, part]) for part in range(3)]
    expected = np.zeros((tokens, heads, 128), dtype=np.float32)
    oracle.oracle_vsa_reference(*(oracle_lib.ptr(part) for part in parts), None,
                                oracle_lib.ptr(starts), oracle_lib.ptr(lengths), plan.tiles,
                                plan.prefix_tiles, heads, 128, SCALE, kept,
                                oracle_lib.ptr(expected))
    actual = synthetic.bf16_bits_to_f32(golden["vsa_output"]).reshape(expected.shape)
    difference = np.linalg.norm((actual - expected).astype(np.float64))
    assert difference / np.linalg.norm(expected.astype(np.float64)) < 0.01
    assert np.max(np.abs(actual - expected)) < 0.05
