"""Pins the CPU oracle to the known answers the reference's own tests hold for this path.

Each case names the reference test it restates. Runs without a GPU.
"""

import ctypes

import numpy as np
import pytest

import oracle_lib
from mmh3_b200 import synthetic
from mmh3_b200.vsa import FASTH3_SPARSITY, PackedLayout, VsaPlan



def oracle_plan(oracle, text, frames, height, width, audio):
    tiles = oracle.oracle_vsa_plan(text, frames, height, width, audio, None, None, None, None)
    starts = np.zeros(tiles, dtype=np.int32)
    lengths = np.zeros(tiles, dtype=np.int32)
    video = frames * (height // 2) * (width // 2)
    order = np.zeros(video, dtype=np.int32)
    meta = np.zeros(3, dtype=np.int32)
    oracle.oracle_vsa_plan(text, frames, height, width, audio, oracle_lib.ptr(starts),
                           oracle_lib.ptr(lengths), oracle_lib.ptr(order), oracle_lib.ptr(meta))
    return starts, lengths, order, meta


def test_bf16_rounding_matches_numeric_rs(oracle):
    """crates/mmh3-core/src/numeric.rs:7-13: nearest, ties to even."""
    assert oracle.oracle_f32_to_bf16(1.0) == 0x3F80
    # 1 + 2^-8 is a tie between 0x3F80 and 0x3F81: to even. 1 + 3 * 2^-8 ties up to 0x3F82.
    assert oracle.oracle_f32_to_bf16(1.00390625) == 0x3F80
    assert oracle.oracle_f32_to_bf16(1.01171875) == 0x3F82
    assert oracle.oracle_f32_to_bf16(-2.0) == 0xC000
    values = np.linspace(-3, 3, 1001, dtype=np.float32)
    ours = synthetic.to_bf16_bits(values)
    assert all(ours[i] == oracle.oracle_f32_to_bf16(float(values[i])) for i in range(values.size))


def test_lcg_matches_the_reference_generator(oracle):
    """crates/mmh3-cuda/tests/attention.rs:8-16, against an independent Python evaluation."""
    state = 200 * 31 + 3
    expected = []
    for _ in range(5):
        state = (state * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        expected.append(np.float32(-2.0) + np.float32(4.0) * (np.float32(state >> 40)
                                                             / np.float32(1 << 24)))
    values, final = oracle_lib.lcg(oracle, 200 * 31 + 3, 5, -2.0, 2.0)
    assert final == state
    assert np.array_equal(values, np.array(expected, dtype=np.float32))


def test_e4m3_conversion_known_values(oracle):
    """E4M3 with saturation to 448 and round to nearest even (the __NV_SATFINITE, __NV_E4M3
    conversion of crates/mmh3-cuda/kernels/quantized_attention.cu:146)."""
    known = {0.0: 0x00, 448.0: 0x7E, -448.0: 0xFE, 1e9: 0x7E, 1.0: 0x38, 1.0625: 0x38,
             1.1875: 0x3A, 2.0 ** -9: 0x01, 2.0 ** -10: 0x00, 3 * 2.0 ** -10: 0x02,
             464.0: 0x7E, 0.015625: 0x08}
    for value, code in known.items():
        assert oracle.oracle_f32_to_e4m3(value) == code, value
    for code in list(range(0x7F)) + list(range(0x80, 0xFF)):
        assert oracle.oracle_f32_to_e4m3(oracle.oracle_e4m3_to_f32(code)) == (
            code if code != 0x80 else 0x80)


def test_tiles_the_prefix_and_the_video_cubes(oracle):
    """crates/mmh3-core/src/dit/vsa.rs:272-294."""
    starts, lengths, order, meta = oracle_plan(oracle, 70, 5, 6, 12, 40)
    assert meta[0] == 4
    assert list(starts[:4]) == [0, 64, 70, 134]
    assert list(lengths[:4]) == [64, 6, 64, 16]
    assert len(starts) - meta[0] == 4
    assert list(lengths[4:]) == [48, 24, 12, 6]
    assert starts[4] == 150
    assert starts[7] == 150 + 48 + 24 + 12
    assert list(order[:6]) == [0, 1, 2, 3, 6, 7]
    assert sorted(order) == list(range(90))
    # The host-side plan of the package agrees with the oracle's.
    plan = VsaPlan.for_layout(PackedLayout.text_to_video(70, 5, 6, 12, 40))
    assert list(plan.tile_starts) == list(starts) and list(plan.tile_lengths) == list(lengths)
    assert list(plan.video_order) == list(order) and plan.prefix_tiles == 4
    sequence = plan.sequence_order(meta[2])
    assert sorted(sequence) == list(range(meta[2]))


def test_counts_kept_tiles_like_fastvideo(oracle):
    """crates/mmh3-core/src/dit/vsa.rs:296-304: 8 x 6 x 11 tiles, 528 -> 53 at sparsity 0.9."""
    starts, lengths, order, meta = oracle_plan(oracle, 36, 32, 48, 84, 124)
    video_tiles = len(starts) - meta[0]
    assert video_tiles == 528
    assert oracle.oracle_vsa_kept(video_tiles, FASTH3_SPARSITY) == 53
    assert oracle.oracle_vsa_kept(video_tiles, 0.0) == 528
    plan = VsaPlan.for_layout(PackedLayout.text_to_video(36, 32, 48, 84, 124))
    assert plan.video_tiles == 528 and plan.kept_video_tiles(FASTH3_SPARSITY) == 53


def test_benchmark_video_plan():
    """The 31 x 48 x 84 grid: 8 prefix tiles, 1,764 tiles of 64 and 252 of 48, 252 kept at 0.875."""
    layout, plan = synthetic.video_plan()
    assert len(layout) == 124992 + 512
    assert plan.prefix_tiles == 8 and plan.video_tiles == 2016
    assert sum(1 for length in plan.tile_lengths[8:] if length == 64) == 1764
    assert sum(1 for length in plan.tile_lengths[8:] if length == 48) == 252
    assert plan.kept_video_tiles(0.875) == 252


def test_selects_the_prefix_and_the_best_video_tiles(oracle):
    """crates/mmh3-core/src/dit/vsa.rs:349-357, ties to the lower index."""
    scores = np.array([0.0, 0.0, 3.0, 1.0, 5.0, 1.0], dtype=np.float32)
    selected = np.zeros(6, dtype=np.int32)

    def select(query_tile, prefix, kept):
        count = oracle.oracle_select_tiles(oracle_lib.ptr(scores), 6, query_tile, prefix, kept,
                                           oracle_lib.ptr(selected))
        return list(selected[:count])

    assert select(3, 2, 2) == [0, 1, 2, 4]
    assert select(3, 2, 3) == [0, 1, 2, 3, 4]
    assert select(1, 2, 1) == [0, 1, 2, 3, 4, 5]


def test_keeping_every_tile_without_a_gate_is_dense_attention(oracle):
    """crates/mmh3-core/src/dit/vsa.rs:306-347."""
    starts, lengths, order, meta = oracle_plan(oracle, 10, 1, 4, 8, 5)
    tokens, heads, dim = int(meta[2]), 2, 4
    values = np.array([((index * 37 % 17) - 8.0) / 8.0 for index in range(tokens * heads * dim)],
                      dtype=np.float32)
    output = np.zeros_like(values)
    video_tiles = len(starts) - meta[0]
    oracle.oracle_vsa_reference(oracle_lib.ptr(values), oracle_lib.ptr(values),
                                oracle_lib.ptr(values), None, oracle_lib.ptr(starts),
                                oracle_lib.ptr(lengths), len(starts), int(meta[0]), heads, dim, 0.5,
                                video_tiles, oracle_lib.ptr(output))
    table = values.reshape(tokens, heads, dim).astype(np.float64)
    result = output.reshape(tokens, heads, dim)
    for token, head in [(0, 0), (12, 1), (tokens - 1, 0)]:
        scores = table[:, head] @ table[token, head] * 0.5
        weights = np.exp(scores - scores.max())
        expected = weights @ table[:, head] / weights.sum()
        assert np.max(np.abs(result[token, head] - expected)) < 1e-5
    # The dense oracle gives the same answer, which ties the two restatements together.
    dense = np.zeros_like(values)
    oracle.oracle_attention_f32(oracle_lib.ptr(values), oracle_lib.ptr(values),
                                oracle_lib.ptr(values), oracle_lib.ptr(dense), tokens, heads, dim,
                                0.5, 1)
    assert np.max(np.abs(dense - output)) < 1e-6


def test_zero_queries_produce_uniform_means(oracle):
    """crates/mmh3-cuda/tests/quantized_attention.rs:86-126: with q = 0 and v = +-448 (exact in
    E4M3, scale one) the quantized attention returns the BF16-rounded mean, exactly."""
    for tokens in [1, 63, 64, 65, 129]:
        qkv = np.zeros((tokens, 3, 1, 128), dtype=np.float32)
        token_index, dimension = np.meshgrid(np.arange(tokens), np.arange(128), indexing="ij")
        qkv[:, 2, 0] = np.where((token_index + dimension) % 2 == 0, 448.0, -448.0)
        bits = synthetic.to_bf16_bits(qkv.reshape(-1))
        blocks = -(-tokens // 64)
        quantized = [np.zeros(tokens * 128, dtype=np.int8) for _ in range(2)]
        scales = [np.zeros(blocks, dtype=np.float32) for _ in range(2)]
        for part in range(2):
            oracle.oracle_quantize_rows(ctypes.c_void_p(bits.ctypes.data + part * 256), 384, 128,
                                        tokens, 1, None, None, 0, oracle_lib.ptr(quantized[part]),
                                        oracle_lib.ptr(scales[part]))
        value8 = np.zeros(128 * blocks * 64, dtype=np.uint8)
        value_scales = np.zeros(1, dtype=np.float32)
        value_maxima = np.zeros(blocks, dtype=np.float32)
        oracle.oracle_quantize_value(ctypes.c_void_p(bits.ctypes.data + 512), 384, 128, tokens, 1,
                                     None, None, 0, oracle_lib.ptr(value8),
                                     oracle_lib.ptr(value_scales), oracle_lib.ptr(value_maxima))
        assert value_scales[0] == 1.0
        output = np.zeros(tokens * 128, dtype=np.uint16)
        oracle.oracle_quantized_attention(
            oracle_lib.ptr(quantized[0]), oracle_lib.ptr(quantized[1]), oracle_lib.ptr(value8),
            oracle_lib.ptr(scales[0]), oracle_lib.ptr(scales[1]), oracle_lib.ptr(value_scales),
            tokens, 1, synthetic.softmax_scale(), None, None, 0, None, None, None, 0, None,
            oracle_lib.ptr(output), 128, 128)
        mean = 0.0 if tokens % 2 == 0 else np.float32(448.0) / np.float32(tokens)
        expected = synthetic.to_bf16_bits(
            np.array([mean if index % 2 == 0 else -mean for index in range(tokens * 128)],
                     dtype=np.float32))
        # As floats, as the reference's assert_eq! compares them (so -0.0 equals 0.0).
        assert np.array_equal(synthetic.bf16_bits_to_f32(output),
                              synthetic.bf16_bits_to_f32(expected)), tokens


def test_score_tree_is_a_dot_product(oracle):
    rng = np.random.default_rng(1)
    q = rng.standard_normal(128).astype(np.float32)
    k = rng.standard_normal(128).astype(np.float32)
    score = oracle.oracle_vsa_score(oracle_lib.ptr(q), oracle_lib.ptr(k), 0.25)
    assert abs(score - float(q.astype(np.float64) @ k.astype(np.float64)) * 0.25) < 1e-4


def test_shard_even_cuts(oracle):
    """crates/mmh3-core/src/shard.rs:168-188: equal contiguous cuts on the alignment, the
    remainder to the last rank."""
    boundaries = np.zeros(9, dtype=np.int64)
    oracle.oracle_shard_even(125504, 8, 1, oracle_lib.ptr(boundaries))
    assert list(boundaries) == [15688 * rank for rank in range(8)] + [125504]
    oracle.oracle_shard_even(1000, 3, 64, oracle_lib.ptr(boundaries))
    assert list(boundaries[:4]) == [0, 320, 640, 1000]
    oracle.oracle_shard_even(32, 8, 1, oracle_lib.ptr(boundaries))
    assert list(boundaries) == [4 * rank for rank in range(9)]
