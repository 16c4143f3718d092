"""Pins the Sol-Attn oracle to the known answers of the reference's own tests
(crates/mmh3-core/src/dit/sparse.rs:237-295) and checks, on the CPU, that the decomposition the
kernels use (routes + pooled tail + row offsets) reproduces the f64 reference. Runs without a GPU.
"""

import numpy as np

import oracle_lib
from mmh3_b200 import synthetic
from mmh3_b200.attention import SparseSinks
from mmh3_b200.vsa import PackedLayout


def test_routes_everything_like_dense_attention(oracle):
    """sparse.rs:240-277: with every block exact the pooled terms vanish and the result is plain
    softmax attention."""
    tokens, heads, dim = 70, 1, 4
    values = np.array([((index * 37 % 17) - 8.0) / 8.0 for index in range(tokens * heads * dim)],
                      dtype=np.float32).reshape(tokens, heads, dim)
    output, routed = oracle_lib.sol_reference(oracle, values, values, values, tau=0.0, scale=0.5,
                                              sinks=(0, 2, 0, 0))
    assert routed == 1.0
    flat = values.reshape(tokens, dim).astype(np.float64)
    for token in (0, 33, 69):
        scores = flat @ flat[token] * 0.5
        weights = np.exp(scores - scores.max())
        expected = weights @ flat / weights.sum()
        assert np.abs(output[token, 0] - expected).max() < 1e-5


def test_places_the_h3_sinks_on_the_conditioning():
    """sparse.rs:279-294: 100 text tokens and 74 audio rows put the video at token 174."""
    layout = PackedLayout.text_to_video(100, 7, 16, 28, 37)
    assert SparseSinks.for_layout(layout) == SparseSinks((0, 3), (1, 3))


def merge_routes_and_tails(work, q, k, v, tokens, heads, scale):
    """What the token attention kernel computes from the routing workspace, in f64."""
    log2_scale = scale * np.log2(np.e)
    output = np.zeros((tokens, heads, 128))
    blocks = -(-tokens // 64)
    for head in range(heads):
        for block in range(blocks):
            rows = slice(block * 64, min(tokens, block * 64 + 64))
            count = work["route_counts"][head, block]
            keys = np.concatenate([np.arange(b * 64, min(tokens, b * 64 + 64))
                                   for b in work["routes"][head, block, :count]])
            scores = q[rows, head] @ k[keys, head].T * log2_scale
            centred = scores - work["row_offsets"][head, rows][:, None]
            tail_max = work["tail_max"][head, block]
            merged = np.maximum(centred.max(axis=1), tail_max)
            weights = np.exp2(centred - merged[:, None])
            tail_weight = np.exp2(tail_max - merged)
            numerator = weights @ v[keys, head] + \
                tail_weight[:, None] * work["tail_values"][head, block][None, :]
            denominator = weights.sum(axis=1) + tail_weight * work["tail_sum"][head, block]
            output[rows, head] = numerator / denominator[:, None]
    return output


def test_routes_and_pooled_tails_reproduce_the_reference(oracle):
    """The FP32 routing workspace (sparse_attention.cu:72-338 in kernel order) merged the way the
    token attention kernel merges it (:493-523) equals the dense f64 reference (sparse.rs:103-234)
    on a sequence with a ragged last block, sinks and a threshold that leaves most blocks pooled."""
    tokens, heads, tau = 64 * 9 + 23, 2, 0.7
    scale = synthetic.softmax_scale()
    qkv = synthetic.dense_qkv(tokens, heads, seed=11)
    bits = qkv.view(__import__("torch").int16).numpy().view(np.uint16)
    sinks = (0, 1, 2, 3)
    work = oracle_lib.sol_route(oracle, bits, tokens, heads, tau, scale, sinks)
    values = qkv.float().numpy().astype(np.float32)
    q, k, v = values[:, 0], values[:, 1], values[:, 2]
    reference, routed = oracle_lib.sol_reference(oracle, q, k, v, tau, scale, sinks)
    blocks = -(-tokens // 64)
    assert routed == work["route_counts"].sum() / (heads * blocks * blocks)
    assert 0.2 < routed < 0.9  # some blocks exact, some pooled
    # Query block 2 is a sink: it routes every key block; key block 0 is in every route.
    assert (work["route_counts"][:, 2] == blocks).all()
    assert (work["routes"][:, :, 0] == 0).all()
    merged = merge_routes_and_tails(work, q.astype(np.float64), k.astype(np.float64),
                                    v.astype(np.float64), tokens, heads, scale)
    assert np.abs(merged - reference).max() < 2e-4


def test_oracle_matches_the_reference_kernels_fixture(oracle):
    """tests/golden/reference_sol.npz holds what the reference's own CUDA kernels
    (sparse_attention.cu, compiled from its sources) left in the workspace for a seeded input
    (tests/golden/make_golden.py): the routing restatement reproduces the statistics, the centred
    keys and the routes bit for bit, the tails and offsets closely, and the f64 reference the
    output within the reference test's bounds."""
    import pathlib
    import sys

    golden_directory = pathlib.Path(__file__).resolve().parent / "golden"
    sys.path.insert(0, str(golden_directory))
    import make_golden

    golden = np.load(golden_directory / "reference_sol.npz")
    case = make_golden.SOL_CASE
    tokens, heads = case["tokens"], case["heads"]
    scale = synthetic.softmax_scale()
    bits = make_golden.sol_inputs(oracle, tokens, heads)
    work = oracle_lib.sol_route(oracle, bits, tokens, heads, case["tau"], scale, case["sinks"])
    for name in ("centroids", "block_keys", "value_sums", "key_mean", "key_variance", "tail_max"):
        assert np.array_equal(work[name].reshape(-1).view(np.uint32),
                              golden[name].reshape(-1).view(np.uint32)), name
    assert np.array_equal(work["route_counts"], golden["route_counts"])
    blocks = -(-tokens // 64)
    packed = np.concatenate([work["routes"][head, block, :work["route_counts"][head, block]]
                             for head in range(heads) for block in range(blocks)])
    assert np.array_equal(packed, golden["routes"])
    for name in ("tail_sum", "tail_values", "row_offsets"):
        assert np.allclose(work[name].reshape(-1), golden[name].reshape(-1), rtol=1e-4,
                           atol=1e-4), name
    values = synthetic.bf16_bits_to_f32(bits)
    expected, _ = oracle_lib.sol_reference(oracle, values[:, 0], values[:, 1], values[:, 2],
                                           case["tau"], scale, case["sinks"])
    actual = synthetic.bf16_bits_to_f32(golden["output"]).reshape(expected.shape)
    difference = np.linalg.norm((actual - expected).astype(np.float64))
    assert difference / np.linalg.norm(expected.astype(np.float64)) < 0.01
    assert np.max(np.abs(actual - expected)) < 0.05
