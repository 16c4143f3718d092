"""Parity of video sparse attention on a B200, through the C ABI.

Mirrors crates/mmh3-cuda/tests/vsa_attention.rs (layout with partial cubes, sparsity 0.7 and 0.0,
gated and not, the closed-form selected fraction, relative L2 < 0.01 and max error < 0.05 against the
f64 reference) and adds what the drop-in must hold bit for bit: the pooled tiles, the routes and the
route counts, against both the CPU oracle and the reference's own kernels.
"""

import ctypes

import numpy as np
import pytest
import torch

import oracle_lib
from mmh3_b200 import attention, synthetic
from mmh3_b200.vsa import PackedLayout, VsaPlan

pytestmark = pytest.mark.gpu

SCALE = synthetic.softmax_scale()


def make_case(oracle, layout, heads):
    """The tokens of a tile share a random direction, so pooled scores spread
    (vsa_attention.rs:38-62)."""
    plan = VsaPlan.for_layout(layout)
    tokens = len(layout)
    inner = heads * 128
    state = tokens + heads
    directions, state = oracle_lib.lcg(oracle, state, plan.tiles * 3 * inner, -1.0, 1.0)
    tile_of = np.zeros(tokens, dtype=np.int64)
    for tile, (start, length) in enumerate(zip(plan.tile_starts, plan.tile_lengths)):
        tile_of[start:start + length] = tile
    noise, state = oracle_lib.lcg(oracle, state, tokens * 3 * inner, -1.0, 1.0)
    qkv = directions.reshape(plan.tiles, 3 * inner)[tile_of] + noise.reshape(tokens, 3 * inner)
    gate, state = oracle_lib.lcg(oracle, state, tokens * inner, -2.0, 2.0)
    return (plan, synthetic.to_bf16_bits(qkv.reshape(-1)).reshape(tokens, 3, heads, 128),
            synthetic.to_bf16_bits(gate).reshape(tokens, heads, 128))


def oracle_reference(oracle, plan, bits, gate_bits, heads, kept):
    tokens = bits.shape[0]
    values = synthetic.bf16_bits_to_f32(bits)
    parts = [np.ascontiguousarray(values[:, part]) for part in range(3)]
    gate = np.ascontiguousarray(synthetic.bf16_bits_to_f32(gate_bits)) if gate_bits is not None else None
    starts = np.array(plan.tile_starts, dtype=np.int32)
    lengths = np.array(plan.tile_lengths, dtype=np.int32)
    output = np.zeros((tokens, heads, 128), dtype=np.float32)
    oracle.oracle_vsa_reference(*(oracle_lib.ptr(part) for part in parts), oracle_lib.ptr(gate),
                                oracle_lib.ptr(starts), oracle_lib.ptr(lengths), plan.tiles,
                                plan.prefix_tiles, heads, 128, SCALE, kept, oracle_lib.ptr(output))
    return output


def oracle_routes(oracle, plan, bits, heads, kept):
    """Pooled tiles, routes and counts as the CPU restatement of pool + select leaves them."""
    inner = heads * 128
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
    routes = np.zeros((heads, plan.tiles, plan.tiles), dtype=np.uint16)
    counts = np.zeros((heads, plan.tiles), dtype=np.int32)
    oracle.oracle_vsa_select(oracle_lib.ptr(pooled[0]), oracle_lib.ptr(pooled[1]), heads,
                             plan.tiles, plan.prefix_tiles, kept, SCALE, oracle_lib.ptr(routes),
                             oracle_lib.ptr(counts), None)
    return pooled, routes, counts


def assert_routes_equal(routes_a, counts_a, routes_b, counts_b):
    assert np.array_equal(counts_a, counts_b)
    heads, tiles = counts_a.shape
    for head in range(heads):
        for tile in range(tiles):
            count = counts_a[head, tile]
            assert np.array_equal(routes_a[head, tile, :count], routes_b[head, tile, :count]), (
                head, tile)


CASES = [(2, 0.7, False), (3, 0.7, True), (2, 0.0, True)]


@pytest.mark.parametrize("heads,sparsity,gated", CASES)
def test_matches_the_reference(oracle, reference_kernels, heads, sparsity, gated):
    # 150 prefix tokens, then a 9 x 8 x 12 patch grid in 3 x 2 x 3 cubes, some of them partial.
    layout = PackedLayout.text_to_video(70, 9, 16, 24, 40)
    plan, bits, gate_bits = make_case(oracle, layout, heads)
    tokens = len(layout)
    inner = heads * 128
    kept = plan.kept_video_tiles(sparsity)
    qkv = synthetic.bf16_tensor(bits, "cuda")
    gate = synthetic.bf16_tensor(gate_bits, "cuda") if gated else None
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.VsaWorkspace(plan, tokens, heads)
    vsa_layout = attention.qkv_layout(heads)
    attention.vsa(qkv, gate, output, vsa_layout, SCALE, kept, workspace)
    assert attention.take_status() == 0

    # Routing: closed form, CPU oracle, and the reference's kernels.
    assert abs(workspace.selected_fraction() - plan.expected_selected_fraction(kept)) < 1e-9
    routes, counts = workspace.routes_host()
    pooled, oracle_route_list, oracle_counts = oracle_routes(oracle, plan, bits, heads, kept)
    for ours, theirs in zip((workspace.pooled_query, workspace.pooled_key, workspace.pooled_value),
                            pooled):
        assert np.array_equal(ours.cpu().numpy().view(np.uint32), theirs.reshape(-1).view(np.uint32))
    assert_routes_equal(routes, counts, oracle_route_list, oracle_counts)

    theirs = attention.VsaWorkspace(plan, tokens, heads)
    reference_output = torch.zeros_like(output)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_vsa_attention(
        base, base + 2 * inner, base + 4 * inner, gate.data_ptr() if gated else None, inner,
        reference_output.data_ptr(), tokens, heads, ctypes.byref(vsa_layout), SCALE, plan.tiles,
        plan.prefix_tiles, kept, ctypes.byref(raw), None, 0, None) == 0
    torch.cuda.synchronize()
    assert_routes_equal(routes, counts, *theirs.routes_host())
    if gated:
        assert torch.allclose(workspace.coarse, theirs.coarse, rtol=1e-4, atol=1e-5)

    # Outputs: the f64 reference, then the reference's kernel.
    expected = oracle_reference(oracle, plan, bits, gate_bits if gated else None, heads, kept)
    actual = output.float().cpu().numpy()
    difference = np.linalg.norm((actual - expected).astype(np.float64))
    norm = np.linalg.norm(expected.astype(np.float64))
    assert difference / norm < 0.01
    assert np.max(np.abs(actual - expected)) < 0.05
    other = reference_output.float().cpu().numpy()
    assert np.max(np.abs(actual - other)) < 0.05
