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
    # The neighbour-overlap diagnostic against the reference's loops (attention.rs:1023-1047).
    pairs, separate, merged = 0, 0.0, 0.0
    for head in range(heads):
        for tile in range(0, plan.tiles - 1, 2):
            lists = [routes[head, other, :counts[head, other]] for other in (tile, tile + 1)]
            if len(lists[0]) + len(lists[1]) == 0:
                continue
            pairs += 1
            separate += len(lists[0]) + len(lists[1])
            merged += len({int(target) for target in np.concatenate(lists) if target < plan.tiles})
    found = workspace.route_overlap()
    assert found[0] == pairs
    assert abs(found[1] - separate / pairs) < 1e-9 and abs(found[2] - merged / pairs) < 1e-9
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


def prepared_case(oracle, layout, heads):
    """Inputs with norm weights and angles, and the normalized rows the attention then sees."""
    from test_inputs_gpu import EPSILON, make_inputs, norm_for

    tokens = len(layout)
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads)
    norm = norm_for(query_weight, key_weight, angles)
    normalized = synthetic.bf16_tensor(bits, "cuda")
    attention.qk_norm_rope(normalized, norm, tokens, heads)
    normalized_bits = normalized.view(torch.int16).cpu().numpy().view(np.uint16)
    return bits, norm, normalized_bits, EPSILON


@pytest.mark.parametrize("with_values", [False, True])
@pytest.mark.parametrize("gated", [False, True])
def test_quantized_vsa_matches_the_reference(oracle, reference_kernels, with_values, gated):
    """crates/mmh3-cuda/tests/attention_inputs.rs:423-572: INT8/FP8 VSA over prepared inputs against
    the f64 reference (relative L2 < 0.02, max error < 0.1), and against the reference's kernel."""
    layout = PackedLayout.text_to_video(70, 9, 16, 24, 40)
    plan = VsaPlan.for_layout(layout)
    tokens, heads = len(layout), 2
    inner = heads * 128
    kept = plan.kept_video_tiles(0.7)
    bits, norm, normalized_bits, epsilon = prepared_case(oracle, layout, heads)
    gate_values, _ = oracle_lib.lcg(oracle, 99, tokens * inner, -2.0, 2.0)
    gate_bits = synthetic.to_bf16_bits(gate_values).reshape(tokens, heads, 128)
    gate = synthetic.bf16_tensor(gate_bits, "cuda") if gated else None
    vsa_layout = attention.qkv_layout(heads)
    inputs = (attention.AttentionInputs.PREPARED_WITH_VALUES if with_values
              else attention.AttentionInputs.PREPARED)

    ours_qkv = synthetic.bf16_tensor(bits, "cuda")
    maxima = ours_qkv[:, 2].float().abs().amax(dim=(0, 2)).contiguous() if with_values else None
    ours = attention.VsaWorkspace(plan, tokens, heads, quantized=True)
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.prepare_inputs(ours_qkv, norm, tokens, heads, vsa=ours, value_head_maxima=maxima)
    attention.vsa(ours_qkv, gate, output, vsa_layout, SCALE, kept, ours, inputs)
    assert attention.take_status() == 0

    theirs_qkv = synthetic.bf16_tensor(bits, "cuda")
    theirs = attention.VsaWorkspace(plan, tokens, heads, quantized=True)
    reference_output = torch.zeros_like(output)
    sparse, quantized, raw = theirs.sparse_raw(), theirs.quantized.raw(), theirs.raw()
    assert reference_kernels.mmh3_attention_inputs(
        theirs_qkv.data_ptr(), norm.query_weight.data_ptr(), norm.key_weight.data_ptr(),
        norm.angles.data_ptr(), norm.pairs, tokens, heads, epsilon, ctypes.byref(sparse),
        ctypes.byref(quantized), theirs.tile_starts.data_ptr(), theirs.tile_lengths.data_ptr(),
        theirs.tiles, maxima.data_ptr() if with_values else None, None) == 0
    base = theirs_qkv.data_ptr()
    assert reference_kernels.mmh3_vsa_attention(
        base, base + 2 * inner, base + 4 * inner, gate.data_ptr() if gated else None, inner,
        reference_output.data_ptr(), tokens, heads, ctypes.byref(vsa_layout), SCALE, plan.tiles,
        plan.prefix_tiles, kept, ctypes.byref(raw), ctypes.byref(quantized), int(inputs),
        None) == 0
    torch.cuda.synchronize()
    assert_routes_equal(*ours.routes_host(), *theirs.routes_host())
    assert torch.equal(ours.quantized.value, theirs.quantized.value)

    expected = oracle_reference(oracle, plan, normalized_bits, gate_bits if gated else None, heads,
                                kept)
    actual = output.float().cpu().numpy()
    difference = np.linalg.norm((actual - expected).astype(np.float64))
    assert difference / np.linalg.norm(expected.astype(np.float64)) < 0.02
    assert np.max(np.abs(actual - expected)) < 0.1
    other = reference_output.float().cpu().numpy()
    a, b = actual.astype(np.float64).ravel(), other.astype(np.float64).ravel()
    assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) >= 0.9995


def test_a_layout_off_the_tma_grid_gives_the_same_bits(oracle):
    """q, k and v two bytes off a 16-byte boundary with an odd token stride: the token attention
    gathers them into dense arrays first (the reference copies with cp.async instead of TMA), and
    pooled tiles, routes and output must be the bits of the aligned layout."""
    heads = 2
    layout = PackedLayout.text_to_video(70, 9, 16, 24, 40)
    plan, bits, gate_bits = make_case(oracle, layout, heads)
    tokens, inner = len(layout), heads * 128
    kept = plan.kept_video_tiles(0.75)
    qkv = synthetic.bf16_tensor(bits, "cuda")
    gate = synthetic.bf16_tensor(gate_bits, "cuda")
    results = []
    for shifted in (False, True):
        token_stride = 3 * inner + (1 if shifted else 0)
        offset = 1 if shifted else 0
        storage = torch.zeros(tokens * token_stride + 8, dtype=torch.bfloat16, device="cuda")
        torch.as_strided(storage, (tokens, 3 * inner), (token_stride, 1), offset).copy_(
            qkv.view(tokens, 3 * inner))
        vsa_layout = attention.make_layout((token_stride,) * 3 + (inner,))
        output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
        workspace = attention.VsaWorkspace(plan, tokens, heads)
        attention.vsa(storage, gate, output, vsa_layout, SCALE, kept, workspace,
                      offsets=(offset, offset + inner, offset + 2 * inner, 0))
        assert attention.take_status() == 0
        results.append((output, workspace))
    (aligned, first), (moved, second) = results
    for name in ("pooled_query", "pooled_key", "pooled_value", "route_counts", "coarse"):
        assert torch.equal(getattr(first, name), getattr(second, name)), name
    routes, counts = first.routes_host()
    other_routes, other_counts = second.routes_host()
    assert np.array_equal(counts, other_counts)
    for head in range(heads):
        for tile in range(plan.tiles):
            count = counts[head, tile]
            assert np.array_equal(routes[head, tile, :count], other_routes[head, tile, :count])
    assert torch.equal(aligned.view(torch.int16), moved.view(torch.int16))


def test_larger_plan_with_an_odd_tile_count(oracle, reference_kernels):
    """More tiles than one CTA pair, an odd tile count, and routes that differ between neighbours."""
    layout = PackedLayout.text_to_video(130, 9, 32, 48, 0)
    plan, bits, gate_bits = make_case(oracle, layout, 2)
    assert plan.tiles % 2 == 1
    tokens, heads = len(layout), 2
    inner = heads * 128
    kept = plan.kept_video_tiles(0.8)
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    reference_output = torch.zeros_like(output)
    workspace = attention.VsaWorkspace(plan, tokens, heads)
    theirs = attention.VsaWorkspace(plan, tokens, heads)
    vsa_layout = attention.qkv_layout(heads)
    attention.vsa(qkv, None, output, vsa_layout, SCALE, kept, workspace)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_vsa_attention(
        base, base + 2 * inner, base + 4 * inner, None, inner, reference_output.data_ptr(), tokens,
        heads, ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept,
        ctypes.byref(raw), None, 0, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert abs(workspace.selected_fraction() - plan.expected_selected_fraction(kept)) < 1e-9
    assert_routes_equal(*workspace.routes_host(), *theirs.routes_host())
    a = output.float().cpu().numpy().astype(np.float64).ravel()
    b = reference_output.float().cpu().numpy().astype(np.float64).ravel()
    assert np.max(np.abs(a - b)) < 0.05
    assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) >= 0.9995


def test_a_row_of_equal_scores_longer_than_the_list_of_open_tiles(reference_kernels):
    """Every key row the same, so every video tile of a row scores alike and none is certain: the
    route kernel lists at most 1,024 open tiles and takes a row with more (here all 2,016) whole.
    The routes must still be the reference kernels': the first `kept` video tiles, ties going to
    the lower index (vsa.rs:341-357 on the GPU, at the benchmark's plan)."""
    layout, plan = synthetic.video_plan()
    tokens, heads = len(layout), 1
    inner = heads * 128
    kept = plan.kept_video_tiles(0.875)
    generator = torch.Generator().manual_seed(21)
    rows = torch.randn((tokens, 3, heads, 128), generator=generator)
    rows[:, 1] = torch.randn((1, heads, 128), generator=generator)
    qkv = rows.to(torch.bfloat16).cuda()
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    reference_output = torch.zeros_like(output)
    workspace = attention.VsaWorkspace(plan, tokens, heads)
    theirs = attention.VsaWorkspace(plan, tokens, heads)
    vsa_layout = attention.qkv_layout(heads)
    attention.vsa(qkv, None, output, vsa_layout, SCALE, kept, workspace)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_vsa_attention(
        base, base + 2 * inner, base + 4 * inner, None, inner, reference_output.data_ptr(), tokens,
        heads, ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept,
        ctypes.byref(raw), None, 0, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    routes, counts = workspace.routes_host()
    assert_routes_equal(routes, counts, *theirs.routes_host())
    assert (counts[:, plan.prefix_tiles:] == plan.prefix_tiles + kept).all()
    a = output.float().cpu().numpy().astype(np.float64).ravel()
    b = reference_output.float().cpu().numpy().astype(np.float64).ravel()
    assert np.max(np.abs(a - b)) < 0.05


def test_route_lists_longer_than_the_schedule_tables(reference_kernels):
    """With 70 % of the benchmark plan's 2,016 video tiles kept a route list holds over 1,400
    tiles, more than the token attention sorts into shared memory once per CTA: it then walks the
    lists entry by entry as the steps come. Routes and output against the reference's kernels."""
    layout, plan = synthetic.video_plan()
    tokens, heads = len(layout), 1
    inner = heads * 128
    kept = plan.kept_video_tiles(0.3)
    assert kept > 1024
    qkv = synthetic.video_qkv_device(layout, plan, heads, seed=13)
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    reference_output = torch.zeros_like(output)
    workspace = attention.VsaWorkspace(plan, tokens, heads)
    theirs = attention.VsaWorkspace(plan, tokens, heads)
    vsa_layout = attention.qkv_layout(heads)
    attention.vsa(qkv, None, output, vsa_layout, SCALE, kept, workspace)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_vsa_attention(
        base, base + 2 * inner, base + 4 * inner, None, inner, reference_output.data_ptr(), tokens,
        heads, ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept,
        ctypes.byref(raw), None, 0, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert_routes_equal(*workspace.routes_host(), *theirs.routes_host())
    a = output.float().cpu().numpy().astype(np.float64).ravel()
    b = reference_output.float().cpu().numpy().astype(np.float64).ravel()
    assert np.max(np.abs(a - b)) < 0.05
    assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) >= 0.9995
