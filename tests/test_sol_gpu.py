"""Parity of Sol-Attn on a B200, through the C ABI.

Mirrors crates/mmh3-cuda/tests/sparse_attention.rs (per-block random directions so that routing is
selective, tau 0.5 with sinks and tau 1.3, routed fraction within 0.01 of the f64 reference and
between 0.1 and 0.9, relative L2 < 0.01 and max error < 0.05) and adds what the drop-in must hold
bit for bit: the block statistics, the centred keys, their mean and variance, the routes and the
route counts, against both the CPU oracle and the reference's own kernels.
"""

import ctypes

import numpy as np
import pytest
import torch

import oracle_lib
from mmh3_b200 import attention, synthetic
from mmh3_b200.attention import SparseSinks

pytestmark = pytest.mark.gpu

SCALE = synthetic.softmax_scale()


def make_case(oracle, tokens, heads):
    """Every block of keys and queries shares a random direction (sparse_attention.rs:26-43)."""
    inner = heads * 128
    blocks = -(-tokens // 64)
    directions, state = oracle_lib.lcg(oracle, tokens, blocks * 3 * inner, -1.0, 1.0)
    noise, state = oracle_lib.lcg(oracle, state, tokens * 3 * inner, -1.0, 1.0)
    block_of = np.arange(tokens) // 64
    qkv = directions.reshape(blocks, 3 * inner)[block_of] + noise.reshape(tokens, 3 * inner)
    return synthetic.to_bf16_bits(qkv.reshape(-1)).reshape(tokens, 3, heads, 128)


def flat_sinks(sinks):
    return (*sinks.key_blocks, *sinks.query_blocks)


def assert_routes_equal(routes_a, counts_a, routes_b, counts_b):
    assert np.array_equal(counts_a, counts_b)
    heads, blocks = counts_a.shape
    for head in range(heads):
        for block in range(blocks):
            count = counts_a[head, block]
            assert np.array_equal(routes_a[head, block, :count], routes_b[head, block, :count]), (
                head, block)


def bits_equal(tensor, array):
    return np.array_equal(tensor.cpu().numpy().view(np.uint32),
                          np.ascontiguousarray(array).reshape(-1).view(np.uint32))


CASES = [
    (1000, 2, 0.5, SparseSinks((0, 2), (1, 2))),
    (777, 3, 1.3, SparseSinks((0, 1), (0, 0))),
]


@pytest.mark.parametrize("quantized", [False, True])
@pytest.mark.parametrize("tokens,heads,tau,sinks", CASES)
def test_matches_the_reference(oracle, reference_kernels, tokens, heads, tau, sinks, quantized):
    """sparse_attention.rs:170-215: both precisions against the same f64 reference and bounds."""
    bits = make_case(oracle, tokens, heads)
    inner = heads * 128
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.SparseWorkspace(tokens, heads, quantized=quantized)
    layout = attention.qkv_layout(heads)
    attention.sparse(qkv, output, layout, SCALE, tau, sinks, workspace)
    assert attention.take_status() == 0

    # Routing against the CPU restatement of the kernels' FP32 order: bit for bit where a route
    # depends on it, close where only the output does.
    work = oracle_lib.sol_route(oracle, bits, tokens, heads, tau, SCALE, flat_sinks(sinks))
    for name in ("centroids", "block_keys", "value_sums", "key_mean", "key_variance"):
        assert bits_equal(getattr(workspace, name), work[name]), name
    routes, counts = workspace.routes_host()
    assert_routes_equal(routes, counts, work["routes"], work["route_counts"])
    assert bits_equal(workspace.tail_max, work["tail_max"])
    for name in ("tail_sum", "tail_values", "row_offsets"):
        ours = getattr(workspace, name).cpu().numpy().reshape(work[name].shape)
        assert np.allclose(ours, work[name], rtol=1e-4, atol=1e-5), name

    # The reference's kernels on the same device buffers.
    theirs = attention.SparseWorkspace(tokens, heads, quantized=quantized)
    reference_output = torch.zeros_like(output)
    raw = theirs.raw()
    their_quantized = theirs.quantized.raw() if quantized else None
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_sparse_attention(
        base, base + 2 * inner, base + 4 * inner, reference_output.data_ptr(), tokens, heads,
        ctypes.byref(layout), SCALE, tau, *flat_sinks(sinks), ctypes.byref(raw),
        ctypes.byref(their_quantized) if quantized else None, 0, None) == 0
    torch.cuda.synchronize()
    assert_routes_equal(routes, counts, *theirs.routes_host())
    for name in ("centroids", "block_keys", "value_sums", "key_mean", "key_variance", "tail_max"):
        assert torch.equal(getattr(workspace, name), getattr(theirs, name)), name
    assert torch.allclose(workspace.tail_sum, theirs.tail_sum, rtol=1e-4, atol=1e-5)
    assert torch.allclose(workspace.tail_values, theirs.tail_values, rtol=1e-4, atol=1e-4)
    assert torch.allclose(workspace.row_offsets, theirs.row_offsets, rtol=1e-5, atol=1e-6)
    if quantized:
        # The quantizer's outputs are the dense path's: INT8 q, k, FP8 V and scales bit for bit.
        for name in ("query", "key", "value", "query_scales", "key_scales", "value_scales"):
            assert torch.equal(getattr(workspace.quantized, name),
                               getattr(theirs.quantized, name)), name

    # Outputs: the f64 reference with the reference test's bounds, then the reference's kernel.
    values = synthetic.bf16_bits_to_f32(bits)
    expected, expected_fraction = oracle_lib.sol_reference(
        oracle, values[:, 0], values[:, 1], values[:, 2], tau, SCALE, flat_sinks(sinks))
    fraction = workspace.routed_fraction()
    assert abs(fraction - expected_fraction) < 0.01
    assert 0.1 < fraction < 0.9
    actual = output.float().cpu().numpy()
    difference = np.linalg.norm((actual - expected).astype(np.float64))
    norm = np.linalg.norm(expected.astype(np.float64))
    assert difference / norm < 0.01
    assert np.max(np.abs(actual - expected)) < 0.05
    other = reference_output.float().cpu().numpy()
    assert np.max(np.abs(actual - other)) < 2e-2
    cosine = np.sum(actual.astype(np.float64) * other) / (
        np.linalg.norm(actual.astype(np.float64)) * np.linalg.norm(other.astype(np.float64)))
    assert cosine >= 0.9995


@pytest.mark.parametrize("tokens,heads", [(64 * 129 + 5, 2), (64 * 16 + 1, 1), (64 * 271, 1)])
def test_routes_where_the_passes_over_the_keys_end_raggedly(oracle, reference_kernels, tokens,
                                                            heads):
    """The routing kernel walks a head's key blocks 128 to a CTA pass and 16 to a warp, and a word
    of the mask of routed blocks is two warps' votes: 130 blocks (two in the second pass), 17 (one
    in the second warp's share), 271 (a last mask word of 15 bits). Routes, counts and the tails'
    maxima must be the CPU restatement's and the reference kernels' bits, the tails' sums close."""
    check_routing(oracle, reference_kernels, make_case(oracle, tokens, heads), tokens, heads)


def test_routes_of_a_sequence_too_long_for_eight_query_blocks_a_cta(oracle, reference_kernels):
    """Past 4,000 blocks the scores of eight query blocks no longer fit a CTA's shared memory and
    the routing kernel takes four to a CTA (the reference halves its own count the same way,
    sparse_attention.cu:289-315): 4,100 blocks and a partial one, same bits."""
    tokens, heads = 64 * 4100 + 3, 1
    qkv = synthetic.dense_qkv(tokens, heads, seed=9)
    bits = qkv.view(torch.int16).numpy().view(np.uint16).reshape(tokens, 3, heads, 128)
    check_routing(oracle, reference_kernels, bits, tokens, heads)


def check_routing(oracle, reference_kernels, bits, tokens, heads):
    tau, sinks = 1.0, SparseSinks((0, 2), (0, 0))
    inner = heads * 128
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.SparseWorkspace(tokens, heads)
    layout = attention.qkv_layout(heads)
    attention.sparse(qkv, output, layout, SCALE, tau, sinks, workspace)
    assert attention.take_status() == 0
    work = oracle_lib.sol_route(oracle, bits, tokens, heads, tau, SCALE, flat_sinks(sinks))
    routes, counts = workspace.routes_host()
    assert_routes_equal(routes, counts, work["routes"], work["route_counts"])
    assert bits_equal(workspace.tail_max, work["tail_max"])
    # The tails are FP32 sums over hundreds of blocks in an order of the kernel's own: held to 1e-6
    # of the largest sum where the terms cancel, to 1e-4 of the value elsewhere.
    for name in ("tail_sum", "tail_values"):
        ours = getattr(workspace, name).cpu().numpy().reshape(work[name].shape)
        slack = 1e-6 * float(np.abs(work[name]).max())
        assert np.allclose(ours, work[name], rtol=1e-4, atol=slack), name
    assert 0.02 < workspace.routed_fraction() < 0.9

    theirs = attention.SparseWorkspace(tokens, heads)
    reference_output = torch.zeros_like(output)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_sparse_attention(
        base, base + 2 * inner, base + 4 * inner, reference_output.data_ptr(), tokens, heads,
        ctypes.byref(layout), SCALE, tau, *flat_sinks(sinks), ctypes.byref(raw), None, 0,
        None) == 0
    torch.cuda.synchronize()
    assert_routes_equal(routes, counts, *theirs.routes_host())
    assert torch.equal(workspace.tail_max, theirs.tail_max)
    assert torch.allclose(workspace.tail_sum, theirs.tail_sum, rtol=1e-4, atol=1e-5)
    assert torch.allclose(workspace.tail_values, theirs.tail_values, rtol=1e-4,
                          atol=1e-6 * float(theirs.tail_values.abs().max()))
    assert torch.max(torch.abs(output.float() - reference_output.float())).item() < 2e-2


def test_routing_everything_is_dense_attention():
    """With a threshold no score fails, every block is exact, the tails are empty, and the result
    is the dense kernel's (sparse.rs:240-277 on the GPU)."""
    tokens, heads = 64 * 5 + 17, 2
    qkv = synthetic.dense_qkv(tokens, heads, seed=5).cuda()
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    dense = torch.zeros_like(output)
    workspace = attention.SparseWorkspace(tokens, heads)
    attention.sparse(qkv, output, attention.qkv_layout(heads), SCALE, -1e30, SparseSinks(),
                     workspace)
    attention.dense_bf16(qkv, dense, tokens, heads, SCALE)
    assert attention.take_status() == 0
    assert workspace.routed_fraction() == 1.0
    assert (workspace.tail_sum == 0).all()
    assert torch.max(torch.abs(output.float() - dense.float())).item() < 2e-2


@pytest.mark.parametrize("quantized", [False, True])
@pytest.mark.parametrize("tokens", [1, 63, 64, 65, 200, 1000])
def test_prepared_inputs_match_separate_passes(oracle, tokens, quantized):
    """attention_inputs.rs:126-256 (sparse_attention_with_prepared_inputs_matches_separate_passes):
    the fused input pass fills the block statistics (and the INT8/FP8 workspace), and Sol-Attn over
    prepared inputs gives the output, bit for bit, of qk_norm_rope followed by Sol-Attn over the
    normalized rows; so does the pass that also takes the head maxima of |v|."""
    from test_inputs_gpu import make_inputs, norm_for

    heads, tau = 3, 1.0
    inner = heads * 128
    sinks = SparseSinks((0, 1), (0, 0))
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads)
    norm = norm_for(query_weight, key_weight, angles)
    layout = attention.qkv_layout(heads)

    separate = synthetic.bf16_tensor(bits, "cuda")
    separate_workspace = attention.SparseWorkspace(tokens, heads, quantized=quantized)
    separate_output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.qk_norm_rope(separate, norm, tokens, heads)
    attention.sparse(separate, separate_output, layout, SCALE, tau, sinks, separate_workspace)

    fused = synthetic.bf16_tensor(bits, "cuda")
    fused_workspace = attention.SparseWorkspace(tokens, heads, quantized=quantized)
    fused_output = torch.zeros_like(separate_output)
    attention.prepare_inputs(fused, norm, tokens, heads, sol=fused_workspace)
    attention.sparse(fused, fused_output, layout, SCALE, tau, sinks, fused_workspace,
                     attention.AttentionInputs.PREPARED)

    if quantized:
        with_values = synthetic.bf16_tensor(bits, "cuda")
        workspace = attention.SparseWorkspace(tokens, heads, quantized=True)
        with_values_output = torch.zeros_like(separate_output)
        maxima = with_values[:, 2].float().abs().amax(dim=(0, 2)).contiguous()
        attention.prepare_inputs(with_values, norm, tokens, heads, sol=workspace,
                                 value_head_maxima=maxima)
        attention.sparse(with_values, with_values_output, layout, SCALE, tau, sinks, workspace,
                         attention.AttentionInputs.PREPARED_WITH_VALUES)
        assert torch.equal(separate_output, with_values_output)
    assert attention.take_status() == 0

    assert separate_workspace.routed_fraction() == fused_workspace.routed_fraction()
    assert_routes_equal(*separate_workspace.routes_host(), *fused_workspace.routes_host())
    assert torch.equal(separate_output, fused_output)
    # Quantized attention reads only INT8 keys, so the fused pass leaves k as it was.
    normalized = 1 if quantized else 2
    assert torch.equal(separate[:, :normalized], fused[:, :normalized])


@pytest.mark.parametrize("quantized", [False, True])
def test_a_layout_off_the_tma_grid_gives_the_same_bits(oracle, quantized):
    """q, k and v two bytes off a 16-byte boundary with an odd token stride: the entry point
    gathers them into dense arrays first (the reference copies with cp.async instead of TMA,
    crates/mmh3-cuda/kernels/attention.cu:386-418), and routes, statistics and output must be
    the bits of the aligned layout."""
    tokens, heads, tau, sinks = CASES[0]
    inner = heads * 128
    qkv = synthetic.bf16_tensor(make_case(oracle, tokens, heads), "cuda")
    results = []
    for shifted in (False, True):
        token_stride = 3 * inner + (1 if shifted else 0)
        offset = 1 if shifted else 0
        storage = torch.zeros(tokens * token_stride + 8, dtype=torch.bfloat16, device="cuda")
        torch.as_strided(storage, (tokens, 3 * inner), (token_stride, 1), offset).copy_(
            qkv.view(tokens, 3 * inner))
        layout = attention.make_layout((token_stride,) * 3 + (inner,))
        output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
        workspace = attention.SparseWorkspace(tokens, heads, quantized=quantized)
        attention.sparse(storage, output, layout, SCALE, tau, sinks, workspace,
                         offsets=(offset, offset + inner, offset + 2 * inner, 0))
        assert attention.take_status() == 0
        results.append((output, workspace))
    (aligned, first), (moved, second) = results
    assert_routes_equal(*first.routes_host(), *second.routes_host())
    for name in ("centroids", "block_keys", "value_sums", "tail_max", "tail_sum", "tail_values",
                 "row_offsets"):
        assert torch.equal(getattr(first, name), getattr(second, name)), name
    assert torch.equal(aligned.view(torch.int16), moved.view(torch.int16))


def test_rejects_what_it_does_not_compute():
    tokens, heads = 128, 1
    qkv = synthetic.dense_qkv(tokens, heads, seed=1).cuda()
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.SparseWorkspace(tokens, heads)
    layout = attention.qkv_layout(heads)
    with pytest.raises(attention.CudaError) as raised:
        attention.sparse(qkv, output, layout, -1.0, 0.5, SparseSinks(), workspace)
    assert raised.value.code == 1  # cudaErrorInvalidValue
    from mmh3_b200 import _lib

    raw = workspace.raw()
    base = qkv.data_ptr()
    code = _lib.library().mmh3_sparse_attention(
        base, base + 256, base + 512, output.data_ptr(), 0, heads, ctypes.byref(layout), SCALE,
        0.5, 0, 0, 0, 0, ctypes.byref(raw), None, 0, None)
    assert code == 1
