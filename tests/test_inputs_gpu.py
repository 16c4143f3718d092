"""Bit-exact parity of the passes that prepare the attention's inputs, on a B200.

INT8 q and k, their scales, the |v| maxima, FP8 V and its scales, the normalized BF16 rows and
VSA's pooled tiles must equal, in every bit, what the reference's kernels leave in the same
workspaces (crates/mmh3-cuda/tests/attention_inputs.rs asserts the same identity between the
reference's fused and separate passes). The reference side is its own CUDA code compiled from its
sources (oracle/_ref); the CPU oracle checks the parts that do not depend on device libm.
"""

import ctypes

import numpy as np
import pytest
import torch

import oracle_lib
from mmh3_b200 import _lib, attention, synthetic
from mmh3_b200.vsa import PackedLayout, VsaPlan

pytestmark = pytest.mark.gpu

PAIRS = 48
EPSILON = 1e-6
SCALE = synthetic.softmax_scale()


def make_inputs(oracle, tokens, heads, pairs=PAIRS):
    """Blocks of tokens share a direction (attention_inputs.rs:51-98)."""
    inner = heads * 128
    state = tokens * 31 + heads
    blocks = -(-tokens // 64)
    directions, state = oracle_lib.lcg(oracle, state, blocks * 3 * inner, -2.0, 2.0)
    noise, state = oracle_lib.lcg(oracle, state, tokens * 3 * inner, -1.0, 1.0)
    index = np.arange(tokens * 3 * inner)
    qkv = directions[(index // (3 * inner) // 64) * 3 * inner + index % (3 * inner)] + noise
    query_weight, state = oracle_lib.lcg(oracle, state, 128, 0.5, 1.5)
    key_weight, state = oracle_lib.lcg(oracle, state, 128, 0.5, 1.5)
    angles, state = oracle_lib.lcg(oracle, state, tokens * pairs, -40.0, 40.0)
    return (synthetic.to_bf16_bits(qkv.astype(np.float32)).reshape(tokens, 3, heads, 128),
            synthetic.to_bf16_bits(query_weight), synthetic.to_bf16_bits(key_weight), angles)


def norm_for(query_weight, key_weight, angles, pairs=PAIRS):
    return attention.HeadNorm(synthetic.bf16_tensor(query_weight, "cuda"),
                              synthetic.bf16_tensor(key_weight, "cuda"),
                              torch.from_numpy(angles).cuda() if angles is not None else None,
                              pairs if angles is not None else 0, EPSILON)


def valid_value_columns(workspace, lengths):
    """FP8 V as [heads, 128, blocks, 64]."""
    return workspace.value.cpu().numpy().reshape(workspace.heads, 128, workspace.blocks, 64)


def assert_workspaces_equal(ours, theirs, values=True, maxima=True):
    for name in ("query", "key", "query_scales", "key_scales"):
        a, b = getattr(ours, name).cpu().numpy(), getattr(theirs, name).cpu().numpy()
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), name
    if maxima:
        assert np.array_equal(ours.value_maxima.cpu().numpy().view(np.uint32),
                              theirs.value_maxima.cpu().numpy().view(np.uint32))
    if values:
        assert np.array_equal(ours.value_scales.cpu().numpy().view(np.uint32),
                              theirs.value_scales.cpu().numpy().view(np.uint32))
        assert np.array_equal(ours.value.cpu().numpy(), theirs.value.cpu().numpy())


def fill(workspace, byte):
    for name in ("query", "key", "value"):
        getattr(workspace, name).fill_(byte)
    for name in ("query_scales", "key_scales", "value_scales", "value_maxima"):
        getattr(workspace, name).fill_(-1.0)


@pytest.mark.parametrize("tokens", [1, 63, 64, 65, 127, 129, 200, 1000])
def test_raw_quantization_is_bit_exact(oracle, reference_kernels, tokens):
    """mmh3_attention_quantized with inputs_ready = 0 prepares the whole workspace itself."""
    heads = 3
    inner = heads * 128
    bits, _, _, _ = make_inputs(oracle, tokens, heads)
    # Per-head value magnitudes, as quantized_attention.rs:33-44 spreads them.
    values = synthetic.bf16_bits_to_f32(bits).copy()
    for head in range(heads):
        values[:, 2, head] *= 2.0 ** ((head - 1) * 3)
    bits = synthetic.to_bf16_bits(values.reshape(-1)).reshape(tokens, 3, heads, 128)
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    ours = attention.QuantizedWorkspace(tokens, heads)
    theirs = attention.QuantizedWorkspace(tokens, heads)
    fill(ours, 0x55)
    fill(theirs, 0x55)
    attention.dense_quantized(qkv, output, SCALE, ours, attention.AttentionInputs.RAW)
    layout = attention.qkv_layout(heads)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_attention_quantized(
        base, base + 2 * inner, base + 4 * inner, output.data_ptr(), tokens, heads,
        ctypes.byref(layout), SCALE, None, ctypes.byref(raw), 0, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert_workspaces_equal(ours, theirs)

    # The CPU restatement of the quantizer agrees too.
    blocks = ours.blocks
    flat = np.ascontiguousarray(bits.reshape(-1))
    for part, name in ((0, "query"), (1, "key")):
        quantized = np.full(tokens * inner, 0x55, dtype=np.int8)
        scales = np.empty(heads * blocks, dtype=np.float32)
        oracle.oracle_quantize_rows(ctypes.c_void_p(flat.ctypes.data + part * inner * 2),
                                    3 * inner, 128, tokens, heads, None, None, 0,
                                    oracle_lib.ptr(quantized), oracle_lib.ptr(scales))
        assert np.array_equal(quantized.view(np.uint8), getattr(ours, name).cpu().numpy())
        assert np.array_equal(scales.view(np.uint32),
                              getattr(ours, name + "_scales").cpu().numpy().view(np.uint32))
    value8 = np.empty(heads * 128 * blocks * 64, dtype=np.uint8)
    value_scales = np.empty(heads, dtype=np.float32)
    value_maxima = np.empty(heads * blocks, dtype=np.float32)
    oracle.oracle_quantize_value(ctypes.c_void_p(flat.ctypes.data + 2 * inner * 2), 3 * inner, 128,
                                 tokens, heads, None, None, 0, oracle_lib.ptr(value8),
                                 oracle_lib.ptr(value_scales), oracle_lib.ptr(value_maxima))
    assert np.array_equal(value8, ours.value.cpu().numpy())
    assert np.array_equal(value_scales.view(np.uint32),
                          ours.value_scales.cpu().numpy().view(np.uint32))
    assert np.array_equal(value_maxima.view(np.uint32),
                          ours.value_maxima.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("tokens", [1, 63, 64, 65, 200, 1000])
@pytest.mark.parametrize("rotate", [True, False])
def test_norm_and_rope_in_place_is_bit_exact(oracle, reference_kernels, tokens, rotate):
    heads = 2
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads)
    norm = norm_for(query_weight, key_weight, angles if rotate else None)
    ours = synthetic.bf16_tensor(bits, "cuda")
    theirs = ours.clone()
    attention.qk_norm_rope(ours, norm, tokens, heads)
    assert reference_kernels.mmh3_qk_norm_rope(
        theirs.data_ptr(), norm.query_weight.data_ptr(), norm.key_weight.data_ptr(),
        norm.angles.data_ptr() if rotate else None, norm.pairs, tokens, heads, heads, EPSILON,
        None) == 0
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16))
    # v is left alone
    assert torch.equal(ours.view(torch.int16)[:, 2].cpu(),
                       synthetic.bf16_tensor(bits).view(torch.int16)[:, 2])


# Multiples of 16 keep both dimensions of a rotary pair in one thread, each with its own unrolled
# turn; every other count crosses threads through shared memory.
@pytest.mark.parametrize("pairs", [16, 32, 64, 1, 7, 20, 40, 63])
@pytest.mark.parametrize("tokens", [65, 200])
def test_rope_with_other_pair_counts_is_bit_exact(oracle, reference_kernels, tokens, pairs):
    heads = 3
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads, pairs)
    norm = norm_for(query_weight, key_weight, angles, pairs)
    ours = synthetic.bf16_tensor(bits, "cuda")
    theirs = ours.clone()
    attention.qk_norm_rope(ours, norm, tokens, heads)
    assert reference_kernels.mmh3_qk_norm_rope(
        theirs.data_ptr(), norm.query_weight.data_ptr(), norm.key_weight.data_ptr(),
        norm.angles.data_ptr(), pairs, tokens, heads, heads, EPSILON, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16))
    # ... and through the fused preparation, whose INT8 rows come from the rotated values.
    ours_qkv = synthetic.bf16_tensor(bits, "cuda")
    theirs_qkv = ours_qkv.clone()
    ours_space = attention.QuantizedWorkspace(tokens, heads)
    theirs_space = attention.QuantizedWorkspace(tokens, heads)
    attention.prepare_inputs(ours_qkv, norm, tokens, heads, quantized=ours_space)
    raw = theirs_space.raw()
    assert reference_kernels.mmh3_attention_inputs(
        theirs_qkv.data_ptr(), norm.query_weight.data_ptr(), norm.key_weight.data_ptr(),
        norm.angles.data_ptr(), pairs, tokens, heads, EPSILON, None, ctypes.byref(raw), None,
        None, 0, None, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert_workspaces_equal(ours_space, theirs_space, values=False)


@pytest.mark.parametrize("tokens", [1, 63, 64, 65, 200, 1000])
@pytest.mark.parametrize("with_values", [False, True])
def test_fused_dense_preparation_is_bit_exact(oracle, reference_kernels, tokens, with_values):
    """mmh3_attention_inputs for dense INT8/FP8 attention: norm, RoPE, INT8 q and k, and either
    the |v| block maxima or, given the per-head maxima, FP8 V."""
    heads = 3
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads)
    norm = norm_for(query_weight, key_weight, angles)
    ours_qkv = synthetic.bf16_tensor(bits, "cuda")
    theirs_qkv = ours_qkv.clone()
    ours = attention.QuantizedWorkspace(tokens, heads)
    theirs = attention.QuantizedWorkspace(tokens, heads)
    fill(ours, 0x33)
    fill(theirs, 0x33)
    maxima = None
    if with_values:
        maxima = ours_qkv[:, 2].float().abs().amax(dim=(0, 2)).contiguous()
    attention.prepare_inputs(ours_qkv, norm, tokens, heads, quantized=ours,
                             value_head_maxima=maxima)
    raw = theirs.raw()
    assert reference_kernels.mmh3_attention_inputs(
        theirs_qkv.data_ptr(), norm.query_weight.data_ptr(), norm.key_weight.data_ptr(),
        norm.angles.data_ptr(), norm.pairs, tokens, heads, EPSILON, None, ctypes.byref(raw), None,
        None, 0, maxima.data_ptr() if with_values else None, None) == 0
    torch.cuda.synchronize()
    assert_workspaces_equal(ours, theirs, values=with_values, maxima=not with_values)
    assert torch.equal(ours_qkv.view(torch.int16), theirs_qkv.view(torch.int16))


@pytest.mark.parametrize("quantized", [False, True])
def test_fused_vsa_preparation_is_bit_exact(oracle, reference_kernels, quantized):
    """mmh3_attention_inputs over VSA tiles: pooled tiles, and INT8/FP8 per tile."""
    layout = PackedLayout.text_to_video(70, 9, 16, 24, 40)
    plan = VsaPlan.for_layout(layout)
    tokens, heads = len(layout), 2
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads)
    norm = norm_for(query_weight, key_weight, angles)
    ours_qkv = synthetic.bf16_tensor(bits, "cuda")
    theirs_qkv = ours_qkv.clone()
    ours = attention.VsaWorkspace(plan, tokens, heads, quantized=quantized)
    theirs = attention.VsaWorkspace(plan, tokens, heads, quantized=quantized)
    maxima = None
    if quantized:
        fill(ours.quantized, 0x11)
        fill(theirs.quantized, 0x11)
        maxima = ours_qkv[:, 2].float().abs().amax(dim=(0, 2)).contiguous()
    attention.prepare_inputs(ours_qkv, norm, tokens, heads, vsa=ours, value_head_maxima=maxima)
    sparse = theirs.sparse_raw()
    raw = theirs.quantized.raw() if quantized else None
    assert reference_kernels.mmh3_attention_inputs(
        theirs_qkv.data_ptr(), norm.query_weight.data_ptr(), norm.key_weight.data_ptr(),
        norm.angles.data_ptr(), norm.pairs, tokens, heads, EPSILON, ctypes.byref(sparse),
        ctypes.byref(raw) if quantized else None, theirs.tile_starts.data_ptr(),
        theirs.tile_lengths.data_ptr(), theirs.tiles, maxima.data_ptr() if quantized else None,
        None) == 0
    torch.cuda.synchronize()
    for name in ("pooled_query", "pooled_key", "pooled_value"):
        assert torch.equal(getattr(ours, name).view(torch.int32),
                           getattr(theirs, name).view(torch.int32)), name
    if quantized:
        assert_workspaces_equal(ours.quantized, theirs.quantized, values=True, maxima=False)
    assert torch.equal(ours_qkv.view(torch.int16), theirs_qkv.view(torch.int16))


def test_fused_pass_agrees_with_separate_passes(oracle):
    """attention_inputs.rs:252-419: the fused pass changes nothing against qk_norm_rope followed by
    the attention's own preparation."""
    tokens, heads = 200, 3
    bits, query_weight, key_weight, angles = make_inputs(oracle, tokens, heads)
    norm = norm_for(query_weight, key_weight, angles)
    fused_qkv = synthetic.bf16_tensor(bits, "cuda")
    separate_qkv = fused_qkv.clone()
    fused = attention.QuantizedWorkspace(tokens, heads)
    separate = attention.QuantizedWorkspace(tokens, heads)
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.prepare_inputs(fused_qkv, norm, tokens, heads, quantized=fused)
    attention.dense_quantized(fused_qkv, output, SCALE, fused, attention.AttentionInputs.PREPARED)
    attention.qk_norm_rope(separate_qkv, norm, tokens, heads)
    attention.dense_quantized(separate_qkv, output, SCALE, separate, attention.AttentionInputs.RAW)
    assert attention.take_status() == 0
    assert_workspaces_equal(fused, separate)


def test_quantization_is_bit_exact_over_many_scales(oracle, reference_kernels):
    """Many blocks whose magnitudes span forty binades, so that the per-block scales take many
    different significands: the quotients must still round exactly as the reference's divisions."""
    tokens, heads = 8192, 4
    inner = heads * 128
    generator = torch.Generator().manual_seed(77)
    values = torch.randn((tokens, 3, heads, 128), generator=generator)
    binades = torch.randint(-20, 21, (tokens // 64, 1, 3, heads, 1), generator=generator).float()
    values = (values.view(tokens // 64, 64, 3, heads, 128) * torch.exp2(binades)).view(
        tokens, 3, heads, 128)
    qkv = values.bfloat16().cuda()
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    ours = attention.QuantizedWorkspace(tokens, heads)
    theirs = attention.QuantizedWorkspace(tokens, heads)
    attention.dense_quantized(qkv, output, SCALE, ours, attention.AttentionInputs.RAW)
    layout = attention.qkv_layout(heads)
    raw = theirs.raw()
    base = qkv.data_ptr()
    assert reference_kernels.mmh3_attention_quantized(
        base, base + 2 * inner, base + 4 * inner, output.data_ptr(), tokens, heads,
        ctypes.byref(layout), SCALE, None, ctypes.byref(raw), 0, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert_workspaces_equal(ours, theirs)
