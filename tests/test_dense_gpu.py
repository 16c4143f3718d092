"""Parity of the dense BF16 attention kernel, through the C ABI, on a B200.

Mirrors crates/mmh3-cuda/tests/attention.rs: the same generator, seeds, shapes and tolerance against
an f64 softmax attention, plus ragged sizes around the kernel's 128/256-row tiles, the benchmark's
value distribution, and the reference's own CUDA kernel on the same device buffers.
"""

import ctypes

import numpy as np
import pytest
import torch

import oracle_lib
from mmh3_b200 import _lib, attention, synthetic

pytestmark = pytest.mark.gpu

SCALE = synthetic.softmax_scale()


def lcg_qkv(oracle, tokens, heads, seed):
    values, _ = oracle_lib.lcg(oracle, seed, tokens * 3 * heads * 128, -2.0, 2.0)
    return synthetic.to_bf16_bits(values).reshape(tokens, 3, heads, 128)


def run_dense(bits, tokens, heads):
    qkv = synthetic.bf16_tensor(bits, "cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.dense_bf16(qkv, output, tokens, heads, SCALE)
    assert attention.take_status() == 0
    return output.float().cpu().numpy()


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def load_selftest():
    library = ctypes.CDLL(str(_lib.SELFTEST_LIBRARY))
    library.mmh3_b200_umma_selftest.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 6
    library.mmh3_b200_umma_selftest.restype = ctypes.c_int
    return library


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    """Failure detection without a fault: every wait in the kernels is bounded; one that runs out
    (here: on a barrier nothing completes) leaves its code in the status word, the kernel returns,
    take_status reads and clears the word, and the next launch on the same context works."""
    library = load_selftest()
    library.mmh3_b200_expired_wait_selftest.argtypes = [ctypes.c_uint]
    library.mmh3_b200_expired_wait_selftest.restype = ctypes.c_int
    library.mmh3_b200_take_status.restype = ctypes.c_int
    code = 0x00770001
    assert library.mmh3_b200_take_status() == 0
    assert library.mmh3_b200_expired_wait_selftest(code) == 64  # every thread gave up
    assert library.mmh3_b200_take_status() == code
    assert library.mmh3_b200_take_status() == 0
    test_umma_bf16_building_blocks()
    tokens, heads = 300, 2
    bits = synthetic.dense_qkv(tokens, heads, seed=3).view(torch.int16).numpy().view(np.uint16)
    run_dense(bits, tokens, heads)
    assert attention.take_status() == 0


def test_umma_bf16_building_blocks():
    """scores = A.B^T from shared memory and output = P.V with P in tensor memory, BF16."""
    library = load_selftest()
    generator = torch.Generator().manual_seed(11)
    a = torch.randn((128, 128), generator=generator).bfloat16().cuda()
    b = torch.randn((128, 128), generator=generator).bfloat16().cuda()
    v = torch.randn((128, 128), generator=generator).bfloat16().cuda()
    p = torch.rand((128, 128), generator=generator).bfloat16().cuda()
    scores = torch.zeros((128, 128), dtype=torch.float32, device="cuda")
    output = torch.zeros((128, 128), dtype=torch.float32, device="cuda")
    code = library.mmh3_b200_umma_selftest(0, a.data_ptr(), b.data_ptr(), v.data_ptr(),
                                           p.data_ptr(), scores.data_ptr(), output.data_ptr())
    assert code == 0
    assert attention.take_status() == 0
    expected_scores = a.float().cpu() @ b.float().cpu().t()
    expected_output = p.float().cpu() @ v.float().cpu()
    assert torch.allclose(scores.cpu(), expected_scores, atol=1e-3, rtol=1e-4)
    assert torch.allclose(output.cpu(), expected_output, atol=1e-3, rtol=1e-4)


def test_umma_int8_fp8_building_blocks(oracle):
    """INT8 A.B^T with INT32 accumulators (exact) and E4M3 P.V^T with P in tensor memory."""
    library = load_selftest()
    rng = np.random.default_rng(12)
    a = rng.integers(-127, 128, size=(128, 128), dtype=np.int8)
    b = rng.integers(-127, 128, size=(128, 128), dtype=np.int8)
    p = rng.integers(0, 0x7F, size=(128, 128), dtype=np.uint8)  # positive finite E4M3
    v = rng.integers(0, 0x7F, size=(128, 128), dtype=np.uint8)
    v |= (rng.integers(0, 2, size=(128, 128), dtype=np.uint8) << 7)
    table = np.array([oracle.oracle_e4m3_to_f32(code) for code in range(256)], dtype=np.float64)
    device = [torch.from_numpy(x.view(np.uint8).copy()).cuda() for x in (a, b, v, p)]
    scores = torch.zeros((128, 128), dtype=torch.int32, device="cuda")
    output = torch.zeros((128, 128), dtype=torch.float32, device="cuda")
    code = library.mmh3_b200_umma_selftest(1, *(x.data_ptr() for x in device), scores.data_ptr(),
                                           output.data_ptr())
    assert code == 0
    assert attention.take_status() == 0
    expected_scores = a.astype(np.int32) @ b.astype(np.int32).T
    assert np.array_equal(scores.cpu().numpy(), expected_scores)
    # v is V^T [dims][keys]: output[m][d] = sum_k p[m][k] v[d][k]
    expected_output = table[p] @ table[v].T
    assert np.allclose(output.cpu().numpy(), expected_output, rtol=2e-3, atol=1e-2)


@pytest.mark.parametrize("tokens,heads", [(1, 1), (64, 2), (200, 3)])
def test_matches_cpu_reference(oracle, tokens, heads):
    """attention.rs:27-90: LCG data uniform in [-2, 2), seed tokens * 31 + heads."""
    bits = lcg_qkv(oracle, tokens, heads, tokens * 31 + heads)
    actual = run_dense(bits, tokens, heads)
    expected = oracle_lib.attention_bf16(oracle, bits, tokens, heads, SCALE)
    assert np.all(np.abs(actual - expected) <= 0.02 + 0.01 * np.abs(expected))


@pytest.mark.parametrize("tokens", [127, 128, 129, 255, 256, 257, 384, 1000])
def test_ragged_sizes(oracle, tokens):
    heads = 2
    bits = synthetic.dense_qkv(tokens, heads, seed=tokens).view(torch.int16).numpy().view(np.uint16)
    actual = run_dense(bits, tokens, heads)
    expected = oracle_lib.attention_bf16(oracle, bits, tokens, heads, SCALE)
    assert np.max(np.abs(actual - expected)) <= 2e-2
    assert cosine(actual, expected) >= 0.9995


def test_cpu_workload_sampled(oracle):
    """B=1, H=8, L=4096 with the benchmark's distribution, every 29th query row on the CPU."""
    tokens, heads = synthetic.CONFIGS["C0"]
    bits = synthetic.dense_qkv(tokens, heads, seed=0).view(torch.int16).numpy().view(np.uint16)
    actual = run_dense(bits, tokens, heads)
    rows = list(range(0, tokens, 29))
    for row in rows:
        expected = oracle_lib.attention_bf16(oracle, bits, tokens, heads, SCALE, row, row + 1)
        assert np.max(np.abs(actual[row] - expected[0])) <= 2e-2
    expected = np.concatenate([
        oracle_lib.attention_bf16(oracle, bits, tokens, heads, SCALE, row, row + 1) for row in rows[:32]
    ])
    assert cosine(actual[rows[:32]], expected) >= 0.9995


def test_agrees_with_the_reference_kernel(reference_kernels):
    """The reference's mma.sync kernel and this one on the same device buffers."""
    tokens, heads = 1000, 3
    inner = heads * 128
    qkv = synthetic.dense_qkv(tokens, heads, seed=5).cuda()
    ours = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    attention.dense_bf16(qkv, ours, tokens, heads, SCALE)
    base = qkv.data_ptr()
    code = reference_kernels.mmh3_attention_bf16(base, base + 2 * inner, base + 4 * inner,
                                                 theirs.data_ptr(), tokens, heads, 3 * inner,
                                                 3 * inner, 3 * inner, inner, SCALE, None)
    assert code == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    a, b = ours.float().cpu().numpy(), theirs.float().cpu().numpy()
    assert np.max(np.abs(a - b)) <= 2e-2
    assert cosine(a, b) >= 0.9995


def test_grouped_heads_and_batches(oracle):
    """mmh3_attention with two query heads per key/value head and a batch of two."""
    tokens, heads, group, batch = 130, 4, 2, 2
    generator = torch.Generator().manual_seed(3)
    q = torch.randn((batch, tokens, heads, 128), generator=generator).bfloat16()
    k = torch.randn((batch, tokens, heads // group, 128), generator=generator).bfloat16()
    v = torch.randn((batch, tokens, heads // group, 128), generator=generator).bfloat16()
    output = torch.zeros((batch, tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    kv_inner = heads // group * 128
    layout = attention.make_layout(
        (heads * 128, kv_inner, kv_inner, heads * 128),
        batch_stride=(tokens * heads * 128, tokens * kv_inner, tokens * kv_inner,
                      tokens * heads * 128),
        heads_per_key_value=group)
    attention.attention(0, 128, q.cuda(), k.cuda(), v.cuda(), output, tokens, heads, batch, layout,
                        SCALE)
    assert attention.take_status() == 0
    scores = torch.einsum("bqhd,bkhd->bhqk", q.double(),
                          k.double().repeat_interleave(group, dim=2)) * SCALE
    expected = torch.einsum("bhqk,bkhd->bqhd", scores.softmax(-1),
                            v.double().repeat_interleave(group, dim=2))
    assert torch.max(torch.abs(output.cpu().double() - expected)) <= 2e-2


def reference_attention(q, k, v, group, causal):
    """softmax(q k^T * scale) v in float64 with torch, [batch, tokens, heads, 128] operands."""
    keys = k.double().repeat_interleave(group, dim=2)
    values = v.double().repeat_interleave(group, dim=2)
    scores = torch.einsum("bqhd,bkhd->bhqk", q.double(), keys) * SCALE
    if causal:
        tokens = q.shape[1]
        future = torch.triu(torch.ones((tokens, tokens), dtype=torch.bool), diagonal=1)
        scores = scores.masked_fill(future, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", scores.softmax(-1), values)


@pytest.mark.parametrize("element_type", [0, 1])
@pytest.mark.parametrize("tokens,causal", [(77, 1), (256, 1), (700, 1), (1000, 0), (513, 1)])
def test_causal_and_fp16_variants(reference_kernels, element_type, tokens, causal):
    """The other users of mmh3_attention at heads of 128 (crates/mmh3-cuda/kernels/attention.cu:
    502-536): the text encoder's causal attention with grouped key/value heads
    (src/text_encoder.rs:653-666), in BF16 and in FP16, against float64 and against the reference's
    kernel on the same buffers."""
    heads, group, batch = 4, 2, 2
    dtype = torch.float16 if element_type == 1 else torch.bfloat16
    generator = torch.Generator().manual_seed(tokens + element_type)
    q = torch.randn((batch, tokens, heads, 128), generator=generator).to(dtype)
    k = torch.randn((batch, tokens, heads // group, 128), generator=generator).to(dtype)
    v = torch.randn((batch, tokens, heads // group, 128), generator=generator).to(dtype)
    kv_inner = heads // group * 128
    layout = attention.make_layout(
        (heads * 128, kv_inner, kv_inner, heads * 128),
        batch_stride=(tokens * heads * 128, tokens * kv_inner, tokens * kv_inner,
                      tokens * heads * 128),
        heads_per_key_value=group, causal=causal)
    device = [tensor.cuda() for tensor in (q, k, v)]
    ours = torch.zeros((batch, tokens, heads, 128), dtype=dtype, device="cuda")
    theirs = torch.zeros_like(ours)
    attention.attention(element_type, 128, *device, ours, tokens, heads, batch, layout, SCALE)
    assert reference_kernels.mmh3_attention(
        element_type, 128, *(tensor.data_ptr() for tensor in device), theirs.data_ptr(), tokens,
        heads, batch, ctypes.byref(layout), SCALE, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    expected = reference_attention(q, k, v, group, causal)
    assert torch.max(torch.abs(ours.cpu().double() - expected)) <= 2e-2
    a, b = ours.float().cpu().numpy(), theirs.float().cpu().numpy()
    assert np.max(np.abs(a - b)) <= 2e-2
    assert cosine(a, b) >= 0.9995


def normalized_rotated(q, angles, pairs, epsilon, dtype):
    """The query after the fused RMS norm and RoPE, rounded to the element type as the kernel
    rounds it (crates/mmh3-cuda/kernels/attention.cu:62-111)."""
    values = q.double()
    values = values * torch.rsqrt(values.pow(2).mean(dim=-1, keepdim=True) + epsilon)
    first, second = values[..., :pairs], values[..., pairs:2 * pairs]
    cosine = torch.cos(angles.double())[None, :, None, :]
    sine = torch.sin(angles.double())[None, :, None, :]
    rotated = values.clone()
    rotated[..., :pairs] = first * cosine - second * sine
    rotated[..., pairs:2 * pairs] = first * sine + second * cosine
    return rotated.to(dtype)


@pytest.mark.parametrize("element_type", [0, 1])
@pytest.mark.parametrize("head_dim,tokens,causal,pairs", [
    (64, 300, 0, None), (64, 513, 1, None), (64, 700, 0, 32), (64, 129, 0, 20),
    (128, 300, 0, 64), (128, 257, 1, 40),
])
def test_heads_of_64_and_the_fused_query_rope(reference_kernels, element_type, head_dim, tokens,
                                              causal, pairs):
    """The VAE decoder's use of mmh3_attention_roped (src/vae.rs:1008): FP16 heads of 64 in a
    batched layout with the query's RMS norm and RoPE inside the attention; and the same options in
    every other combination the reference's kernel takes, against float64 and against that kernel
    on the same buffers."""
    heads, batch, epsilon = 3, 2, 1e-6
    scale = 1.0 / head_dim ** 0.5
    dtype = torch.float16 if element_type == 1 else torch.bfloat16
    generator = torch.Generator().manual_seed(tokens + head_dim + element_type)
    q, k, v = (torch.randn((batch, tokens, heads, head_dim), generator=generator).to(dtype)
               for _ in range(3))
    inner = heads * head_dim
    layout = attention.make_layout((inner,) * 4, head_stride=(head_dim,) * 4,
                                   batch_stride=(tokens * inner,) * 4, causal=causal)
    device = [tensor.cuda() for tensor in (q, k, v)]
    ours = torch.zeros((batch, tokens, heads, head_dim), dtype=dtype, device="cuda")
    theirs = torch.zeros_like(ours)
    angles = None
    if pairs is not None:
        angles = (torch.rand((tokens, pairs), generator=generator) * 6.0 - 3.0).cuda()
        attention.attention_roped(element_type, head_dim, *device, ours, tokens, heads, batch,
                                  layout, scale, angles, pairs, epsilon)
    else:
        attention.attention(element_type, head_dim, *device, ours, tokens, heads, batch, layout,
                            scale)
    assert reference_kernels.mmh3_attention_roped(
        element_type, head_dim, *(tensor.data_ptr() for tensor in device), theirs.data_ptr(),
        tokens, heads, batch, ctypes.byref(layout), scale,
        angles.data_ptr() if angles is not None else None, pairs or 0, epsilon, None) == 0
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    query = normalized_rotated(q, angles.cpu(), pairs, epsilon, dtype) if pairs else q
    scores = torch.einsum("bqhd,bkhd->bhqk", query.double(), k.double()) * scale
    if causal:
        future = torch.triu(torch.ones((tokens, tokens), dtype=torch.bool), diagonal=1)
        scores = scores.masked_fill(future, float("-inf"))
    expected = torch.einsum("bhqk,bkhd->bqhd", scores.softmax(-1), v.double())
    assert torch.max(torch.abs(ours.cpu().double() - expected)) <= 2e-2
    a, b = ours.float().cpu().numpy(), theirs.float().cpu().numpy()
    assert np.max(np.abs(a - b)) <= 2e-2
    assert cosine(a, b) >= 0.9995


def test_unsupported_combinations_report_an_error():
    tokens, heads = 64, 1
    qkv = torch.zeros((tokens, 3, heads, 128), dtype=torch.bfloat16, device="cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    layout = attention.qkv_layout(heads)
    library = _lib.library()
    arguments = (qkv.data_ptr(), qkv.data_ptr() + 256, qkv.data_ptr() + 512, output.data_ptr(),
                 tokens, heads, 1, ctypes.byref(layout), SCALE)
    assert library.mmh3_attention(2, 128, *arguments, None) == _lib.CUDA_ERROR_INVALID_VALUE
    assert library.mmh3_attention(0, 96, *arguments, None) == _lib.CUDA_ERROR_INVALID_VALUE
    angles = torch.zeros((tokens, 64), dtype=torch.float32, device="cuda")
    # more rotary pairs than half a head
    assert library.mmh3_attention_roped(0, 64, *arguments, angles.data_ptr(), 33, 1e-6,
                                        None) == _lib.CUDA_ERROR_INVALID_VALUE


@pytest.mark.parametrize("element_type,head_dim,group,causal",
                         [(0, 128, 1, 0), (1, 64, 1, 0), (0, 128, 2, 1)])
def test_layouts_off_the_tma_grid_equal_aligned_ones(element_type, head_dim, group, causal):
    """Operands whose base or strides are not multiples of 16 bytes: the reference copies them with
    cp.async instead of TMA and asks for the same bits either way
    (crates/mmh3-cuda/tests/attention.rs:91-114). Here they are gathered into dense arrays first,
    and the output must be the bits of the same values in an aligned layout."""
    tokens, heads = 200, 4
    kv_heads = heads // group
    dtype = torch.float16 if element_type else torch.bfloat16
    generator = torch.Generator(device="cpu").manual_seed(31)
    query = (torch.rand((tokens, heads, head_dim), generator=generator) * 4 - 2).to(dtype).cuda()
    key = (torch.rand((tokens, kv_heads, head_dim), generator=generator) * 4 - 2).to(dtype).cuda()
    value = (torch.rand((tokens, kv_heads, head_dim), generator=generator) * 4 - 2).to(dtype).cuda()
    library = _lib.library()
    scale = 1.0 / head_dim ** 0.5

    def run(operands, token_strides, head_strides):
        output = torch.zeros((tokens, heads, head_dim), dtype=dtype, device="cuda")
        layout = attention.make_layout(tuple(token_strides) + (heads * head_dim,),
                                       tuple(head_strides) + (head_dim,),
                                       heads_per_key_value=group if group > 1 else 0,
                                       causal=causal)
        assert library.mmh3_attention(element_type, head_dim, *operands, output.data_ptr(), tokens,
                                      heads, 1, ctypes.byref(layout), scale, None) == 0
        torch.cuda.synchronize()
        assert attention.take_status() == 0
        return output

    aligned = run([tensor.data_ptr() for tensor in (query, key, value)],
                  [heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], [head_dim] * 3)

    # The same values two bytes off a 16-byte boundary, with a token stride of an odd number of
    # elements and heads head_dim + 2 elements apart.
    def shifted(tensor):
        count = tensor.shape[1]
        head_stride = head_dim + 2
        token_stride = count * head_stride + 1
        storage = torch.zeros(tokens * token_stride + 16, dtype=dtype, device="cuda")
        view = torch.as_strided(storage, (tokens, count, head_dim), (token_stride, head_stride, 1), 1)
        view.copy_(tensor)
        return storage, storage.data_ptr() + 2, token_stride, head_stride

    storages = [shifted(tensor) for tensor in (query, key, value)]
    moved = run([entry[1] for entry in storages], [entry[2] for entry in storages],
                [entry[3] for entry in storages])
    assert torch.equal(moved.view(torch.int16), aligned.view(torch.int16))
    # One operand off the grid is enough to take the copy, and the others are left where they are.
    mixed = run([storages[0][1], key.data_ptr(), value.data_ptr()],
                [storages[0][2], kv_heads * head_dim, kv_heads * head_dim],
                [storages[0][3], head_dim, head_dim])
    assert torch.equal(mixed.view(torch.int16), aligned.view(torch.int16))


@pytest.mark.parametrize("groups", [1, 4, 0])
def test_host_pipeline_equals_one_call(groups):
    """Pinned host buffers in and out, a group of heads at a time on four streams (the first and
    the last group one head each): the same bits as one call over device buffers, twice in a row
    over the same buffers."""
    tokens, heads = 700, 6
    host_qkv = synthetic.dense_qkv(tokens, heads, seed=21, pinned=True)
    expected = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.dense_bf16(host_qkv.cuda(), expected, tokens, heads, SCALE)
    qkv = torch.zeros((tokens, 3, heads, 128), dtype=torch.bfloat16, device="cuda")
    output = torch.zeros_like(expected)
    host_output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16).pin_memory()
    pipeline = attention.HostPipeline(tokens, heads, groups=groups)
    # One group; four, the first and the last of one head; or runs that double and drain.
    assert [span for _, span in pipeline.groups] == ([6] if groups == 1 else [1, 2, 2, 1])
    for _ in range(2):
        host_output.zero_()
        pipeline.run(host_qkv, qkv, output, host_output, SCALE)
        torch.cuda.synchronize()
        assert attention.take_status() == 0
        assert torch.equal(host_output, expected.cpu())


def test_sharded_host_pipeline_on_one_rank():
    """World size 1: the sharded pipeline is one copy in, the dense layer, one copy out. (With
    more ranks `bench.py --gpus N` compares it with the resident run on every rank.)"""
    from mmh3_b200.shard import HostUlyssesPipeline, Shard

    tokens, heads = 500, 3
    host_qkv = synthetic.dense_qkv(tokens, heads, seed=22, pinned=True)
    expected = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.dense_bf16(host_qkv.cuda(), expected, tokens, heads, SCALE)

    def dense(qkv, output, count, span):
        attention.dense_bf16(qkv, output, count, span, SCALE)

    pipeline = HostUlyssesPipeline(Shard.even(0, 1, tokens, heads), tokens, heads, dense, 2)
    qkv = torch.zeros((tokens, 3, heads, 128), dtype=torch.bfloat16, device="cuda")
    output = torch.zeros_like(expected)
    host_output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16).pin_memory()
    pipeline.run(host_qkv, qkv, output, host_output)
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.equal(host_output, expected.cpu())
