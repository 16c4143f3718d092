"""Parity at the benchmark's own sizes (L = 66,048, H = 32 for the dense, quantized and Sol-Attn
paths; the 31 x 48 x 84 video grid + 512 text tokens for VSA), where the CPU oracle cannot compute a
whole layer. Each path is held to:

- the reference's own CUDA kernel on the same device buffers (oracle/_ref), whole tensors:
  max-abs <= 2e-2 and cosine >= 0.9995 for BF16 outputs, cosine >= 0.9995 for quantized and sparse
  outputs, INT8 q/k, scales, FP8 V, pooled tiles and routes bit for bit;
- the f64 CPU oracle on sampled query rows (dense);
- size-independent properties: a constant value gives that constant back, and the output is linear
  in the values.
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
TOKENS, HEADS = synthetic.CONFIGS["C1"]
INNER = HEADS * 128


def milliseconds(call, repeats: int = 3) -> float:
    """Device time of one `call`, CUDA events around `repeats` of them after one warm-up."""
    call()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        call()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / repeats


def report(path: str, ours: float, theirs: float) -> None:
    """Both libraries ran on the legacy default stream of the same device."""
    print(f"\n{path}: {ours:.2f} ms here, {theirs:.2f} ms for the reference's kernels "
          f"compiled for sm_100a ({theirs / ours:.1f} x)")
    assert ours < theirs


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm()))


@pytest.fixture(scope="module")
def dense_case():
    host = synthetic.dense_qkv(TOKENS, HEADS, seed=1)
    return host, host.cuda()


def test_dense_bf16_at_the_benchmark_size(oracle, reference_kernels, dense_case):
    host, qkv = dense_case
    ours = torch.zeros((TOKENS, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    attention.dense_bf16(qkv, ours, TOKENS, HEADS, SCALE)
    base = qkv.data_ptr()

    def reference_call():
        assert reference_kernels.mmh3_attention_bf16(
            base, base + 2 * INNER, base + 4 * INNER, theirs.data_ptr(), TOKENS, HEADS, 3 * INNER,
            3 * INNER, 3 * INNER, INNER, SCALE, None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 2e-2
    assert cosine(ours, theirs) >= 0.9995

    report("dense BF16, L=66,048, H=32",
           milliseconds(lambda: attention.dense_bf16(qkv, ours, TOKENS, HEADS, SCALE)),
           milliseconds(reference_call))

    # Sampled query rows of four heads against all 66,048 keys in f64 on the CPU.
    bits = host.view(torch.int16).numpy().view(np.uint16)
    for row in (0, 255, 256, 33_333, TOKENS - 1):
        for head in (0, 13, 31):
            expected = oracle_lib.attention_bf16(oracle, bits, TOKENS, HEADS, SCALE, row, row + 1,
                                                 head, head + 1)
            actual = ours[row, head].float().cpu().numpy()
            assert np.max(np.abs(actual - expected[0, 0])) <= 2e-2

    # A constant value row comes back whatever the weights are; the output is linear in v.
    constant = qkv.clone()
    pattern = torch.linspace(-2.0, 2.0, 128, device="cuda").bfloat16()
    constant[:, 2] = pattern
    attention.dense_bf16(constant, theirs, TOKENS, HEADS, SCALE)
    assert torch.max(torch.abs(theirs.float() - pattern.float())).item() <= 2 ** -6
    halved = qkv.clone()
    halved[:, 2] = (qkv[:, 2].float() * 0.5).bfloat16()  # exact in BF16
    attention.dense_bf16(halved, theirs, TOKENS, HEADS, SCALE)
    assert attention.take_status() == 0
    assert torch.max(torch.abs(theirs.float() * 2.0 - ours.float())).item() <= 2 ** -7


def test_quantized_at_the_benchmark_size(reference_kernels, dense_case):
    _, qkv = dense_case
    ours = torch.zeros((TOKENS, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    workspace = attention.QuantizedWorkspace(TOKENS, HEADS)
    other = attention.QuantizedWorkspace(TOKENS, HEADS)
    attention.dense_quantized(qkv, ours, SCALE, workspace, attention.AttentionInputs.RAW)
    layout = attention.qkv_layout(HEADS)
    raw = other.raw()
    base = qkv.data_ptr()
    def reference_call(ready=0):
        assert reference_kernels.mmh3_attention_quantized(
            base, base + 2 * INNER, base + 4 * INNER, theirs.data_ptr(), TOKENS, HEADS,
            ctypes.byref(layout), SCALE, None, ctypes.byref(raw), ready, None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    for name in ("query", "key", "value", "query_scales", "key_scales", "value_scales"):
        assert torch.equal(getattr(workspace, name), getattr(other, name)), name
    prepared = attention.AttentionInputs.PREPARED_WITH_VALUES
    report("INT8/FP8 over a prepared workspace, L=66,048, H=32",
           milliseconds(lambda: attention.dense_quantized(qkv, ours, SCALE, workspace, prepared)),
           milliseconds(lambda: reference_call(2)))
    report("INT8/FP8 from BF16 rows (quantizer included)",
           milliseconds(lambda: attention.dense_quantized(qkv, ours, SCALE, workspace,
                                                          attention.AttentionInputs.RAW)),
           milliseconds(reference_call))
    assert cosine(ours, theirs) >= 0.9995
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 0.1


def test_sol_attention_at_the_benchmark_size(reference_kernels, dense_case):
    _, qkv = dense_case
    tau, sinks = 1.3, SparseSinks((0, 8), (0, 0))
    ours = torch.zeros((TOKENS, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    workspace = attention.SparseWorkspace(TOKENS, HEADS)
    other = attention.SparseWorkspace(TOKENS, HEADS)
    layout = attention.qkv_layout(HEADS)
    attention.sparse(qkv, ours, layout, SCALE, tau, sinks, workspace)
    raw = other.raw()
    base = qkv.data_ptr()
    def reference_call():
        assert reference_kernels.mmh3_sparse_attention(
            base, base + 2 * INNER, base + 4 * INNER, theirs.data_ptr(), TOKENS, HEADS,
            ctypes.byref(layout), SCALE, tau, *sinks.key_blocks, *sinks.query_blocks,
            ctypes.byref(raw), None, 0, None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.equal(workspace.route_counts, other.route_counts)
    blocks = workspace.blocks
    valid = (torch.arange(blocks, device="cuda")[None, :] <
             workspace.route_counts.view(-1, 1))
    assert torch.equal(workspace.routes.view(-1, blocks)[valid],
                       other.routes.view(-1, blocks)[valid])
    for name in ("centroids", "block_keys", "value_sums", "key_mean", "key_variance", "tail_max"):
        assert torch.equal(getattr(workspace, name), getattr(other, name)), name
    assert 0.05 < workspace.routed_fraction() < 0.5
    assert cosine(ours, theirs) >= 0.9995
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 2e-2
    report("Sol-Attn, L=66,048, H=32, tau 1.3",
           milliseconds(lambda: attention.sparse(qkv, ours, layout, SCALE, tau, sinks, workspace)),
           milliseconds(reference_call))


@pytest.fixture(scope="module")
def video_case():
    layout, plan = synthetic.video_plan()
    tokens = len(layout)
    generator = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn((tokens, 3, HEADS, 128), generator=generator, device="cuda").bfloat16()
    # A smooth component per head and channel so that the pooled scores are not uniform.
    positions = torch.linspace(0.0, 12.0, tokens, device="cuda")
    for head in range(HEADS):
        phase = torch.rand((3, 128), generator=generator, device="cuda") * 6.283
        qkv[:, :, head, :] = (qkv[:, :, head, :].float() +
                              0.5 * torch.sin(positions[:, None, None] + phase)).bfloat16()
    return plan, tokens, plan.kept_video_tiles(0.875), qkv


def test_video_sparse_attention_at_the_benchmark_size(reference_kernels, video_case):
    plan, tokens, kept, qkv = video_case
    ours = torch.zeros((tokens, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    workspace = attention.VsaWorkspace(plan, tokens, HEADS)
    other = attention.VsaWorkspace(plan, tokens, HEADS)
    vsa_layout = attention.qkv_layout(HEADS)
    attention.vsa(qkv, None, ours, vsa_layout, SCALE, kept, workspace)
    raw = other.raw()
    base = qkv.data_ptr()
    def reference_call():
        assert reference_kernels.mmh3_vsa_attention(
            base, base + 2 * INNER, base + 4 * INNER, None, INNER, theirs.data_ptr(), tokens,
            HEADS, ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept,
            ctypes.byref(raw), None, 0, None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert abs(workspace.selected_fraction() - plan.expected_selected_fraction(kept)) < 1e-9
    for name in ("pooled_query", "pooled_key", "pooled_value", "route_counts"):
        assert torch.equal(getattr(workspace, name), getattr(other, name)), name
    valid = (torch.arange(plan.tiles, device="cuda")[None, :] <
             workspace.route_counts.view(-1, 1))
    assert torch.equal(workspace.routes.view(-1, plan.tiles)[valid],
                       other.routes.view(-1, plan.tiles)[valid])
    assert cosine(ours, theirs) >= 0.9995
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 2e-2
    report("VSA, L=125,504, H=32, 252 of 2,016 video tiles kept",
           milliseconds(lambda: attention.vsa(qkv, None, ours, vsa_layout, SCALE, kept, workspace)),
           milliseconds(reference_call))


def test_gated_video_sparse_attention_at_the_benchmark_size(reference_kernels, video_case):
    """The same layer with the gate of the coarse branch: the coarse output of all 2,024 x 32 query
    tiles to 1e-4 of the reference kernel's, the routes its bits, the gated output close."""
    plan, tokens, kept, qkv = video_case
    generator = torch.Generator(device="cuda").manual_seed(5)
    gate = torch.randn((tokens, INNER), generator=generator, device="cuda").bfloat16()
    ours = torch.zeros((tokens, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    workspace = attention.VsaWorkspace(plan, tokens, HEADS)
    other = attention.VsaWorkspace(plan, tokens, HEADS)
    vsa_layout = attention.qkv_layout(HEADS)
    attention.vsa(qkv, gate, ours, vsa_layout, SCALE, kept, workspace)
    raw = other.raw()
    base = qkv.data_ptr()
    def reference_call():
        assert reference_kernels.mmh3_vsa_attention(
            base, base + 2 * INNER, base + 4 * INNER, gate.data_ptr(), INNER, theirs.data_ptr(),
            tokens, HEADS, ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept,
            ctypes.byref(raw), None, 0, None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.equal(workspace.route_counts, other.route_counts)
    valid = (torch.arange(plan.tiles, device="cuda")[None, :] <
             workspace.route_counts.view(-1, 1))
    assert torch.equal(workspace.routes.view(-1, plan.tiles)[valid],
                       other.routes.view(-1, plan.tiles)[valid])
    assert torch.allclose(workspace.coarse, other.coarse, rtol=1e-4, atol=1e-5)
    assert cosine(ours, theirs) >= 0.9995
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 2e-2
    report("gated VSA, L=125,504, H=32, 252 of 2,016 video tiles kept",
           milliseconds(lambda: attention.vsa(qkv, gate, ours, vsa_layout, SCALE, kept, workspace)),
           milliseconds(reference_call))


def test_quantized_video_sparse_attention_at_the_benchmark_size(reference_kernels, video_case):
    """The INT8/FP8 form of the same layer, as the DiT calls it with inputs_ready = 2: both
    libraries prepare their own copy of the rows (norm, INT8 q/k, FP8 V, pooled tiles), select and
    attend. Everything the fused pass and the selection leave is held to the reference's bits,
    whole tensors; the output to its cosine."""
    plan, tokens, kept, source = video_case
    ones = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    norm = attention.HeadNorm(ones, ones, None, 0, 1e-6)
    maxima = source[:, 2].float().abs().amax(dim=(0, 2)).contiguous()
    vsa_layout = attention.qkv_layout(HEADS)
    prepared = attention.AttentionInputs.PREPARED_WITH_VALUES

    qkv = source.clone()
    ours = torch.zeros((tokens, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    workspace = attention.VsaWorkspace(plan, tokens, HEADS, quantized=True)
    attention.prepare_inputs(qkv, norm, tokens, HEADS, vsa=workspace, value_head_maxima=maxima)
    attention.vsa(qkv, None, ours, vsa_layout, SCALE, kept, workspace, prepared)

    their_qkv = source.clone()
    theirs = torch.zeros_like(ours)
    other = attention.VsaWorkspace(plan, tokens, HEADS, quantized=True)
    sparse, quantized, raw = other.sparse_raw(), other.quantized.raw(), other.raw()
    assert reference_kernels.mmh3_attention_inputs(
        their_qkv.data_ptr(), ones.data_ptr(), ones.data_ptr(), None, 0, tokens, HEADS, 1e-6,
        ctypes.byref(sparse), ctypes.byref(quantized), other.tile_starts.data_ptr(),
        other.tile_lengths.data_ptr(), other.tiles, maxima.data_ptr(), None) == 0
    base = their_qkv.data_ptr()

    def reference_call():
        assert reference_kernels.mmh3_vsa_attention(
            base, base + 2 * INNER, base + 4 * INNER, None, INNER, theirs.data_ptr(), tokens,
            HEADS, ctypes.byref(vsa_layout), SCALE, plan.tiles, plan.prefix_tiles, kept,
            ctypes.byref(raw), ctypes.byref(quantized), int(prepared), None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.equal(qkv, their_qkv)  # the normalized rows both left in place
    for name in ("query", "key", "value", "query_scales", "key_scales", "value_scales"):
        assert torch.equal(getattr(workspace.quantized, name), getattr(other.quantized, name)), name
    for name in ("pooled_query", "pooled_key", "pooled_value", "route_counts"):
        assert torch.equal(getattr(workspace, name), getattr(other, name)), name
    assert abs(workspace.selected_fraction() - plan.expected_selected_fraction(kept)) < 1e-9
    valid = (torch.arange(plan.tiles, device="cuda")[None, :] <
             workspace.route_counts.view(-1, 1))
    assert torch.equal(workspace.routes.view(-1, plan.tiles)[valid],
                       other.routes.view(-1, plan.tiles)[valid])
    assert cosine(ours, theirs) >= 0.9995
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 0.1
    report("INT8/FP8 VSA over prepared inputs, L=125,504, H=32",
           milliseconds(lambda: attention.vsa(qkv, None, ours, vsa_layout, SCALE, kept, workspace,
                                              prepared)),
           milliseconds(reference_call))


def test_quantized_sol_attention_at_the_benchmark_size(reference_kernels, dense_case):
    """Sol-Attn with INT8 QK / FP8 PV routed products at L = 66,048: routes, block statistics and
    the quantizer's outputs bit for bit against the reference's kernels, the output to its
    cosine."""
    _, qkv = dense_case
    tau, sinks = 1.3, SparseSinks((0, 8), (0, 0))
    ours = torch.zeros((TOKENS, HEADS, 128), dtype=torch.bfloat16, device="cuda")
    theirs = torch.zeros_like(ours)
    workspace = attention.SparseWorkspace(TOKENS, HEADS, quantized=True)
    other = attention.SparseWorkspace(TOKENS, HEADS, quantized=True)
    layout = attention.qkv_layout(HEADS)
    attention.sparse(qkv, ours, layout, SCALE, tau, sinks, workspace)
    raw, their_quantized = other.raw(), other.quantized.raw()
    base = qkv.data_ptr()

    def reference_call():
        assert reference_kernels.mmh3_sparse_attention(
            base, base + 2 * INNER, base + 4 * INNER, theirs.data_ptr(), TOKENS, HEADS,
            ctypes.byref(layout), SCALE, tau, *sinks.key_blocks, *sinks.query_blocks,
            ctypes.byref(raw), ctypes.byref(their_quantized), 0, None) == 0

    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.equal(workspace.route_counts, other.route_counts)
    blocks = workspace.blocks
    valid = (torch.arange(blocks, device="cuda")[None, :] <
             workspace.route_counts.view(-1, 1))
    assert torch.equal(workspace.routes.view(-1, blocks)[valid],
                       other.routes.view(-1, blocks)[valid])
    for name in ("centroids", "block_keys", "value_sums", "key_mean", "key_variance", "tail_max"):
        assert torch.equal(getattr(workspace, name), getattr(other, name)), name
    for name in ("query", "key", "value", "query_scales", "key_scales", "value_scales"):
        assert torch.equal(getattr(workspace.quantized, name), getattr(other.quantized, name)), name
    assert cosine(ours, theirs) >= 0.9995
    assert torch.max(torch.abs(ours.float() - theirs.float())).item() <= 0.1
    report("Sol-Attn with INT8/FP8 routed products, L=66,048, H=32, tau 1.3",
           milliseconds(lambda: attention.sparse(qkv, ours, layout, SCALE, tau, sinks, workspace)),
           milliseconds(reference_call))


def test_qkv_projection_at_the_benchmark_size(reference_kernels):
    """The INT8 qkv projection of the same layer (M = 66,048, N = 12,288, K = 4,096): outputs and
    per-head |v| maxima bit-identical to the reference's kernel, whole tensors; and a property that
    needs no reference: doubling every activation scale doubles every output exactly."""
    from mmh3_b200 import gemm

    generator = torch.Generator(device="cuda").manual_seed(4)
    activations = torch.randint(-127, 128, (TOKENS, INNER), dtype=torch.int8, device="cuda",
                                generator=generator)
    weights = torch.randint(-127, 128, (3 * INNER, INNER), dtype=torch.int8, device="cuda",
                            generator=generator)
    activation_scales = torch.rand(TOKENS, device="cuda", generator=generator) + 0.5
    weight_scales = torch.rand(3 * INNER, device="cuda", generator=generator) * 1e-4 + 1e-5
    ours = torch.zeros((TOKENS, 3 * INNER), dtype=torch.int16, device="cuda")
    theirs = torch.zeros_like(ours)
    maxima = torch.zeros(HEADS, dtype=torch.float32, device="cuda")
    their_maxima = torch.zeros_like(maxima)

    def call(scales=activation_scales, output=ours, tracked=maxima):
        gemm.int8(None, activations, weights, scales, weight_scales,
                  gemm.Output(output, column_maxima=gemm.ColumnMaxima(tracked, 2 * INNER)),
                  TOKENS, 3 * INNER, INNER)

    def reference_call():
        assert reference_kernels.mmh3_int8_gemm(
            -1, 0, activations.data_ptr(), weights.data_ptr(), activation_scales.data_ptr(),
            weight_scales.data_ptr(), None, theirs.data_ptr(), 0, 0, TOKENS, 3 * INNER, INNER, 0,
            None, None, 0, 0, 0.0, their_maxima.data_ptr(), 2 * INNER, None) == 0

    call()
    torch.cuda.synchronize()
    reference_call()
    torch.cuda.synchronize()
    assert attention.take_status() == 0
    assert torch.equal(ours, theirs)
    assert torch.equal(maxima, their_maxima)
    values = ours.view(torch.bfloat16).view(TOKENS, 3, HEADS, 128)[:, 2]
    assert torch.equal(maxima, values.float().abs().amax(dim=(0, 2)))

    doubled = torch.zeros_like(ours)
    call(scales=activation_scales * 2.0, output=doubled, tracked=torch.zeros_like(maxima))
    assert torch.equal(doubled.view(torch.bfloat16).float(), ours.view(torch.bfloat16).float() * 2.0)
    del doubled

    # The reference times its tilings on the first call of a shape; it has, above.
    report("INT8 qkv projection, M=66,048, N=12,288, K=4,096", milliseconds(call),
           milliseconds(reference_call))
