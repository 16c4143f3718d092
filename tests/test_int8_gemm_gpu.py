"""Parity of the scaled INT8 GEMM on a B200, through the C ABI.

Mirrors crates/mmh3-cuda/tests/int8_gemm.rs (the same shapes, value
ranges and bounds against the definition in float64, with and without the low-rank adapter, the
column maxima equal to those of the kernel's own output, every tiling the same bits) and adds what the drop-in must hold: outputs and
maxima bit-identical to the CPU restatement and to the reference's own kernel, and the per-head
maxima of |v| feeding the fused attention inputs.
"""

import ctypes

import numpy as np
import pytest
import torch

import gemm_cases
import oracle_lib
from mmh3_b200 import _lib, attention, gemm, synthetic
from mmh3_b200.gemm import Adapter, ColumnMaxima, Int8Tiling, Output

pytestmark = pytest.mark.gpu

TILINGS = [None, Int8Tiling(0, 4), Int8Tiling(0, 16), Int8Tiling(1, 8)]


def upload(array):
    return None if array is None else torch.from_numpy(np.ascontiguousarray(array)).cuda()


def run(case, m, n, k, f16=False, swiglu=False, first_column=None, tiling=None, stride=0,
        adapter=None):
    a, w, a_scales, w_scales, bias = (upload(array) for array in case)
    if adapter is not None:
        down, up, rank, scale = adapter
        adapter = Adapter(upload(down).view(torch.int16), upload(up).view(torch.int16), rank,
                          down.shape[1], scale)
    columns = n // 2 if swiglu else n
    row = stride if stride else columns
    # A sentinel shows what the kernel does not write.
    output = torch.full((m, row), 0x7fc1, dtype=torch.int16, device="cuda")
    maxima = None
    if first_column is not None:
        maxima = ColumnMaxima(torch.zeros(max((n - first_column) // 128, 1), dtype=torch.float32,
                                          device="cuda"), first_column)
    gemm.int8(tiling, a, w, a_scales, w_scales,
              Output(output, f16=f16, bias=bias, swiglu=swiglu, column_maxima=maxima,
                     stride=stride), m, n, k, adapter)
    assert attention.take_status() == 0
    bits = output.cpu().numpy().view(np.uint16)
    return bits, None if maxima is None else maxima.values.cpu().numpy()


def run_reference(library, case, m, n, k, f16=False, swiglu=False, first_column=None,
                  adapter=None):
    a, w, a_scales, w_scales, bias = (upload(array) for array in case)
    down = up = None
    rank, down_stride, scale = 0, 0, 0.0
    if adapter is not None:
        down, up, rank, scale = adapter
        down_stride = down.shape[1]
        down, up = upload(down), upload(up)
    columns = n // 2 if swiglu else n
    output = torch.zeros((m, columns), dtype=torch.int16, device="cuda")
    maxima = torch.zeros(max((n - (first_column or 0)) // 128, 1), dtype=torch.float32,
                         device="cuda")
    pointer = lambda tensor: ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())
    torch.cuda.synchronize()
    code = library.mmh3_int8_gemm(
        0, 8, pointer(a), pointer(w), pointer(a_scales), pointer(w_scales), pointer(bias),
        pointer(output), int(f16), int(swiglu), m, n, k, 0, pointer(down), pointer(up), rank,
        down_stride, scale, pointer(maxima if first_column is not None else None),
        first_column or 0, None)
    assert code == 0
    torch.cuda.synchronize()
    return output.cpu().numpy().view(np.uint16), maxima.cpu().numpy()


@pytest.mark.parametrize("m,n,k,f16,seed", [
    (300, 512, 384, False, 7),      # int8_gemm.rs:231-233
    (2000, 3072, 384, False, 8),    # 236-240: more tiles than SMs, a ragged last row of tiles
    (600, 3072, 256, True, 11),     # 256-258: FP16 with a bias
    (257, 384, 128, False, 3),      # one row into the second tile, a last tile of 128 columns
])
def test_matches_the_definition_oracle_and_reference(oracle, reference_kernels, m, n, k, f16, seed):
    case = gemm_cases.operands(m, n, k, seed, bias=f16)
    first_column = None if f16 else 128
    bits, maxima = run(case, m, n, k, f16=f16, first_column=first_column)
    expected = gemm_cases.definition(*case)
    actual = gemm_cases.widen(bits, f16)
    assert np.all(np.abs(actual - expected) <= np.abs(expected) / 256.0 + 1e-4)  # rs:212
    oracle_bits, oracle_maxima = oracle_lib.int8_gemm(oracle, *case, f16=f16,
                                                      maxima_first_column=first_column)
    assert np.array_equal(bits, oracle_bits)
    reference_bits, reference_maxima = run_reference(reference_kernels, case, m, n, k, f16=f16,
                                                     first_column=first_column)
    assert np.array_equal(bits, reference_bits)
    if not f16:
        expected_maxima = gemm_cases.column_maxima(bits, first_column)
        assert np.array_equal(maxima, expected_maxima)  # rs:199-203
        assert np.array_equal(maxima, oracle_maxima)
        assert np.array_equal(maxima, reference_maxima)
    for tiling in TILINGS[1:]:
        if tiling.config == 1 and n % 256:
            continue
        other, other_maxima = run(case, m, n, k, f16=f16, first_column=first_column,
                                  tiling=tiling)
        assert np.array_equal(bits, other), tiling  # rs:221-227
        if not f16:
            assert np.array_equal(maxima, other_maxima)


@pytest.mark.parametrize("f16", [False, True])
def test_swiglu_of_interleaved_rows(oracle, reference_kernels, f16):
    # int8_gemm.rs:269-383 without the adapter; the rows interleaved by the library itself.
    m, features, k = 300, 1024, 256
    n = 2 * features
    a, w, a_scales, w_scales, bias = gemm_cases.operands(m, n, k, 12 + f16, bias=True,
                                                          swiglu=True)

    def interleaved(array, row_bytes):
        source = upload(array)
        destination = torch.empty_like(source)
        gemm.interleave_swiglu_rows(source, destination, n, row_bytes)
        return destination.cpu().numpy()

    w_mixed = interleaved(w, k)
    assert np.array_equal(w_mixed, gemm_cases.interleave(w))
    case = (a, w_mixed, a_scales, interleaved(w_scales, 4), interleaved(bias, 4))
    bits, _ = run(case, m, n, k, f16=f16, swiglu=True)
    assert bits.shape == (m, features)
    products = gemm_cases.definition(a, w, a_scales, w_scales, bias).astype(np.float32)
    if f16:
        products = products.astype(np.float16).astype(np.float32)
    else:
        products = synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(products)).reshape(m, n)
    gate, up = products[:, :features].astype(np.float64), products[:, features:].astype(np.float64)
    expected = gate / (1.0 + np.exp(-gate)) * up
    actual = gemm_cases.widen(bits, f16)
    assert np.all(np.abs(actual - expected) <= np.abs(expected) / 64.0 + 1e-3)  # rs:375
    reference_bits, _ = run_reference(reference_kernels, case, m, n, k, f16=f16, swiglu=True)
    assert np.array_equal(bits, reference_bits)


@pytest.mark.parametrize("m,n,k,rank,stride,seed", [
    (300, 512, 256, 128, 128, 9),    # int8_gemm.rs:243-247
    (600, 3072, 256, 384, 384, 10),  # the rank of the fused qkv adapters, more tiles than SMs
    (300, 512, 256, 64, 128, 12),    # 250-253: down rows wider than the rank
])
def test_adds_a_low_rank_adapter(reference_kernels, m, n, k, rank, stride, seed):
    case = gemm_cases.operands(m, n, k, seed)
    down, up = gemm_cases.adapter_operands(m, n, rank, stride, seed + 100)
    adapter = (down, up, rank, 1.5)
    bits, maxima = run(case, m, n, k, first_column=128, adapter=adapter)
    expected = gemm_cases.definition(*case, adapter=adapter)
    actual = gemm_cases.widen(bits, False)
    assert np.all(np.abs(actual - expected) <= np.abs(expected) / 256.0 + 1e-4)  # rs:212
    assert np.array_equal(maxima, gemm_cases.column_maxima(bits, 128))
    # The reference's kernel sums the BF16 products in another order: the same bounds, and
    # nearly always the same BF16 value.
    reference_bits, _ = run_reference(reference_kernels, case, m, n, k, first_column=128,
                                      adapter=adapter)
    theirs = gemm_cases.widen(reference_bits, False)
    assert np.all(np.abs(actual - theirs) <= np.abs(theirs) / 128.0 + 2e-4)
    assert np.mean(bits != reference_bits) < 0.01
    for tiling in TILINGS[1:]:
        other, _ = run(case, m, n, k, first_column=128, tiling=tiling, adapter=adapter)
        assert np.array_equal(bits, other), tiling


@pytest.mark.parametrize("f16", [False, True])
def test_swiglu_with_an_adapter(reference_kernels, f16):
    # int8_gemm.rs:269-383 in full: interleaved rows, a bias and an adapter of rank 128.
    m, features, k, rank = 300, 1024, 256, 128
    n = 2 * features
    a, w, a_scales, w_scales, bias = gemm_cases.operands(m, n, k, 12 + f16, bias=True,
                                                          swiglu=True)
    down, up = gemm_cases.adapter_operands(m, n, rank, rank, 50 + f16, span=0.5)
    case = (a, gemm_cases.interleave(w), a_scales, gemm_cases.interleave(w_scales),
            gemm_cases.interleave(bias))
    bits, _ = run(case, m, n, k, f16=f16, swiglu=True,
                  adapter=(down, gemm_cases.interleave(up), rank, 0.75))
    products = gemm_cases.definition(a, w, a_scales, w_scales, bias,
                                     adapter=(down, up, rank, 0.75)).astype(np.float32)
    if f16:
        products = products.astype(np.float16).astype(np.float32)
    else:
        products = synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(products)).reshape(m, n)
    gate, up_values = (products[:, :features].astype(np.float64),
                       products[:, features:].astype(np.float64))
    expected = gate / (1.0 + np.exp(-gate)) * up_values
    actual = gemm_cases.widen(bits, f16)
    # rs:375. The adapter's FP32 sums come in the tensor cores' order, so a product that lies
    # within FP32 rounding of the midpoint of two BF16 values may round the other way, and where
    # silu is steep (gate near -5.5) one such step moves the output by more than the bound: a
    # handful of 307,200 outputs at most, and nearly every output is the reference kernel's.
    excess = np.abs(actual - expected) - (np.abs(expected) / 64.0 + 1e-3)
    assert np.count_nonzero(excess > 0) <= 3 and excess.max() < 0.01
    reference_bits, _ = run_reference(reference_kernels, case, m, n, k, f16=f16, swiglu=True,
                                      adapter=(down, gemm_cases.interleave(up), rank, 0.75))
    assert np.mean(bits == reference_bits) > 0.998


def test_writes_rows_at_their_stride():
    # A shared-out step writes one rank's columns into a row that holds every rank's
    # (crates/mmh3-cuda/src/gemm.rs:175-177).
    m, n, k, stride = 130, 256, 128, 640
    case = gemm_cases.operands(m, n, k, 21)
    bits, _ = run(case, m, n, k)
    wide, _ = run(case, m, n, k, stride=stride)
    assert np.array_equal(wide[:, :n], bits)
    assert np.all(wide[:, n:] == 0x7fc1)


def test_bf16_entry_point(oracle):
    m, n, k = 100, 256, 256
    case = gemm_cases.operands(m, n, k, 5)
    a, w, a_scales, w_scales, _ = (upload(array) for array in case)
    output = torch.zeros((m, n), dtype=torch.int16, device="cuda")
    pointer = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    code = _lib.library().mmh3_int8_gemm_bf16(1, 4, pointer(a), pointer(w), pointer(a_scales),
                                              pointer(w_scales), pointer(output), m, n, k, None)
    assert code == 0 and attention.take_status() == 0
    expected, _ = oracle_lib.int8_gemm(oracle, *case)
    assert np.array_equal(output.cpu().numpy().view(np.uint16), expected)


def test_rejects_what_the_reference_rejects():
    m, n, k = 64, 256, 256
    case = gemm_cases.operands(m, n, k, 1)
    a, w, a_scales, w_scales, _ = (upload(array) for array in case)
    output = torch.zeros((m, n), dtype=torch.int16, device="cuda")
    maxima = torch.zeros(2, dtype=torch.float32, device="cuda")
    pointer = lambda tensor: ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())

    def call(config=0, group_m=8, m=m, n=n, k=k, f16=0, swiglu=0, down=None, maxima=None,
             first_column=0):
        return _lib.library().mmh3_int8_gemm(
            config, group_m, pointer(a), pointer(w), pointer(a_scales), pointer(w_scales), None,
            pointer(output), f16, swiglu, m, n, k, 0, pointer(down), None, 0, 0, 0.0,
            pointer(maxima), first_column, None)

    invalid = _lib.CUDA_ERROR_INVALID_VALUE
    assert call() == 0
    assert call(n=192) == invalid                          # int8_gemm.cu:640
    assert call(config=1, n=128) == invalid                # the wide tiling needs 256 columns
    assert call(k=192) == invalid
    assert call(m=0) == invalid
    assert call(group_m=0) == invalid
    assert call(config=2) == invalid                       # int8_gemm.cu:710
    assert call(config=-1, group_m=0) == 0                 # the chosen tiling names no band
    assert call(maxima=maxima, f16=1) == invalid           # int8_gemm.cu:919-921
    assert call(maxima=maxima, swiglu=1) == invalid        # int8_gemm.cu:720
    assert call(maxima=maxima, first_column=64) == invalid
    assert attention.take_status() == 0
    assert gemm.configs() == 2 and gemm.group_heights() == [4, 8, 16]
    # The tiling search's bookkeeping: nothing chosen, a key that names this library.
    key = ctypes.create_string_buffer(128)
    assert _lib.library().mmh3_int8_gemm_tilings(None, 0) == 0
    assert _lib.library().mmh3_int8_gemm_tiling_key(key, 128) == 0 and b"tcgen05" in key.value
    assert _lib.library().mmh3_int8_gemm_tiling_key(key, 4) == invalid


def test_value_maxima_feed_the_attention_inputs():
    """crates/mmh3-cuda/src/dit.rs:1873-1877, 1965: the qkv projection leaves the maximum |v| of
    each head, and the fused input pass quantizes V by them: the same FP8 V and scales as the
    quantizer finds from the BF16 values itself."""
    tokens, heads, k = 333, 2, 256
    inner = heads * 128
    n = 3 * inner
    case = gemm_cases.operands(tokens, n, k, 31)
    a, w, a_scales, w_scales, _ = (upload(array) for array in case)
    qkv = torch.zeros((tokens, n), dtype=torch.bfloat16, device="cuda")
    quantized = attention.QuantizedWorkspace(tokens, heads)
    maxima = torch.zeros(heads, dtype=torch.float32, device="cuda")
    gemm.int8(None, a, w, a_scales, w_scales,
              Output(qkv.view(torch.int16), column_maxima=ColumnMaxima(maxima, 2 * inner)),
              tokens, n, k)
    values = qkv.view(tokens, 3, heads, 128)[:, 2].float().abs().amax(dim=(0, 2))
    assert torch.equal(maxima, values)

    weight = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    norm = attention.HeadNorm(weight, weight, None, 0, 1e-6)
    prepared = qkv.clone()
    attention.prepare_inputs(prepared, norm, tokens, heads, quantized, value_head_maxima=maxima)
    # The separate passes: the norm in place, then the quantizer over the BF16 rows.
    separate = qkv.clone()
    attention.qk_norm_rope(separate, norm, tokens, heads)
    own = attention.QuantizedWorkspace(tokens, heads)
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.dense_quantized(separate, output, synthetic.softmax_scale(), own,
                              inputs=attention.AttentionInputs.RAW)
    assert attention.take_status() == 0
    assert torch.equal(quantized.value, own.value)
    assert torch.equal(quantized.value_scales, own.value_scales)
    # And the attention over inputs made complete that way (inputs_ready = 2) is the same.
    complete = torch.zeros_like(output)
    attention.dense_quantized(prepared, complete, synthetic.softmax_scale(), quantized,
                              inputs=attention.AttentionInputs.PREPARED_WITH_VALUES)
    assert attention.take_status() == 0
    assert torch.equal(complete, output)
