"""The CPU restatement of the scaled INT8 GEMM against its definition in float64, with the shapes
and bounds of the reference's own tests (crates/mmh3-cuda/tests/int8_gemm.rs)."""

import numpy as np
import pytest

import gemm_cases
import oracle_lib
from mmh3_b200 import synthetic


@pytest.fixture(scope="module")
def oracle():
    return oracle_lib.load()


@pytest.mark.parametrize("m,n,k,f16,seed", [(300, 512, 384, False, 7), (150, 768, 256, True, 11)])
def test_matches_the_definition(oracle, m, n, k, f16, seed):
    # int8_gemm.rs:230-259: BF16 with column maxima from column 128 on, FP16 with a bias.
    a, w, a_scales, w_scales, bias = gemm_cases.operands(m, n, k, seed, bias=f16)
    bits, maxima = oracle_lib.int8_gemm(oracle, a, w, a_scales, w_scales, bias, f16=f16,
                                        maxima_first_column=None if f16 else 128)
    expected = gemm_cases.definition(a, w, a_scales, w_scales, bias)
    actual = gemm_cases.widen(bits, f16)
    # int8_gemm.rs:212
    assert np.all(np.abs(actual - expected) <= np.abs(expected) / 256.0 + 1e-4)
    if not f16:
        np.testing.assert_array_equal(maxima, gemm_cases.column_maxima(bits, 128))


def test_rounds_once_to_nearest_even(oracle):
    # One product whose exact value lies halfway between two BF16 values: 257 * 1 * 1 = 0x101
    # rounds to 256 (even mantissa), 259 to 260.
    a = np.zeros((2, 128), dtype=np.int8)
    w = np.zeros((128, 128), dtype=np.int8)
    a[0, :3] = [127, 127, 3]
    a[1, :3] = [127, 127, 5]
    w[0, :3] = 1
    ones_m, ones_n = np.ones(2, dtype=np.float32), np.ones(128, dtype=np.float32)
    bits, _ = oracle_lib.int8_gemm(oracle, a, w, ones_m, ones_n)
    assert gemm_cases.widen(bits, False)[:, 0].tolist() == [256.0, 260.0]


@pytest.mark.parametrize("f16", [False, True])
def test_swiglu_of_interleaved_rows(oracle, f16):
    # int8_gemm.rs:269-383 without the adapter.
    m, features, k = 60, 256, 256
    n = 2 * features
    a, w, a_scales, w_scales, bias = gemm_cases.operands(m, n, k, 12 + f16, bias=True, swiglu=True)
    bits, _ = oracle_lib.int8_gemm(oracle, a, gemm_cases.interleave(w), a_scales,
                                   gemm_cases.interleave(w_scales), gemm_cases.interleave(bias),
                                   f16=f16, swiglu=True)
    assert bits.shape == (m, features)
    rounded = np.float16 if f16 else None
    products = gemm_cases.definition(a, w, a_scales, w_scales, bias).astype(np.float32)
    if f16:
        products = products.astype(rounded).astype(np.float32)
    else:
        products = synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(products)).reshape(products.shape)
    gate, up = products[:, :features].astype(np.float64), products[:, features:].astype(np.float64)
    expected = gate / (1.0 + np.exp(-gate)) * up
    actual = gemm_cases.widen(bits, f16)
    # int8_gemm.rs:375
    assert np.all(np.abs(actual - expected) <= np.abs(expected) / 64.0 + 1e-3)

