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



def test_oracle_matches_the_reference_kernel_fixture(oracle):
    """tests/golden/reference_int8_gemm.npz holds what the reference's own kernel (int8_gemm.cu,
    compiled from its sources) wrote for seeded operands (tests/golden/make_golden.py): the
    restatement reproduces the outputs and the column maxima bit for bit, and the SwiGLU outputs
    to the last place of the rounded result (expf stands where the kernel has __expf)."""
    import pathlib
    import sys

    golden = pathlib.Path(__file__).resolve().parent / "golden"
    sys.path.insert(0, str(golden))
    import make_golden

    fixture = np.load(golden / "reference_int8_gemm.npz")
    for name, (m, n, k, _, f16, swiglu) in make_golden.GEMM_CASES.items():
        tracked = not f16 and not swiglu
        bits, maxima = oracle_lib.int8_gemm(oracle, *make_golden.gemm_operands(name), f16=f16,
                                            swiglu=swiglu,
                                            maxima_first_column=128 if tracked else None)
        expected = fixture[f"{name}_output"]
        if swiglu:
            # BF16 bit patterns of one sign are ordered: at most one step apart.
            assert np.all(np.abs(bits.astype(np.int32) - expected.astype(np.int32)) <= 1)
            assert np.mean(bits != expected) < 0.01
        else:
            assert np.array_equal(bits, expected), name
        if tracked:
            assert np.array_equal(maxima, fixture[f"{name}_maxima"])
