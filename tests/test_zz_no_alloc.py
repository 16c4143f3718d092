"""The allocation-free INT8/FP8 attention entry point, on a B200.

Some callers of this library cannot allocate device memory: a host that budgets the whole device
itself, or a loop that cannot afford cudaMalloc's device-wide stall. For them
mmh3_b200_attention_quantized_static keeps its scratch in a fixed array inside the library. This
test calls it through the C ABI twice in a row, the second time on a smaller problem so that the
array still holds the first call's bytes, and holds each result to what mmh3_attention_quantized
computes with a caller-allocated workspace: the same kernels run over the same bytes, so the outputs
must be identical. It also checks that the shape limit is enforced. The file sorts last so that a
run that stops at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

from mmh3_b200 import _lib, attention, synthetic

pytestmark = pytest.mark.gpu

SCALE = synthetic.softmax_scale()


def test_static_scratch_matches_a_caller_owned_workspace_twice_in_a_row():
    # The second shape fills the array to its last byte (4,096 tokens of 8 heads is the limit);
    # the third is smaller, so the array still holds the bytes of the one before.
    for tokens, heads, seed in [(1000, 3, 21), (4096, 8, 23), (321, 2, 22)]:
        qkv = synthetic.dense_qkv(tokens, heads, seed=seed).cuda()
        expected = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
        actual = torch.zeros_like(expected)
        workspace = attention.QuantizedWorkspace(tokens, heads)
        attention.dense_quantized(qkv, expected, SCALE, workspace, attention.AttentionInputs.RAW)
        attention.dense_quantized_static(qkv, actual, tokens, heads, SCALE)
        assert attention.take_status() == 0
        assert float(expected.float().abs().max()) > 0.0
        assert torch.equal(actual.view(torch.int16), expected.view(torch.int16)), (tokens, heads)


def test_a_repeated_call_takes_no_device_memory():
    """Once the first call on the device has run (it is where the driver backs the array and loads
    the kernels), a further call leaves the device's free memory where it was: nothing is
    allocated, by the CUDA runtime or by torch's allocator."""
    tokens, heads = 640, 4
    qkv = synthetic.dense_qkv(tokens, heads, seed=24).cuda()
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    attention.dense_quantized_static(qkv, output, tokens, heads, SCALE)
    torch.cuda.synchronize()
    reserved = torch.cuda.memory_reserved()
    free_before, _ = torch.cuda.mem_get_info()
    attention.dense_quantized_static(qkv, output, tokens, heads, SCALE)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert attention.take_status() == 0
    assert torch.cuda.memory_reserved() == reserved
    assert free_after == free_before


def test_shapes_past_the_scratch_are_refused():
    tokens, heads = 4096 + 1, 8
    qkv = torch.zeros((tokens, 3, heads, 128), dtype=torch.bfloat16, device="cuda")
    output = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(attention.CudaError) as refused:
        attention.dense_quantized_static(qkv, output, tokens, heads, SCALE)
    assert refused.value.code == _lib.CUDA_ERROR_INVALID_VALUE
    layout = attention.qkv_layout(65)
    code = _lib.library().mmh3_b200_attention_quantized_static(
        None, None, None, None, 64, 65, ctypes.byref(layout), SCALE, None)
    assert code == _lib.CUDA_ERROR_INVALID_VALUE
