"""The C-ABI library loads without a GPU, exports every symbol the headers of include/ declare,
lays its structs out as the reference's #[repr(C)] mirrors do, and rejects bad arguments with the
reference's error codes before touching a device. No kernel runs here."""

import ctypes
import pathlib
import re
import subprocess

import pytest

from mmh3_b200 import _lib

REPO = pathlib.Path(__file__).resolve().parent.parent
HEADERS = sorted((REPO / "include").glob("*.h"))


def declared_functions():
    names = set()
    for header in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"^int\s+(mmh3_\w+)\s*\(", text, flags=re.M))
    return sorted(names)


def test_headers_compile_as_c():
    assert [header.name for header in HEADERS] == ["mmh3_attention.h", "mmh3_int8_gemm.h"]
    for header in HEADERS:
        subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", str(header)], check=True)


def test_every_declared_symbol_is_exported():
    library = _lib.library()
    names = declared_functions()
    assert len(names) == 20
    assert sorted(_lib.SIGNATURES) == names
    for name in names + ["mmh3_int8_gemm_adopt"]:  # the one declared function that returns void
        assert getattr(library, name) is not None


def test_struct_layouts():
    # crates/mmh3-cuda/src/attention.rs:13-23, 49-58, 143-156, 962-972
    assert ctypes.sizeof(_lib.AttentionLayout) == 104
    assert _lib.AttentionLayout.head_stride.offset == 32
    assert _lib.AttentionLayout.batch_stride.offset == 64
    assert _lib.AttentionLayout.heads_per_key_value.offset == 96
    assert _lib.AttentionLayout.causal.offset == 100
    assert ctypes.sizeof(_lib.QuantizedWorkspaceStruct) == 7 * 8
    assert ctypes.sizeof(_lib.SparseWorkspace) == 11 * 8
    assert ctypes.sizeof(_lib.VsaWorkspaceStruct) == 8 * 8


def test_bad_arguments_are_rejected_before_any_launch():
    library = _lib.library()
    layout = _lib.AttentionLayout()
    for index in range(4):
        layout.token_stride[index] = 384
        layout.head_stride[index] = 128
    invalid = _lib.CUDA_ERROR_INVALID_VALUE
    assert library.mmh3_attention(0, 128, None, None, None, None, 0, 1, 1, ctypes.byref(layout),
                                  0.1, None) == invalid
    assert library.mmh3_attention(0, 128, None, None, None, None, 8, 0, 1, ctypes.byref(layout),
                                  0.1, None) == invalid
    layout.heads_per_key_value = 3
    assert library.mmh3_attention(0, 128, None, None, None, None, 8, 4, 1, ctypes.byref(layout),
                                  0.1, None) == invalid
    layout.heads_per_key_value = 0
    assert library.mmh3_attention(0, 96, None, None, None, None, 8, 4, 1, ctypes.byref(layout),
                                  0.1, None) == invalid
    assert library.mmh3_attention(1, 64, None, None, None, None, 8, 4, 1, ctypes.byref(layout),
                                  -0.1, None) == invalid  # the scale must be positive
    workspace = _lib.QuantizedWorkspaceStruct()
    layout.causal = 1
    assert library.mmh3_attention_quantized(None, None, None, None, 8, 1, ctypes.byref(layout),
                                            0.1, None, ctypes.byref(workspace), 0, None) == invalid
    layout.causal = 0
    assert library.mmh3_attention_quantized(None, None, None, None, -1, 1, ctypes.byref(layout),
                                            0.1, None, ctypes.byref(workspace), 0, None) == invalid
    vsa = _lib.VsaWorkspaceStruct()
    # kept < 1, prefix_tiles > tiles, quantized without prepared inputs
    assert library.mmh3_vsa_attention(None, None, None, None, 0, None, 8, 1, ctypes.byref(layout),
                                      0.1, 4, 1, 0, ctypes.byref(vsa), None, 0, None) == invalid
    assert library.mmh3_vsa_attention(None, None, None, None, 0, None, 8, 1, ctypes.byref(layout),
                                      0.1, 4, 5, 1, ctypes.byref(vsa), None, 0, None) == invalid
    assert library.mmh3_vsa_attention(None, None, None, None, 0, None, 8, 1, ctypes.byref(layout),
                                      0.1, 4, 1, 1, ctypes.byref(vsa), ctypes.byref(workspace), 0,
                                      None) == invalid
    assert library.mmh3_attention_inputs(None, None, None, None, 0, 8, 1, 1e-6, None, None, None,
                                         None, 0, None, None) == invalid
    assert library.mmh3_dit_shard_pack(None, None, 8, 3, 4, 100, 0, 2, None) == invalid
    # The gathers move 16-byte groups: a pointer off that boundary is refused on the host.
    even, odd = ctypes.c_void_p(4096), ctypes.c_void_p(4096 + 8)
    assert library.mmh3_dit_shard_pack(odd, even, 8, 3, 4, 128, 0, 2, None) == invalid
    assert library.mmh3_dit_shard_pack(even, odd, 8, 3, 4, 128, 0, 2, None) == invalid
    assert library.mmh3_dit_shard_unpack(odd, even, 8, 4, 128, 0, 2, None) == invalid
    assert library.mmh3_dit_shard_unpack(even, odd, 8, 4, 128, 0, 2, None) == invalid
    assert library.mmh3_dit_shard_unpack(even, even, 8, 4, 128, 3, 2, None) == invalid
    # no workspace, no tokens
    assert library.mmh3_sparse_attention(None, None, None, None, 8, 1, ctypes.byref(layout), 0.1,
                                         0.5, 0, 0, 0, 0, None, None, 0, None) == invalid
    sol = _lib.SparseWorkspace()
    assert library.mmh3_sparse_attention(None, None, None, None, 0, 1, ctypes.byref(layout), 0.1,
                                         0.5, 0, 0, 0, 0, ctypes.byref(sol), None, 0,
                                         None) == invalid


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_library", None)
    monkeypatch.setattr(_lib, "LIBRARY", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.library()


def test_gemm_arguments_are_rejected_before_any_launch():
    # crates/mmh3-cuda/kernels/int8_gemm.cu:640-645, 710, 720, 919-921
    library = _lib.library()
    invalid = _lib.CUDA_ERROR_INVALID_VALUE
    assert library.mmh3_int8_gemm_config_count() == 2
    heights = (ctypes.c_int * 2)()
    assert library.mmh3_int8_gemm_group_heights(heights, 2) == 3 and list(heights) == [4, 8]
    operand = ctypes.c_void_p(4096)  # never dereferenced: every call below fails its checks

    def call(config=0, group_m=8, m=64, n=256, k=256, f16=0, swiglu=0, down=None, maxima=None,
             first_column=0, activations=operand):
        return library.mmh3_int8_gemm(config, group_m, activations, operand, operand, operand,
                                      None, operand, f16, swiglu, m, n, k, 0, down, None, 0, 0,
                                      0.0, maxima, first_column, None)

    assert call(activations=None) == invalid
    assert call(n=192) == invalid
    assert call(config=1, n=384) == invalid
    assert call(k=100) == invalid
    assert call(m=0) == invalid
    assert call(group_m=0) == invalid
    assert call(config=2) == invalid
    assert call(maxima=operand, f16=1) == invalid
    assert call(maxima=operand, swiglu=1) == invalid
    assert call(maxima=operand, first_column=64) == invalid
    # Nothing is ever chosen, and what the reference's search saved is not adopted.
    assert library.mmh3_int8_gemm_tilings(None, 0) == 0
    library.mmh3_int8_gemm_adopt.restype = None
    library.mmh3_int8_gemm_adopt(None, 0)
    assert library.mmh3_interleave_swiglu_rows(operand, operand, 12, 256, None) == invalid
    assert library.mmh3_interleave_swiglu_rows(operand, operand, 16, 6, None) == invalid
