"""Attention over the DiT's fused qkv projection output, through the library's C ABI.

The functions and workspaces here mirror the safe wrappers of niw/mmh3's CUDA crate
(crates/mmh3-cuda/src/attention.rs): the same names, argument meaning, buffer sizes and bounds
checks, with `torch` tensors standing where the crate has `DeviceBuffer`s. Every call goes through
`extern "C"` entry points with raw device pointers; torch only owns the memory and the stream.
A failing call raises `CudaError` with the cudaError_t the entry point returned.
"""

from __future__ import annotations

import ctypes
import enum

import torch

from . import _lib
from .vsa import VSA_TILE, VsaPlan

HEAD_DIM = 128
SPARSE_BLOCK = 64


class CudaError(RuntimeError):
    def __init__(self, code: int, call: str):
        super().__init__(f"{call} returned cudaError {code}")
        self.code = code


def check(code: int, call: str) -> None:
    if code != 0:
        raise CudaError(code, call)


class AttentionInputs(enum.IntEnum):
    """Where the attention finds its per-block inputs (attention.rs:495-514)."""

    RAW = 0
    PREPARED = 1
    PREPARED_WITH_VALUES = 2


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _pointer(tensor: torch.Tensor | None, offset_elements: int = 0) -> ctypes.c_void_p:
    if tensor is None:
        return ctypes.c_void_p(0)
    assert tensor.is_cuda and tensor.is_contiguous()
    return ctypes.c_void_p(tensor.data_ptr() + offset_elements * tensor.element_size())


def make_layout(token_stride, head_stride=(HEAD_DIM,) * 4, batch_stride=(0,) * 4,
                heads_per_key_value: int = 0, causal: int = 0) -> _lib.AttentionLayout:
    layout = _lib.AttentionLayout()
    for index in range(4):
        layout.token_stride[index] = token_stride[index]
        layout.head_stride[index] = head_stride[index]
        layout.batch_stride[index] = batch_stride[index]
    layout.heads_per_key_value = heads_per_key_value
    layout.causal = causal
    return layout


def qkv_layout(heads: int) -> _lib.AttentionLayout:
    """The DiT's layout: qkv [tokens, 3, heads, 128] and output [tokens, heads, 128]."""
    inner = heads * HEAD_DIM
    return make_layout((3 * inner, 3 * inner, 3 * inner, inner))


def take_status() -> int:
    """Synchronizes and returns the kernels' status word: 0 unless a bounded wait ran out."""
    return _lib.library().mmh3_b200_take_status()


# -------------------------------------------------------------------------------------------------
# Dense BF16


def attention(element_type: int, head_dim: int, query: torch.Tensor, key: torch.Tensor,
              value: torch.Tensor, output: torch.Tensor, tokens: int, heads: int, batch: int,
              layout: _lib.AttentionLayout, scale: float, offsets=(0, 0, 0, 0)) -> None:
    """Softmax attention over tensors described by `layout` (attention.rs:371-435).

    `query`, `key`, `value` and `output` are the buffers the operands live in, each starting
    `offsets[i]` elements in. Every addressed element must lie inside its buffer.
    """
    group = max(layout.heads_per_key_value, 1)
    if heads % group != 0:
        raise ValueError("heads must be a multiple of the heads per key and value head")
    buffers = (query, key, value, output)
    for operand in range(4):
        operand_heads = heads // group if operand in (1, 2) else heads
        last = (offsets[operand] + (batch - 1) * layout.batch_stride[operand]
                + (tokens - 1) * layout.token_stride[operand]
                + (operand_heads - 1) * layout.head_stride[operand] + head_dim)
        if last > buffers[operand].numel():
            raise ValueError(f"operand {operand} reaches past its buffer")
    check(
        _lib.library().mmh3_attention(
            element_type, head_dim, _pointer(query, offsets[0]), _pointer(key, offsets[1]),
            _pointer(value, offsets[2]), _pointer(output, offsets[3]), tokens, heads, batch,
            ctypes.byref(layout), scale, _stream()),
        "mmh3_attention",
    )


def attention_roped(element_type: int, head_dim: int, query: torch.Tensor, key: torch.Tensor,
                    value: torch.Tensor, output: torch.Tensor, tokens: int, heads: int, batch: int,
                    layout: _lib.AttentionLayout, scale: float, angles: torch.Tensor, pairs: int,
                    epsilon: float) -> None:
    """`attention` with the query's RMS norm and RoPE fused in, as the video VAE's decoder calls it
    (attention.rs:437-500): `angles` is FP32 [tokens, pairs]; dimension p pairs with p + pairs."""
    if angles.dtype != torch.float32 or angles.numel() < tokens * pairs:
        raise ValueError("angles must be FP32 [tokens, pairs]")
    if 2 * pairs > head_dim:
        raise ValueError("more rotary pairs than half the head dimension")
    check(
        _lib.library().mmh3_attention_roped(
            element_type, head_dim, _pointer(query), _pointer(key), _pointer(value),
            _pointer(output), tokens, heads, batch, ctypes.byref(layout), scale,
            _pointer(angles), pairs, epsilon, _stream()),
        "mmh3_attention_roped",
    )


def dense_bf16(qkv: torch.Tensor, output: torch.Tensor, tokens: int, heads: int,
               scale: float) -> None:
    """Dense bidirectional attention with head dimension 128 (attention.rs:469-493).

    `qkv` is BF16 [tokens, 3, heads, 128] as the fused projection leaves it and `output` receives
    BF16 [tokens, heads, 128].
    """
    inner = heads * HEAD_DIM
    if qkv.numel() < tokens * 3 * inner:
        raise ValueError("qkv is smaller than tokens x 3 x heads x 128")
    if output.numel() < tokens * inner:
        raise ValueError("output is smaller than tokens x heads x 128")
    assert qkv.dtype == torch.bfloat16 and output.dtype == torch.bfloat16
    check(
        _lib.library().mmh3_attention_bf16(
            _pointer(qkv), _pointer(qkv, inner), _pointer(qkv, 2 * inner), _pointer(output),
            tokens, heads, 3 * inner, 3 * inner, 3 * inner, inner, scale, _stream()),
        "mmh3_attention_bf16",
    )


class HostPipeline:
    """Dense BF16 attention from pinned host buffers to pinned host buffers, for hosts that keep
    activations off the device between layers.

    Heads are independent, so the sequence of copy in, attention and copy out is run per group of
    heads on three streams: while one group is attended, the next one's q, k and v cross the bus
    and the last one's output goes back. Each group's rows are strided in the fused layouts
    ([tokens, 3, heads, 128] and [tokens, heads, 128]), which a 2D copy describes, and the entry
    point takes a group as a pointer offset with the same strides. The copies go through
    cuda-python's runtime binding; torch owns the buffers and the streams.

    Nothing hides the first group's way in and the last group's way out, so those two groups are
    one head each; a group's copy in must fit behind the attention of the group before, and a
    head's rows cross the bus in about half the time the kernel needs for them, so with
    `groups = 0` every group is at most twice the one before (1, 2, 4, 8, 16, 1 of 32 heads);
    and the groups' kernels alternate between two streams, so that the first blocks of one fill
    the multiprocessors the last blocks of the one before leave idle.
    """

    def __init__(self, tokens: int, heads: int, groups: int = 0, growth: float = 2.0):
        from cuda.bindings import runtime

        self.runtime = runtime
        self.tokens, self.heads = tokens, heads
        from .shard import group_sizes, growing_sizes

        self.groups = []
        first = 0
        sizes = (growing_sizes(heads, growth) if groups <= 0
                 else group_sizes(heads, min(groups, heads), ramped=True))
        for span in sizes:
            if span:
                self.groups.append((first, span))
                first += span
        self.copy_in, self.copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.second = torch.cuda.Stream()
        self.arrived = [torch.cuda.Event() for _ in self.groups]
        self.attended = [torch.cuda.Event() for _ in self.groups]
        self.finished = torch.cuda.Event()

    def copy_rows(self, destination: int, source: int, pitch: int, width: int, rows: int,
                  to_device: bool, stream: torch.cuda.Stream) -> None:
        """`rows` runs of `width` bytes, `pitch` bytes apart on both sides, on `stream`."""
        kind = (self.runtime.cudaMemcpyKind.cudaMemcpyHostToDevice if to_device
                else self.runtime.cudaMemcpyKind.cudaMemcpyDeviceToHost)
        (code,) = self.runtime.cudaMemcpy2DAsync(destination, pitch, source, pitch, width, rows,
                                                 kind, stream.cuda_stream)
        check(int(code), "cudaMemcpy2DAsync")

    def run(self, host_qkv: torch.Tensor, qkv: torch.Tensor, output: torch.Tensor,
            host_output: torch.Tensor, scale: float) -> None:
        """Enqueues everything and returns; the current stream ends up behind the last copy."""
        tokens, heads = self.tokens, self.heads
        inner = heads * HEAD_DIM
        if min(host_qkv.numel(), qkv.numel()) < tokens * 3 * inner or \
                min(host_output.numel(), output.numel()) < tokens * inner:
            raise ValueError("a buffer is smaller than the sequence")
        if not (host_qkv.is_pinned() and host_output.is_pinned()):
            raise ValueError("the host buffers must be pinned")
        current = torch.cuda.current_stream()
        # What the last call left running on the device buffers comes first.
        self.copy_in.wait_stream(current)
        self.copy_out.wait_stream(current)
        self.second.wait_stream(current)
        pitch = inner * 2
        for index, (first, span) in enumerate(self.groups):
            offset = first * HEAD_DIM * 2
            self.copy_rows(qkv.data_ptr() + offset, host_qkv.data_ptr() + offset, pitch,
                           span * HEAD_DIM * 2, tokens * 3, True, self.copy_in)
            self.arrived[index].record(self.copy_in)
        for index, (first, span) in enumerate(self.groups):
            stream = self.second if index % 2 else current
            stream.wait_event(self.arrived[index])
            offset = first * HEAD_DIM
            check(
                _lib.library().mmh3_attention_bf16(
                    _pointer(qkv, offset), _pointer(qkv, inner + offset),
                    _pointer(qkv, 2 * inner + offset), _pointer(output, offset), tokens, span,
                    3 * inner, 3 * inner, 3 * inner, inner, scale,
                    ctypes.c_void_p(stream.cuda_stream)),
                "mmh3_attention_bf16",
            )
            self.attended[index].record(stream)
            self.copy_out.wait_event(self.attended[index])
            self.copy_rows(host_output.data_ptr() + offset * 2, output.data_ptr() + offset * 2,
                           pitch, span * HEAD_DIM * 2, tokens, False, self.copy_out)
        self.finished.record(self.copy_out)
        current.wait_event(self.finished)
        current.wait_stream(self.second)


# -------------------------------------------------------------------------------------------------
# Quantized


class QuantizedWorkspace:
    """Scratch for one sequence of INT8/FP8 attention, reused across layers (attention.rs:61-140)."""

    def __init__(self, tokens: int, heads: int, blocks: int | None = None, device="cuda"):
        if not (0 < tokens <= 2**31 - 64 and 0 < heads <= 65535):
            raise ValueError("invalid attention shape")
        self.tokens, self.heads = tokens, heads
        self.blocks = blocks if blocks is not None else -(-tokens // SPARSE_BLOCK)
        rows = tokens * heads * HEAD_DIM
        byte = dict(dtype=torch.uint8, device=device)
        real = dict(dtype=torch.float32, device=device)
        self.query = torch.empty(rows, **byte)
        self.key = torch.empty(rows, **byte)
        self.value = torch.empty(self.blocks * SPARSE_BLOCK * heads * HEAD_DIM, **byte)
        self.query_scales = torch.empty(heads * self.blocks, **real)
        self.key_scales = torch.empty(heads * self.blocks, **real)
        self.value_scales = torch.empty(heads, **real)
        self.value_maxima = torch.empty(heads * self.blocks, **real)
        self.value_head_maxima = torch.zeros(heads, **real)

    def raw(self) -> _lib.QuantizedWorkspaceStruct:
        return _lib.QuantizedWorkspaceStruct(
            self.query.data_ptr(), self.key.data_ptr(), self.value.data_ptr(),
            self.query_scales.data_ptr(), self.key_scales.data_ptr(),
            self.value_scales.data_ptr(), self.value_maxima.data_ptr())


def dense_quantized(qkv: torch.Tensor, output: torch.Tensor, scale: float,
                    workspace: QuantizedWorkspace,
                    inputs: AttentionInputs = AttentionInputs.RAW) -> None:
    """Dense attention with INT8 QK and FP8 PV (attention.rs:778-817)."""
    tokens, heads = workspace.tokens, workspace.heads
    inner = heads * HEAD_DIM
    if qkv.numel() < tokens * 3 * inner or output.numel() < tokens * inner:
        raise ValueError("qkv or output is smaller than the workspace's sequence")
    layout = qkv_layout(heads)
    raw = workspace.raw()
    check(
        _lib.library().mmh3_attention_quantized(
            _pointer(qkv), _pointer(qkv, inner), _pointer(qkv, 2 * inner), _pointer(output),
            tokens, heads, ctypes.byref(layout), scale, None, ctypes.byref(raw), int(inputs),
            _stream()),
        "mmh3_attention_quantized",
    )


def dense_quantized_static(qkv: torch.Tensor, output: torch.Tensor, tokens: int, heads: int,
                           scale: float) -> None:
    """`dense_quantized` from raw BF16 inputs without a workspace: the scratch is a fixed array
    inside the library, for callers that cannot allocate device memory. Shapes past the array's
    size (tokens rounded up to 64, times heads, at most 32,768; at most 64 heads) are refused.
    Calls on one device share the array, so overlapping calls on different streams race."""
    inner = heads * HEAD_DIM
    if qkv.numel() < tokens * 3 * inner or output.numel() < tokens * inner:
        raise ValueError("qkv or output is smaller than tokens x heads x 128")
    layout = qkv_layout(heads)
    check(
        _lib.library().mmh3_b200_attention_quantized_static(
            _pointer(qkv), _pointer(qkv, inner), _pointer(qkv, 2 * inner), _pointer(output),
            tokens, heads, ctypes.byref(layout), scale, _stream()),
        "mmh3_b200_attention_quantized_static",
    )


class HeadNorm:
    """Per-head RMSNorm weights of q and k and the rotary angles of every token."""

    def __init__(self, query_weight: torch.Tensor, key_weight: torch.Tensor,
                 angles: torch.Tensor | None, pairs: int, epsilon: float):
        if query_weight.numel() < HEAD_DIM or key_weight.numel() < HEAD_DIM:
            raise ValueError("the norm weights hold 128 BF16 values")
        if 2 * pairs > HEAD_DIM:
            raise ValueError("the rotary pairs exceed the head")
        self.query_weight, self.key_weight = query_weight, key_weight
        self.angles, self.pairs, self.epsilon = angles, pairs, epsilon

    def check(self, qkv: torch.Tensor, tokens: int, heads: int) -> None:
        if qkv.numel() < tokens * 3 * heads * HEAD_DIM:
            raise ValueError("qkv is smaller than tokens x 3 x heads x 128")
        if self.angles is not None and self.angles.numel() < tokens * self.pairs:
            raise ValueError("the angles do not cover every token")


def qk_norm_rope(qkv: torch.Tensor, norm: HeadNorm, tokens: int, heads: int) -> None:
    """Per-head RMSNorm of q and k in [tokens, 3, heads, 128] rows, then RoPE, in place."""
    norm.check(qkv, tokens, heads)
    check(
        _lib.library().mmh3_qk_norm_rope(
            _pointer(qkv), _pointer(norm.query_weight), _pointer(norm.key_weight),
            _pointer(norm.angles), norm.pairs, tokens, heads, heads, norm.epsilon, _stream()),
        "mmh3_qk_norm_rope",
    )


# -------------------------------------------------------------------------------------------------
# Video sparse attention


class VsaWorkspace:
    """The tiles of one VSA plan and scratch for its sequence and heads (attention.rs:975-1110)."""

    def __init__(self, plan: VsaPlan, tokens: int, heads: int, quantized: bool = False,
                 device="cuda"):
        tiles = plan.tiles
        if not 0 < tiles <= 65536:
            raise ValueError(f"invalid tile count {tiles}")
        if not all(1 <= length <= VSA_TILE for length in plan.tile_lengths) or not all(
                start + length <= tokens
                for start, length in zip(plan.tile_starts, plan.tile_lengths)):
            raise ValueError("the plan's tiles do not fit the sequence")
        self.tokens, self.heads, self.tiles = tokens, heads, tiles
        self.prefix_tiles = plan.prefix_tiles
        self.quantized = (QuantizedWorkspace(tokens, heads, blocks=tiles, device=device)
                          if quantized else None)
        self.tile_starts = torch.tensor(plan.tile_starts, dtype=torch.int32, device=device)
        self.tile_lengths = torch.tensor(plan.tile_lengths, dtype=torch.int32, device=device)
        per_tile = heads * tiles * HEAD_DIM
        real = dict(dtype=torch.float32, device=device)
        self.pooled_query = torch.empty(per_tile, **real)
        self.pooled_key = torch.empty(per_tile, **real)
        self.pooled_value = torch.empty(per_tile, **real)
        self.routes = torch.empty(heads * tiles * tiles, dtype=torch.int16, device=device)
        self.route_counts = torch.zeros(heads * tiles, dtype=torch.int32, device=device)
        self.coarse = torch.empty(per_tile, **real)

    def raw(self) -> _lib.VsaWorkspaceStruct:
        return _lib.VsaWorkspaceStruct(
            self.tile_starts.data_ptr(), self.tile_lengths.data_ptr(),
            self.pooled_query.data_ptr(), self.pooled_key.data_ptr(),
            self.pooled_value.data_ptr(), self.routes.data_ptr(), self.route_counts.data_ptr(),
            self.coarse.data_ptr())

    def sparse_raw(self) -> _lib.SparseWorkspace:
        """The pooled buffers under the names the fused input pass writes them by."""
        workspace = _lib.SparseWorkspace()
        workspace.centroids = self.pooled_query.data_ptr()
        workspace.block_keys = self.pooled_key.data_ptr()
        workspace.value_sums = self.pooled_value.data_ptr()
        return workspace

    def selected_fraction(self) -> float:
        """Mean fraction of the tiles the query tiles of the last call attended token by token."""
        selected = int(self.route_counts.to(torch.int64).sum().item())
        return selected / (self.heads * self.tiles * self.tiles)

    def route_overlap(self) -> tuple[int, float, float]:
        """How much neighbouring query tiles share (attention.rs:1005-1048): the pairs (2i, 2i + 1)
        with any selection, the mean number of tiles the two load between them, and the mean
        number of distinct tiles, which is what one block over both rows loads. A diagnostic, not
        a hot path; the token attention's CTAs take exactly these pairs."""
        tiles, heads = self.tiles, self.heads
        counts = self.route_counts.view(heads, tiles).to(torch.int64)
        routes = self.routes.view(heads, tiles, tiles).to(torch.int64) & 0xFFFF
        entries = torch.arange(tiles, device=routes.device)
        pairs, separate, merged = 0, 0.0, 0.0
        even = tiles - tiles % 2
        for head in range(heads):
            listed = entries[None, :] < counts[head][:, None]
            selected = torch.zeros((tiles, tiles + 1), dtype=torch.bool, device=routes.device)
            # Entries past a row's count, and targets past the last tile, go to a spare column.
            targets = torch.where(listed & (routes[head] < tiles), routes[head],
                                  torch.full_like(routes[head], tiles))
            selected.scatter_(1, targets, True)
            selected = selected[:even, :tiles]
            both = counts[head][:even].view(-1, 2).sum(dim=1)
            some = both > 0
            pairs += int(some.sum().item())
            separate += float(both[some].sum().item())
            merged += float((selected[0::2] | selected[1::2])[some].sum().item())
        if pairs:
            separate /= pairs
            merged /= pairs
        return pairs, separate, merged

    def routes_host(self):
        """Routes [heads, tiles, tiles] as uint16 and counts [heads, tiles], on the host."""
        routes = self.routes.cpu().numpy().view("uint16").reshape(self.heads, self.tiles,
                                                                 self.tiles)
        counts = self.route_counts.cpu().numpy().reshape(self.heads, self.tiles)
        return routes, counts


def prepare_inputs(qkv: torch.Tensor, norm: HeadNorm, tokens: int, heads: int,
                   quantized: QuantizedWorkspace | None = None, vsa: VsaWorkspace | None = None,
                   value_head_maxima: torch.Tensor | None = None, sol=None) -> None:
    """qk_norm_rope fused with the attention's per-block work (attention.rs:670-760).

    With `vsa`, the blocks are its tiles, its pooled buffers are filled, and its own quantized
    workspace (if any) is used. With `sol` (a `SparseWorkspace`), the block statistics of Sol-Attn
    are filled over blocks of 64 tokens.
    """
    norm.check(qkv, tokens, heads)
    if vsa is not None and vsa.quantized is not None:
        quantized = vsa.quantized
    if sol is not None and sol.quantized is not None:
        quantized = sol.quantized
    sparse = vsa.sparse_raw() if vsa is not None else (sol.raw() if sol is not None else None)
    raw = quantized.raw() if quantized is not None else None
    check(
        _lib.library().mmh3_attention_inputs(
            _pointer(qkv), _pointer(norm.query_weight), _pointer(norm.key_weight),
            _pointer(norm.angles), norm.pairs, tokens, heads, norm.epsilon,
            ctypes.byref(sparse) if sparse is not None else None,
            ctypes.byref(raw) if raw is not None else None,
            _pointer(vsa.tile_starts) if vsa is not None else None,
            _pointer(vsa.tile_lengths) if vsa is not None else None,
            vsa.tiles if vsa is not None else 0, _pointer(value_head_maxima), _stream()),
        "mmh3_attention_inputs",
    )


def vsa(qkv: torch.Tensor, gate: torch.Tensor | None, output: torch.Tensor,
        layout: _lib.AttentionLayout, scale: float, kept: int, workspace: VsaWorkspace,
        inputs: AttentionInputs = AttentionInputs.RAW, offsets=None) -> None:
    """VSA over BF16 heads of 128 in the workspace's tile order (attention.rs:1189-1250).

    `gate`, BF16 [tokens, heads, 128], adds the coarse branch.
    """
    tokens, heads = workspace.tokens, workspace.heads
    inner = heads * HEAD_DIM
    if offsets is None:
        offsets = (0, inner, 2 * inner, 0)
    for operand in range(4):
        buffer = output if operand == 3 else qkv
        last = (offsets[operand] + (tokens - 1) * layout.token_stride[operand]
                + (heads - 1) * layout.head_stride[operand] + HEAD_DIM)
        if last > buffer.numel():
            raise ValueError(f"operand {operand} reaches past its buffer")
    if gate is not None and gate.numel() < tokens * inner:
        raise ValueError("the gate is smaller than tokens x heads x 128")
    if workspace.quantized is not None and inputs == AttentionInputs.RAW:
        raise ValueError("quantized VSA needs prepared inputs")
    raw = workspace.raw()
    quantized = workspace.quantized.raw() if workspace.quantized is not None else None
    check(
        _lib.library().mmh3_vsa_attention(
            _pointer(qkv, offsets[0]), _pointer(qkv, offsets[1]), _pointer(qkv, offsets[2]),
            _pointer(gate), inner, _pointer(output, offsets[3]), tokens, heads,
            ctypes.byref(layout), scale, workspace.tiles, workspace.prefix_tiles, kept,
            ctypes.byref(raw), ctypes.byref(quantized) if quantized is not None else None,
            int(inputs), _stream()),
        "mmh3_vsa_attention",
    )


# -------------------------------------------------------------------------------------------------
# Sol-Attn


class SparseSinks:
    """Block ranges [start, end) that are always exact (mmh3-core/src/dit/sparse.rs:79-101):
    `key_blocks` every query attends token by token, `query_blocks` attend every key so."""

    def __init__(self, key_blocks=(0, 0), query_blocks=(0, 0)):
        self.key_blocks = tuple(key_blocks)
        self.query_blocks = tuple(query_blocks)

    @classmethod
    def for_layout(cls, layout) -> "SparseSinks":
        """H3's conditioning: every query attends the text and audio prefix exactly, and the audio
        queries run dense. `layout` is a `vsa.PackedLayout`."""
        video, audio = layout.segment("video"), layout.segment("audio")
        prefix_blocks = -(-video.start // SPARSE_BLOCK)
        return cls((0, prefix_blocks), (audio.start // SPARSE_BLOCK, prefix_blocks))

    def __eq__(self, other):
        return (self.key_blocks, self.query_blocks) == (other.key_blocks, other.query_blocks)

    def __repr__(self):
        return f"SparseSinks(key_blocks={self.key_blocks}, query_blocks={self.query_blocks})"


class SparseWorkspace:
    """Scratch buffers of Sol-Attn for one sequence length and head count (attention.rs:818-908).
    Routing and the pooled tail are BF16/FP32 either way; `quantized` adds the INT8/FP8 workspace
    of the routed products (`SparseWorkspace::with_precision`)."""

    def __init__(self, tokens: int, heads: int, quantized: bool = False, device="cuda"):
        blocks = -(-tokens // SPARSE_BLOCK)
        if not 0 < blocks <= 65535:
            raise ValueError(f"invalid block count {blocks}")
        self.tokens, self.heads, self.blocks = tokens, heads, blocks
        self.quantized = QuantizedWorkspace(tokens, heads, device=device) if quantized else None
        per_block = heads * blocks * HEAD_DIM
        real = dict(dtype=torch.float32, device=device)
        self.centroids = torch.empty(per_block, **real)
        self.block_keys = torch.empty(per_block, **real)
        self.value_sums = torch.empty(per_block, **real)
        self.key_mean = torch.empty(heads * HEAD_DIM, **real)
        self.key_variance = torch.empty(heads * HEAD_DIM, **real)
        self.row_offsets = torch.empty(heads * tokens, **real)
        self.routes = torch.empty(heads * blocks * blocks, dtype=torch.int16, device=device)
        self.route_counts = torch.zeros(heads * blocks, dtype=torch.int32, device=device)
        self.tail_max = torch.empty(heads * blocks, **real)
        self.tail_sum = torch.empty(heads * blocks, **real)
        self.tail_values = torch.empty(per_block, **real)

    def raw(self) -> _lib.SparseWorkspace:
        workspace = _lib.SparseWorkspace()
        for name, _ in _lib.SparseWorkspace._fields_:
            setattr(workspace, name, getattr(self, name).data_ptr())
        return workspace

    def routed_fraction(self) -> float:
        """Fraction of (head, query block, key block) triples the last call routed token by
        token."""
        routed = int(self.route_counts.to(torch.int64).sum().item())
        return routed / (self.heads * self.blocks * self.blocks)

    def routes_host(self):
        """Routes [heads, blocks, blocks] as uint16 and counts [heads, blocks], on the host."""
        routes = self.routes.cpu().numpy().view("uint16").reshape(self.heads, self.blocks,
                                                                 self.blocks)
        counts = self.route_counts.cpu().numpy().reshape(self.heads, self.blocks)
        return routes, counts


def sparse(qkv: torch.Tensor, output: torch.Tensor, layout: _lib.AttentionLayout, scale: float,
           tau: float, sinks: SparseSinks, workspace: SparseWorkspace,
           inputs: AttentionInputs = AttentionInputs.RAW, offsets=None) -> None:
    """Sol-Attn over BF16 heads of 128 for one sequence (attention.rs:1253-1306). With prepared
    inputs the workspace already holds the block statistics (`prepare_inputs(..., sol=...)`)."""
    tokens, heads = workspace.tokens, workspace.heads
    inner = heads * HEAD_DIM
    if offsets is None:
        offsets = (0, inner, 2 * inner, 0)
    for operand in range(4):
        buffer = output if operand == 3 else qkv
        last = (offsets[operand] + (tokens - 1) * layout.token_stride[operand]
                + (heads - 1) * layout.head_stride[operand] + HEAD_DIM)
        if last > buffer.numel():
            raise ValueError(f"operand {operand} reaches past its buffer")
    raw = workspace.raw()
    quantized = workspace.quantized.raw() if workspace.quantized is not None else None
    check(
        _lib.library().mmh3_sparse_attention(
            _pointer(qkv, offsets[0]), _pointer(qkv, offsets[1]), _pointer(qkv, offsets[2]),
            _pointer(output, offsets[3]), tokens, heads, ctypes.byref(layout), scale, tau,
            sinks.key_blocks[0], sinks.key_blocks[1], sinks.query_blocks[0],
            sinks.query_blocks[1], ctypes.byref(raw),
            ctypes.byref(quantized) if quantized is not None else None, int(inputs), _stream()),
        "mmh3_sparse_attention",
    )


# -------------------------------------------------------------------------------------------------
# Ulysses layout changes


def shard_pack(source: torch.Tensor, packed: torch.Tensor, tokens: int, tensors: int, heads: int,
               first_head: int, span: int, dim: int = HEAD_DIM) -> None:
    """[tokens][tensors][heads][dim] -> [tokens][tensors][span][dim] at `first_head`."""
    if source.numel() < tokens * tensors * heads * dim or packed.numel() < tokens * tensors * span * dim:
        raise ValueError("a buffer is smaller than its shape")
    check(
        _lib.library().mmh3_dit_shard_pack(_pointer(source), _pointer(packed), tokens, tensors,
                                           heads, dim, first_head, span, _stream()),
        "mmh3_dit_shard_pack",
    )


def shard_unpack(part: torch.Tensor, output: torch.Tensor, tokens: int, heads: int,
                 first_head: int, span: int, dim: int = HEAD_DIM) -> None:
    """[tokens][span][dim] -> [tokens][heads][dim] at `first_head`."""
    if part.numel() < tokens * span * dim or output.numel() < tokens * heads * dim:
        raise ValueError("a buffer is smaller than its shape")
    check(
        _lib.library().mmh3_dit_shard_unpack(_pointer(part), _pointer(output), tokens, heads, dim,
                                             first_head, span, _stream()),
        "mmh3_dit_shard_unpack",
    )
