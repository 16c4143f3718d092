"""The Ulysses head gathers on a B200, and a split run against a whole one on a single GPU.

The reference refuses to trust a sharded step until `check_layout` has pushed non-repeating 16-bit
patterns through `mmh3_dit_shard_pack` / `mmh3_dit_shard_unpack`, past the point where a gather
without a grid stride would leave values behind (crates/mmh3-cuda/src/shard.rs:194-281,
src/bin/mmh3-tools/check.rs:34-48), and until a run split across ranks equals the unsplit one
(check.rs:312-349, 547-647: its in-process split stages every rank's data through one process).
Both are mirrored here through the C ABI: the gathers against a torch gather and against the
reference's own kernels, and "virtual ranks" on one GPU, where each rank's chunks are placed
where the all-to-all would have put them, against one dense call over every head.
"""

import pytest
import torch

from mmh3_b200 import _lib, attention, synthetic
from mmh3_b200.shard import Shard, UlyssesAttention

pytestmark = pytest.mark.gpu

SCALE = synthetic.softmax_scale()


def pattern(count: int) -> torch.Tensor:
    """16-bit values that differ in every position a gather could confuse: a step of 40503 walks
    the whole 16-bit range without repeating (shard.rs:199-201)."""
    index = torch.arange(count, dtype=torch.int64, device="cuda")
    return ((index * 40503) & 0xFFFF).to(torch.int16)


def pack_with(library, source, packed, tokens, tensors, heads, dim, first_head, span):
    assert library.mmh3_dit_shard_pack(source.data_ptr(), packed.data_ptr(), tokens, tensors,
                                       heads, dim, first_head, span, None) == 0


def unpack_with(library, part, output, tokens, heads, dim, first_head, span):
    assert library.mmh3_dit_shard_unpack(part.data_ptr(), output.data_ptr(), tokens, heads, dim,
                                         first_head, span, None) == 0


# (tokens, tensors, heads, dim, first_head, span). The second is the reference's default check,
# whose 3.7 million 16-byte groups are several times what one wave of this library's grid covers,
# so the grid-stride loop is taken; the last two are uneven spans at either end of the heads and a
# head dimension of 64.
CASES = [
    (1, 1, 2, 128, 1, 1),
    (2731, 3, 56, 128, 28, 28),
    (2731, 1, 56, 128, 28, 28),
    (1000, 3, 32, 128, 0, 10),
    (1000, 3, 32, 128, 20, 12),
    (517, 4, 7, 64, 2, 3),
]


@pytest.mark.parametrize("tokens,tensors,heads,dim,first_head,span", CASES)
def test_pack_and_unpack_move_every_value(reference_kernels, tokens, tensors, heads, dim,
                                          first_head, span):
    ours = _lib.library()
    source = pattern(tokens * tensors * heads * dim)
    expected = source.view(tokens, tensors, heads, dim)[:, :, first_head:first_head + span]
    packed = torch.zeros(tokens * tensors * span * dim, dtype=torch.int16, device="cuda")
    theirs = torch.zeros_like(packed)
    pack_with(ours, source, packed, tokens, tensors, heads, dim, first_head, span)
    pack_with(reference_kernels, source, theirs, tokens, tensors, heads, dim, first_head, span)
    torch.cuda.synchronize()
    assert torch.equal(packed.view(tokens, tensors, span, dim), expected)
    assert torch.equal(packed, theirs)

    part = pattern(tokens * span * dim)
    # Heads outside the span belong to another rank and must stay untouched: fill them with a
    # sentinel no pattern value takes at that place.
    output = torch.full((tokens, heads, dim), 0x5A5A, dtype=torch.int16, device="cuda")
    theirs = output.clone()
    wanted = output.clone()
    wanted[:, first_head:first_head + span] = part.view(tokens, span, dim)
    unpack_with(ours, part, output, tokens, heads, dim, first_head, span)
    unpack_with(reference_kernels, part, theirs, tokens, heads, dim, first_head, span)
    torch.cuda.synchronize()
    assert torch.equal(output, wanted)
    assert torch.equal(output, theirs)


def test_a_packed_span_unpacks_to_itself():
    """pack then unpack of every span of an uneven cut rebuilds the source, one tensor at a
    time."""
    tokens, heads, dim = 777, 11, 128
    source = pattern(tokens * heads * dim)
    rebuilt = torch.zeros_like(source)
    for first_head, span in ((0, 3), (3, 3), (6, 5)):
        packed = torch.empty(tokens * span * dim, dtype=torch.int16, device="cuda")
        attention.shard_pack(source, packed, tokens, 1, heads, first_head, span, dim)
        attention.shard_unpack(packed, rebuilt, tokens, heads, first_head, span, dim)
    torch.cuda.synchronize()
    assert torch.equal(rebuilt, source)


def dense(qkv, output, tokens, heads):
    attention.dense_bf16(qkv, output, tokens, heads, SCALE)


@pytest.mark.parametrize("ranks", [2, 3, 8])
def test_virtual_ranks_equal_one_dense_call(ranks):
    """Every rank's `UlyssesAttention` steps run in one process on one GPU, with the two
    all-to-alls replaced by copies of each sent chunk to where NCCL would deliver it. The rows
    every rank ends up with must be the bits of one dense call over all heads: the kernel works a
    head at a time, so neither the head count of a launch nor its token stride may change a bit.
    Cuts are uneven at three ranks (10, 10 and 12 heads; the last rank takes the token
    remainder)."""
    tokens, heads = 1000, 32
    qkv = synthetic.dense_qkv(tokens, heads, seed=21).cuda()
    whole = torch.zeros((tokens, heads, 128), dtype=torch.bfloat16, device="cuda")
    dense(qkv, whole, tokens, heads)

    layers = [UlyssesAttention(Shard.even(rank, ranks, tokens, heads), tokens, heads, dense,
                               "cuda", pack=attention.shard_pack, unpack=attention.shard_unpack)
              for rank in range(ranks)]
    # Step 1 on every rank: its tokens' heads gathered per peer.
    for layer in layers:
        own = layer.shard.own_tokens
        rows = qkv[own.start:own.stop].contiguous()
        offset = 0
        for peer, span in enumerate(layer.shard.heads):
            count = layer.input_send_splits[peer]
            attention.shard_pack(rows, layer.send_inputs[offset:offset + count], len(own), 3,
                                 heads, span.start, len(span))
            offset += count
    # The first all-to-all: chunk p of rank r's send buffer becomes chunk r of rank p's inputs.
    for receiver, layer in enumerate(layers):
        landed = 0
        for sender, peer in enumerate(layers):
            count = layer.input_recv_splits[sender]
            start = sum(peer.input_send_splits[:receiver])
            assert peer.input_send_splits[receiver] == count
            layer.inputs[landed:landed + count].copy_(peer.send_inputs[start:start + count])
            landed += count
        assert landed == layer.inputs.numel()
    # Step 2: every rank attends all tokens on its own heads, through the strides of its share.
    for layer in layers:
        dense(layer.inputs, layer.attended, tokens, layer.own_heads)
    # The second all-to-all, then the scatter into [own tokens, heads, 128].
    for receiver, layer in enumerate(layers):
        landed = 0
        for sender, peer in enumerate(layers):
            count = layer.output_recv_splits[sender]
            start = sum(peer.output_send_splits[:receiver])
            assert peer.output_send_splits[receiver] == count
            layer.received[landed:landed + count].copy_(peer.attended[start:start + count])
            landed += count
        own = layer.shard.own_tokens
        rows = torch.zeros((len(own), heads, 128), dtype=torch.bfloat16, device="cuda")
        offset = 0
        for peer, span in enumerate(layer.shard.heads):
            count = layer.output_recv_splits[peer]
            attention.shard_unpack(layer.received[offset:offset + count], rows, len(own), heads,
                                   span.start, len(span))
            offset += count
        torch.cuda.synchronize()
        assert torch.equal(rows, whole[own.start:own.stop]), f"rank {receiver} of {ranks}"
    assert attention.take_status() == 0
