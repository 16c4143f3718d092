"""The Ulysses partitioning and exchange on CPU ranks (gloo, world size 2 and 3), no GPU.

The attention itself is a plain torch softmax attention here: what is under test is that the cuts,
the packing, the two all-to-alls and the unpacking put every head's output back on the rank that
owns its tokens, for even and uneven cuts. A split run must equal a whole run, as the reference
checks its own split (crates/mmh3-cuda/src/shard.rs:52-56).
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mmh3_b200.shard import (OverlappedUlyssesAttention, ProjectedUlyssesAttention, Shard,
                              UlyssesAttention, group_sizes, growing_sizes, head_groups,
                              own_projection_rows)

HEAD_DIM = 128


def torch_attention(qkv, output, tokens, heads):
    view = qkv.view(tokens, 3, heads, HEAD_DIM).float()
    q, k, v = (view[:, part].transpose(0, 1) for part in range(3))
    result = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    output.view(tokens, heads, HEAD_DIM).copy_(result.transpose(0, 1).to(output.dtype))


def free_port():
    with socket.socket() as listener:
        listener.bind(("127.0.0.1", 0))
        return listener.getsockname()[1]


def worker(rank, ranks, port, tokens, heads, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ranks)
    try:
        generator = torch.Generator().manual_seed(7)
        qkv = torch.randn((tokens, 3, heads, HEAD_DIM), generator=generator)
        shard = Shard.even(rank, ranks, tokens, heads, 1)
        own = shard.own_tokens
        layer = UlyssesAttention(shard, tokens, heads, torch_attention, "cpu", torch.float32)
        output = torch.zeros((len(own), heads, HEAD_DIM))
        layer.run(qkv[own.start:own.stop].contiguous(), output)
        whole = torch.zeros((tokens, heads, HEAD_DIM))
        torch_attention(qkv.contiguous(), whole, tokens, heads)
        error = float((output - whole[own.start:own.stop]).abs().max())
        # The same layer a group of heads at a time: every rank's heads cut in two runs (one of
        # them may be empty when a rank owns a single head).
        grouped = torch.zeros_like(output)
        for cut in head_groups(shard, 2):
            UlyssesAttention(cut, tokens, heads, torch_attention, "cpu", torch.float32).run(
                qkv[own.start:own.stop].contiguous(), grouped)
        error = max(error, float((grouped - whole[own.start:own.stop]).abs().max()))
        # A profiled step charges every stretch it has and leaves the result alone
        # (MMH3_SHARD_PROFILE=sync, crates/mmh3-core/src/shard.rs:413-502).
        os.environ["MMH3_SHARD_PROFILE"] = "sync"
        profiled = torch.zeros_like(output)
        for _ in range(2):
            layer.run(qkv[own.start:own.stop].contiguous(), profiled)
        del os.environ["MMH3_SHARD_PROFILE"]
        spent = layer.timing.stretches
        assert torch.equal(profiled, output)
        assert all(spent[name] > 0.0 for name in ("before", "publish", "input exchange",
                                                  "attention", "output exchange"))
        assert spent["own projections"] == 0.0 and "attention" in layer.timing.describe_stretches()
        # And through the layer that overlaps the groups' exchanges with their attention on a GPU
        # (on CPU ranks its steps run in the same order, one after the other).
        overlapped = torch.zeros_like(output)
        OverlappedUlyssesAttention(shard, tokens, heads, torch_attention, 4, "cpu",
                                   torch.float32).run(qkv[own.start:own.stop].contiguous(),
                                                      overlapped)
        results[rank] = max(error, float((overlapped - whole[own.start:own.stop]).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ranks,tokens,heads", [(2, 96, 4), (3, 100, 7)])
def test_split_run_equals_whole_run(ranks, tokens, heads):
    port = free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(ranks, port, tokens, heads, results), nprocs=ranks, join=True)
    assert len(results) == ranks
    assert all(error < 1e-5 for error in results.values()), dict(results)


def projected_worker(rank, ranks, port, tokens, heads, hidden, results):
    """The INT8 wire format: every rank gathers the quantized block input and projects the whole
    sequence onto its own heads. The projection here is the GEMM's definition in float64."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ranks)
    try:
        generator = torch.Generator().manual_seed(11)
        rows = torch.randint(-127, 128, (tokens, hidden), generator=generator, dtype=torch.int8)
        scales = torch.rand(tokens, generator=generator) * 0.01 + 0.005
        weights = torch.randint(-127, 128, (3 * heads * HEAD_DIM, hidden), generator=generator,
                                dtype=torch.int8)
        weight_scales = torch.rand(3 * heads * HEAD_DIM, generator=generator) * 0.01 + 0.005

        def projection(selected):
            def project(part_rows, part_scales, qkv):
                sums = part_rows.double() @ weights[selected].double().T
                qkv.copy_((sums * part_scales.double()[:, None] *
                           weight_scales[selected].double()[None, :]).float())
            return project

        shard = Shard.even(rank, ranks, tokens, heads, 1)
        own = shard.own_tokens
        layer = ProjectedUlyssesAttention(
            shard, tokens, heads, hidden, projection(own_projection_rows(heads, shard.own_heads)),
            torch_attention, "cpu", torch.float32)
        output = torch.zeros((len(own), heads, HEAD_DIM))
        layer.run(rows[own.start:own.stop].contiguous(), scales[own.start:own.stop].contiguous(),
                  output)
        whole_shard = Shard.even(0, 1, tokens, heads, 1)
        whole_layer = ProjectedUlyssesAttention(
            whole_shard, tokens, heads, hidden,
            projection(own_projection_rows(heads, range(heads))), torch_attention, "cpu",
            torch.float32)
        whole = torch.zeros((tokens, heads, HEAD_DIM))
        whole_layer.run(rows, scales, whole)
        results[rank] = (float((output - whole[own.start:own.stop]).abs().max()),
                         layer.exchange_bytes())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ranks,tokens,heads", [(2, 96, 4), (3, 100, 7)])
def test_projected_split_run_equals_whole_run(ranks, tokens, heads):
    hidden = 64
    port = free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(projected_worker, args=(ranks, port, tokens, heads, hidden, results), nprocs=ranks,
             join=True)
    assert len(results) == ranks
    assert all(error < 1e-4 for error, _ in results.values()), dict(results)
    # What a rank sends: its rows and scales to every peer, and its heads of the others' tokens.
    shard = Shard.even(0, ranks, tokens, heads, 1)
    own_tokens, own_heads = len(shard.own_tokens), len(shard.own_heads)
    expected = (ranks - 1) * own_tokens * (hidden + 4) + \
        (tokens - own_tokens) * own_heads * HEAD_DIM * 4
    assert results[0][1] == expected


def test_own_projection_rows():
    rows = own_projection_rows(4, range(1, 3))
    assert rows.tolist()[:2] == [128, 129] and len(rows) == 3 * 2 * 128
    assert rows[256].item() == 4 * 128 + 128 and rows[512].item() == 8 * 128 + 128


def test_head_groups():
    shard = Shard.even(1, 2, 10, 7, 1)  # heads 0-2 and 3-6
    cuts = head_groups(shard, 2)
    assert [cut.heads for cut in cuts] == [(range(0, 1), range(3, 5)), (range(1, 3), range(5, 7))]
    assert all(cut.tokens == shard.tokens and cut.rank == 1 for cut in cuts)
    # More groups than a rank has heads: its empty runs stay, wholly empty groups go.
    assert len(head_groups(Shard.even(0, 2, 10, 2, 1), 4)) == 1


def test_ramped_groups_cover_every_head_once():
    """The overlapped layer's groups: one head first and last where there are heads enough, every
    head of every rank in exactly one group, and no group empty on every rank."""
    assert group_sizes(16, 4, ramped=True) == [1, 7, 7, 1]
    assert group_sizes(8, 4, ramped=True) == [1, 3, 3, 1]
    assert group_sizes(4, 4, ramped=True) == [1, 1, 1, 1]
    assert group_sizes(5, 2, ramped=True) == [2, 3]
    assert group_sizes(3, 4, ramped=True) == [0, 1, 1, 1]
    assert growing_sizes(32, 2.0) == [1, 2, 4, 8, 14, 2, 1]
    assert growing_sizes(16, 3.0, 10.0) == [1, 3, 9, 2, 1]
    assert growing_sizes(4, 1.0) == [1, 1, 1, 1] and growing_sizes(1, 2.0) == [1]
    for ranks, heads in ((2, 32), (3, 7), (8, 40)):
        shard = Shard.even(0, ranks, 1000, heads)
        cuts = head_groups(shard, 0, growth=3.0)
        for peer in range(ranks):
            assert [head for cut in cuts for head in cut.heads[peer]] == list(shard.heads[peer])
    for ranks, heads, groups in ((2, 32, 4), (3, 32, 4), (8, 32, 4), (8, 40, 4), (3, 7, 5), (4, 5, 3)):
        shard = Shard.even(0, ranks, 1000, heads)
        cuts = head_groups(shard, groups, ramped=True)
        for peer in range(ranks):
            seen = [head for cut in cuts for head in cut.heads[peer]]
            assert seen == list(shard.heads[peer]), (ranks, heads, groups, peer)
        assert all(any(len(run) for run in cut.heads) for cut in cuts)


def test_even_cuts():
    shard = Shard.even(1, 8, 125504, 32, 1)
    assert shard.own_tokens == range(15688, 31376) and shard.own_heads == range(4, 8)
    shard = Shard.even(2, 3, 1000, 7, 64)
    assert [len(cut) for cut in shard.tokens] == [320, 320, 360]
    assert [len(cut) for cut in shard.heads] == [2, 2, 3]
    assert Shard.even(0, 1, 10, 3).is_whole
