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

from mmh3_b200.shard import Shard, UlyssesAttention

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
        results[rank] = float((output - whole[own.start:own.stop]).abs().max())
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


def test_even_cuts():
    shard = Shard.even(1, 8, 125504, 32, 1)
    assert shard.own_tokens == range(15688, 31376) and shard.own_heads == range(4, 8)
    shard = Shard.even(2, 3, 1000, 7, 64)
    assert [len(cut) for cut in shard.tokens] == [320, 320, 360]
    assert [len(cut) for cut in shard.heads] == [2, 2, 3]
    assert Shard.even(0, 1, 10, 3).is_whole
