"""Head-sharded (Ulysses) attention across the GPUs of one box.

Every rank carries a contiguous run of the sequence and every head outside the attention, and every
token and a contiguous run of heads inside it, as niw/mmh3 splits a DiT step
(crates/mmh3-core/src/shard.rs:1-11, 155-188; crates/mmh3-cuda/src/dit.rs:1416-1604, 1713-1800).
The reference moves the data with its own socket/RDMA/peer-copy exchange; here the two exchanges are
NCCL all-to-alls over NVLink through `torch.distributed`, one process per GPU. On CPU ranks (gloo)
the same code runs with the attention itself supplied by the caller, which is how the partitioning
and the exchange are tested without a GPU.

`UlyssesAttention` exchanges the projected q, k and v. `ProjectedUlyssesAttention` is the
reference's own wire format (crates/mmh3-cuda/src/dit.rs:1609-1711): the ranks exchange the
quantized block input, INT8 rows with one scale each, and every rank projects the whole sequence
onto its own heads.
"""

from __future__ import annotations

import contextlib
import dataclasses
import os
import time
from typing import Callable

import torch
import torch.distributed as dist

HEAD_DIM = 128


@dataclasses.dataclass(frozen=True)
class Shard:
    """Which tokens and which heads each rank owns; both cuts are contiguous."""

    rank: int
    tokens: tuple[range, ...]
    heads: tuple[range, ...]

    @staticmethod
    def even(rank: int, ranks: int, tokens: int, heads: int, alignment: int = 1) -> "Shard":
        """Cuts `tokens` and `heads` into `ranks` shares. Tokens divide on a multiple of
        `alignment` (VSA needs whole tiles), and the remainder of either cut goes to the last rank
        (shard.rs:168-188)."""

        def cut(total: int, step: int) -> tuple[range, ...]:
            step = max(step, 1)
            each = (total // ranks // step) * step
            return tuple(
                range(index * each, total if index + 1 == ranks else (index + 1) * each)
                for index in range(ranks))

        return Shard(rank, cut(tokens, alignment), cut(heads, 1))

    @property
    def ranks(self) -> int:
        return len(self.tokens)

    @property
    def own_tokens(self) -> range:
        return self.tokens[self.rank]

    @property
    def own_heads(self) -> range:
        return self.heads[self.rank]

    @property
    def is_whole(self) -> bool:
        return self.ranks == 1


# The stretches of a shared block in the order it runs them, under the reference's names
# (crates/mmh3-core/src/shard.rs:455-486).
STRETCH_NAMES = ("before", "publish", "own projections", "input exchange", "peer projections",
                 "attention", "output exchange")


@contextlib.contextmanager
def stretch_range(name: str, device):
    """An NVTX range around a stretch of a shared layer on a GPU rank, so that a timeline shows
    the exchanges beside the attention kernels; nothing on CPU ranks."""
    marked = torch.device(device).type == "cuda"
    if marked:
        torch.cuda.nvtx.range_push("mmh3." + name)
    try:
        yield
    finally:
        if marked:
            torch.cuda.nvtx.range_pop()


def profile() -> str:
    """How a shared step is timed, from MMH3_SHARD_PROFILE (shard.rs:488-502): "sync" waits for
    the device at the end of every stretch, which gives up the overlap between them and says where
    the time went; anything else is "off". (The reference's "no-copies" leaves out the copies
    between the ranks of one process; here a rank is a process.)"""
    return "sync" if os.environ.get("MMH3_SHARD_PROFILE") == "sync" else "off"


class ShardTiming:
    """Where a profiled shared step went: seconds per stretch (shard.rs:413-452)."""

    def __init__(self, device=None):
        self.stretches = dict.fromkeys(STRETCH_NAMES, 0.0)
        self.mark = None
        self.device = device

    def end(self, stretch: str) -> None:
        """Ends `stretch` now, the device done with it. The first stretch of a step starts the
        clock rather than being charged, since it has no end before it."""
        if self.device is not None and torch.device(self.device).type == "cuda":
            torch.cuda.synchronize()
        now = time.perf_counter()
        if self.mark is not None:
            self.stretches[stretch] += now - self.mark
        self.mark = now

    def total(self) -> float:
        return sum(self.stretches.values())

    def describe_stretches(self) -> str:
        return ", ".join(f"{name} {spent:.2f} s" for name, spent in self.stretches.items())


# attention(qkv [tokens, 3, heads, 128], output [tokens, heads, 128], tokens, heads)
AttentionFn = Callable[[torch.Tensor, torch.Tensor, int, int], None]
# pack(source, packed, tokens, tensors, heads, first_head, span); unpack(part, output, tokens, heads,
# first_head, span)
PackFn = Callable[..., None]


def _torch_pack(source, packed, tokens, tensors, heads, first_head, span):
    view = source.view(tokens, tensors, heads, HEAD_DIM)
    packed.view(tokens, tensors, span, HEAD_DIM).copy_(view[:, :, first_head:first_head + span])


def _torch_unpack(part, output, tokens, heads, first_head, span):
    output.view(tokens, heads, HEAD_DIM)[:, first_head:first_head + span].copy_(
        part.view(tokens, span, HEAD_DIM))


class UlyssesAttention:
    """One attention layer over a sequence-sharded qkv, with persistent exchange buffers.

    `run(qkv_own, output_own)` takes this rank's rows of the fused projection,
    [own tokens, 3, heads, 128], and fills this rank's rows of the output, [own tokens, heads, 128].
    """

    def __init__(self, shard: Shard, total_tokens: int, heads: int, attention: AttentionFn,
                 device, dtype=torch.bfloat16, pack: PackFn | None = None,
                 unpack: PackFn | None = None, group=None, exchanges_qkv: bool = True):
        self.shard, self.tokens, self.heads = shard, total_tokens, heads
        self.attention = attention
        self.group = group
        self.device = device
        self.pack = pack or _torch_pack
        self.unpack = unpack or _torch_unpack
        own_tokens, own_heads = len(shard.own_tokens), len(shard.own_heads)
        self.own_tokens, self.own_heads = own_tokens, own_heads
        make = dict(dtype=dtype, device=device)
        # Sent: for each peer, its heads of my tokens. Received: my heads of every rank's tokens,
        # which is already [all tokens, 3, own heads, 128] because tokens are outermost.
        exchanged = sum(len(peer) for peer in shard.heads)  # all heads, or a group of them
        self.send_inputs = torch.empty(own_tokens * 3 * exchanged * HEAD_DIM if exchanges_qkv
                                       else 0, **make)
        self.inputs = torch.empty(total_tokens * 3 * own_heads * HEAD_DIM, **make)
        self.attended = torch.empty(total_tokens * own_heads * HEAD_DIM, **make)
        self.received = torch.empty(own_tokens * exchanged * HEAD_DIM, **make)
        self.input_send_splits = [own_tokens * 3 * len(peer) * HEAD_DIM for peer in shard.heads]
        self.input_recv_splits = [len(peer) * 3 * own_heads * HEAD_DIM for peer in shard.tokens]
        self.output_send_splits = [len(peer) * own_heads * HEAD_DIM for peer in shard.tokens]
        self.output_recv_splits = [own_tokens * len(peer) * HEAD_DIM for peer in shard.heads]
        # Filled by `run` when MMH3_SHARD_PROFILE=sync.
        self.timing = ShardTiming(device)

    def exchange_bytes(self) -> int:
        """Bytes this rank sends to other ranks per layer."""
        rank = self.shard.rank
        elements = (sum(self.input_send_splits) - self.input_send_splits[rank]
                    + sum(self.output_send_splits) - self.output_send_splits[rank])
        return elements * self.send_inputs.element_size()

    def run(self, qkv_own: torch.Tensor, output_own: torch.Tensor) -> None:
        if self.shard.is_whole:
            self.attention(qkv_own, output_own, self.tokens, self.heads)
            return
        timing = self.timing if profile() == "sync" else None
        if timing is not None:
            timing.end("before")
        self.exchange_inputs(qkv_own, timing)
        self.attend()
        if timing is not None:
            timing.end("attention")
        self.exchange_outputs(output_own)
        if timing is not None:
            timing.end("output exchange")

    def exchange_inputs(self, qkv_own: torch.Tensor, timing: ShardTiming | None = None) -> None:
        """Turns "my tokens, every head" into "every token, my heads" in `inputs`: every peer's
        heads of this rank's rows packed, then the all-to-all."""
        with stretch_range("publish", self.device):
            offset = 0
            for peer, heads in enumerate(self.shard.heads):
                count = self.input_send_splits[peer]
                if count:
                    self.pack(qkv_own, self.send_inputs[offset:offset + count], self.own_tokens,
                              3, self.heads, heads.start, len(heads))
                offset += count
        if timing is not None:
            timing.end("publish")
        with stretch_range("input exchange", self.device):
            dist.all_to_all_single(self.inputs, self.send_inputs, self.input_recv_splits,
                                   self.input_send_splits, group=self.group)
        if timing is not None:
            timing.end("input exchange")

    def attend(self) -> None:
        """The attention of every token on this rank's heads, `inputs` to `attended`."""
        if self.own_heads:
            with stretch_range("attention", self.device):
                self.attention(self.inputs, self.attended, self.tokens, self.own_heads)

    def exchange_outputs(self, output_own: torch.Tensor) -> None:
        """Turns "every token, my heads" in `attended` back into "my tokens, every head"
        (dit.rs:1713-1800)."""
        with stretch_range("output exchange", self.device):
            dist.all_to_all_single(self.received, self.attended, self.output_recv_splits,
                                   self.output_send_splits, group=self.group)
            offset = 0
            for peer, heads in enumerate(self.shard.heads):
                count = self.output_recv_splits[peer]
                if count:
                    self.unpack(self.received[offset:offset + count], output_own,
                                self.own_tokens, self.heads, heads.start, len(heads))
                offset += count


def group_sizes(count: int, groups: int, ramped: bool = False) -> list[int]:
    """`count` heads in `groups` runs, as even as they come. `ramped` makes the first and the last
    run one head each when there are heads enough, for a pipeline whose first way in and last way
    out nothing hides."""
    if ramped and groups >= 3 and count >= groups:
        return [1] + group_sizes(count - 2, groups - 2) + [1]
    return [count * (group + 1) // groups - count * group // groups for group in range(groups)]


def growing_sizes(count: int, growth: float, drain: float = 6.0) -> list[int]:
    """`count` heads in runs for a pipeline with a stage before the attention (a copy from the
    host, an exchange) that takes 1 / `growth` of the attention's time per head and a stage after
    it that takes 1 / `drain`: one head first, whose way in nothing hides; every run at most
    `growth` times the one before, so that its way in fits behind the attention of the run
    before; and no run more than `drain` times what follows it, so that its way out fits behind
    the attention of the runs after it, which ends the list on one head."""
    sizes, left = [], count
    while left > 0:
        room_in = max(1, int(sizes[-1] * growth)) if sizes else 1
        room_out = max(1, int(drain * left / (1.0 + drain)))
        sizes.append(left if left == 1 else min(room_in, room_out, left))
        left -= sizes[-1]
    return sizes


def head_groups(shard: Shard, groups: int, ramped: bool = False,
                growth: float | None = None) -> list[Shard]:
    """Cuts every rank's heads into `groups` runs (`group_sizes`), or with `growth` into
    `growing_sizes` runs: shard g holds the g-th run of each rank. The layer can then go through
    a group at a time, every rank busy in every group."""
    if growth is not None:
        sizes = [growing_sizes(len(owned), growth) for owned in shard.heads]
        groups = max(len(runs) for runs in sizes)
        sizes = [runs + [0] * (groups - len(runs)) for runs in sizes]
    else:
        sizes = [group_sizes(len(owned), groups, ramped) for owned in shard.heads]
    cuts = []
    for group in range(groups):
        heads = tuple(range(owned.start + sum(sizes[peer][:group]),
                            owned.start + sum(sizes[peer][:group + 1]))
                      for peer, owned in enumerate(shard.heads))
        if any(len(run) for run in heads):
            cuts.append(Shard(shard.rank, shard.tokens, heads))
    return cuts


class OverlappedUlyssesAttention:
    """`UlyssesAttention` a group of heads at a time (`head_groups`), with the exchanges on a
    stream of their own: while one group is attended, the next group's q, k and v are packed and
    exchanged and the last group's output goes back and is unpacked. Only the first group's way in
    and the last group's way out are left outside the attention kernels. The reference overlaps
    its exchange with the projection of the rank's own rows on a copy stream the same way
    (crates/mmh3-cuda/src/dit.rs:1416-1604). Every rank issues its collectives in the same order.

    The groups' attention kernels alternate between the caller's stream and a second one, so that
    the first blocks of one group fill the multiprocessors the last blocks of the group before
    leave idle: cutting the heads costs no partial wave. The exchange stream has the higher
    priority, so its gathers and NCCL's blocks (when the process group was made with
    `is_high_priority_stream`) take the next multiprocessor an attention block leaves rather than
    queueing behind the whole launch. On CPU ranks there are no streams and the same steps run one
    after the other."""

    def __init__(self, shard: Shard, total_tokens: int, heads: int, attention: AttentionFn,
                 groups: int, device, dtype=torch.bfloat16, pack: PackFn | None = None,
                 unpack: PackFn | None = None, group=None):
        self.shard = shard
        self.cuts = [shard] if shard.is_whole else head_groups(shard, groups, ramped=True)
        self.layers = [UlyssesAttention(cut, total_tokens, heads, attention, device, dtype, pack,
                                        unpack, group) for cut in self.cuts]
        self.overlapped = torch.device(device).type == "cuda" and not shard.is_whole
        if self.overlapped:
            self.exchange = torch.cuda.Stream(priority=-1)
            self.second = torch.cuda.Stream()
            self.arrived = [torch.cuda.Event() for _ in self.cuts]
            self.attended = [torch.cuda.Event() for _ in self.cuts]
            self.finished = torch.cuda.Event()

    def exchange_bytes(self) -> int:
        return sum(layer.exchange_bytes() for layer in self.layers)

    def run(self, qkv_own: torch.Tensor, output_own: torch.Tensor) -> None:
        if not self.overlapped:
            for layer in self.layers:
                layer.run(qkv_own, output_own)
            return
        current = torch.cuda.current_stream()
        self.exchange.wait_stream(current)
        self.second.wait_stream(current)

        def way_in(index: int) -> None:
            with torch.cuda.stream(self.exchange):
                self.layers[index].exchange_inputs(qkv_own)
                self.arrived[index].record(self.exchange)

        def way_out(index: int) -> None:
            with torch.cuda.stream(self.exchange):
                self.exchange.wait_event(self.attended[index])
                self.layers[index].exchange_outputs(output_own)

        # The exchange stream: in(0), in(1), out(0), in(2), out(1), ...; the two attention
        # streams: each group once its rows have arrived.
        way_in(0)
        for index, layer in enumerate(self.layers):
            if index + 1 < len(self.layers):
                way_in(index + 1)
            stream = self.second if index % 2 else current
            with torch.cuda.stream(stream):
                stream.wait_event(self.arrived[index])
                layer.attend()
                self.attended[index].record(stream)
            way_out(index)
        self.finished.record(self.exchange)
        current.wait_event(self.finished)
        current.wait_stream(self.second)


class HostUlyssesPipeline:
    """`UlyssesAttention` from this rank's rows in pinned host memory to its rows of the output in
    pinned host memory, a group of heads at a time (`head_groups`, the first and the last group one
    head of every rank): a group's rows cross the bus on one stream, are packed and exchanged on a
    second (of higher priority, as in `OverlappedUlyssesAttention`), attended on the caller's or a
    third in turn, exchanged back on the second and copied out on a fourth, so that every stage
    of one group runs beside other stages of its neighbours. A group's heads are one run per rank,
    so its rows are that many strided 2D copies each way."""

    def __init__(self, shard: Shard, total_tokens: int, heads: int, attention: AttentionFn,
                 groups: int, pack: PackFn | None = None, unpack: PackFn | None = None,
                 group=None, growth: float | None = None):
        from .attention import HostPipeline

        self.shard, self.heads = shard, heads
        self.own_tokens = len(shard.own_tokens)
        self.cuts = [shard] if shard.is_whole else head_groups(shard, groups, ramped=True,
                                                               growth=growth)
        self.layers = [UlyssesAttention(cut, total_tokens, heads, attention, "cuda",
                                        torch.bfloat16, pack, unpack, group)
                       for cut in self.cuts]
        # Only its streams and its 2D copy are used.
        self.copies = HostPipeline(total_tokens, heads, groups=1)
        self.exchange = torch.cuda.Stream(priority=-1)
        self.arrived = [torch.cuda.Event() for _ in self.cuts]
        self.gathered = [torch.cuda.Event() for _ in self.cuts]
        self.attended = [torch.cuda.Event() for _ in self.cuts]
        self.returned = [torch.cuda.Event() for _ in self.cuts]
        self.finished = torch.cuda.Event()

    def _rows(self, device: torch.Tensor, host: torch.Tensor, cut: Shard, tensors: int,
              to_device: bool, stream) -> None:
        pitch = self.heads * HEAD_DIM * 2
        for run in (cut.heads if not cut.is_whole else (range(self.heads),)):
            if len(run) == 0:
                continue
            offset = run.start * HEAD_DIM * 2
            source, destination = (host, device) if to_device else (device, host)
            self.copies.copy_rows(destination.data_ptr() + offset, source.data_ptr() + offset,
                                  pitch, len(run) * HEAD_DIM * 2, self.own_tokens * tensors,
                                  to_device, stream)

    def run(self, host_qkv: torch.Tensor, qkv: torch.Tensor, output: torch.Tensor,
            host_output: torch.Tensor) -> None:
        """Enqueues everything and returns; the current stream ends up behind the last copy."""
        copy_in, copy_out = self.copies.copy_in, self.copies.copy_out
        second, exchange = self.copies.second, self.exchange
        current = torch.cuda.current_stream()
        for stream in (copy_in, copy_out, second, exchange):
            stream.wait_stream(current)
        for index, cut in enumerate(self.cuts):
            self._rows(qkv, host_qkv, cut, 3, True, copy_in)
            self.arrived[index].record(copy_in)
        if self.shard.is_whole:
            current.wait_event(self.arrived[0])
            self.layers[0].run(qkv, output)
            self.attended[0].record(current)
            copy_out.wait_event(self.attended[0])
            self._rows(output, host_output, self.cuts[0], 1, False, copy_out)
            self.finished.record(copy_out)
            current.wait_event(self.finished)
            return

        def way_in(index: int) -> None:
            with torch.cuda.stream(exchange):
                exchange.wait_event(self.arrived[index])
                self.layers[index].exchange_inputs(qkv)
                self.gathered[index].record(exchange)

        # The exchange stream, the same on every rank: in(0), in(1), out(0), in(2), out(1), ...
        way_in(0)
        for index, (cut, layer) in enumerate(zip(self.cuts, self.layers)):
            if index + 1 < len(self.cuts):
                way_in(index + 1)
            stream = second if index % 2 else current
            with torch.cuda.stream(stream):
                stream.wait_event(self.gathered[index])
                layer.attend()
                self.attended[index].record(stream)
            with torch.cuda.stream(exchange):
                exchange.wait_event(self.attended[index])
                layer.exchange_outputs(output)
                self.returned[index].record(exchange)
            copy_out.wait_event(self.returned[index])
            self._rows(output, host_output, cut, 1, False, copy_out)
        self.finished.record(copy_out)
        current.wait_event(self.finished)
        current.wait_stream(second)
        current.wait_stream(exchange)


# project(rows INT8 [count, hidden], scales FP32 [count], qkv [count, 3, own heads, 128]): the
# rank's own columns of the fused qkv projection over `count` rows of the block input.
ProjectFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor], None]


def own_projection_rows(heads: int, own: range) -> torch.Tensor:
    """Rows of the fused qkv weight [3 * heads * 128, hidden] that produce q, k and v of the heads
    in `own`, in the order [3, own heads, 128]."""
    inner = heads * HEAD_DIM
    one = torch.arange(own.start * HEAD_DIM, own.stop * HEAD_DIM)
    return torch.cat([one, inner + one, 2 * inner + one])


class ProjectedUlyssesAttention(UlyssesAttention):
    """One attention layer over a sequence-sharded, quantized block input.

    `run(rows_own, scales_own, output_own)` takes this rank's rows of the block input as the INT8
    GEMM reads them, [own tokens, hidden] with one FP32 scale a row, gathers every rank's
    (dit.rs:1609-1711: publish, send, fetch), projects the whole sequence onto this rank's heads
    with `project`, attends, and fills this rank's rows of the output like `UlyssesAttention`.
    The rank's own rows are projected while the others' are on the wire.
    """

    def __init__(self, shard: Shard, total_tokens: int, heads: int, hidden: int,
                 project: ProjectFn, attention: AttentionFn, device, dtype=torch.bfloat16,
                 unpack: PackFn | None = None, group=None):
        super().__init__(shard, total_tokens, heads, attention, device, dtype, None, unpack,
                         group, exchanges_qkv=False)
        self.hidden, self.project = hidden, project
        self.rows = torch.empty((total_tokens, hidden), dtype=torch.int8, device=device)
        self.scales = torch.empty(total_tokens, dtype=torch.float32, device=device)
        shares = {len(cut) for cut in shard.tokens}
        self.even = len(shares) == 1

    def exchange_bytes(self) -> int:
        """Bytes this rank sends to other ranks per layer."""
        rank = self.shard.rank
        peers = self.shard.ranks - 1
        gathered = peers * self.own_tokens * (self.hidden + 4)
        outputs = sum(self.output_send_splits) - self.output_send_splits[rank]
        return gathered + outputs * self.attended.element_size()

    def gather_inputs(self, rows_own: torch.Tensor, scales_own: torch.Tensor):
        """Starts the exchange of the block input and returns what to wait on."""
        shard = self.shard
        if self.even:
            return [dist.all_gather_into_tensor(self.rows, rows_own, group=self.group,
                                                async_op=True),
                    dist.all_gather_into_tensor(self.scales, scales_own, group=self.group,
                                                async_op=True)]
        # Uneven cuts: every rank's rows go out as one broadcast into their place.
        own = shard.own_tokens
        self.rows[own.start:own.stop].copy_(rows_own)
        self.scales[own.start:own.stop].copy_(scales_own)
        pending = []
        for peer, cut in enumerate(shard.tokens):
            source = peer if self.group is None else dist.get_global_rank(self.group, peer)
            pending.append(dist.broadcast(self.rows[cut.start:cut.stop], source,
                                          group=self.group, async_op=True))
            pending.append(dist.broadcast(self.scales[cut.start:cut.stop], source,
                                          group=self.group, async_op=True))
        return pending

    def run(self, rows_own: torch.Tensor, scales_own: torch.Tensor,  # type: ignore[override]
            output_own: torch.Tensor) -> None:
        shard = self.shard
        width = 3 * self.own_heads * HEAD_DIM
        inputs = self.inputs.view(self.tokens, width)
        if shard.is_whole:
            self.project(rows_own, scales_own, inputs)
            self.attention(self.inputs, output_own, self.tokens, self.heads)
            return
        pending = self.gather_inputs(rows_own, scales_own)
        own = shard.own_tokens
        self.project(rows_own, scales_own, inputs[own.start:own.stop])
        for work in pending:
            work.wait()
        # The rows before and after this rank's own.
        for cut in (range(0, own.start), range(own.stop, self.tokens)):
            if len(cut) > 0:
                self.project(self.rows[cut.start:cut.stop], self.scales[cut.start:cut.stop],
                             inputs[cut.start:cut.stop])
        self.attention(self.inputs, self.attended, self.tokens, self.own_heads)
        self.exchange_outputs(output_own)
