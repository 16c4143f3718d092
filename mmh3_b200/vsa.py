"""Host side of video sparse attention: the tiling of the packed sequence.

Mirrors `VsaPlan` of niw/mmh3 (crates/mmh3-core/src/dit/vsa.rs:22-139) and the part of
`PackedLayout::text_to_video` it reads (crates/mmh3-core/src/dit/layout.rs:188-204, 300-321). This
is integer host logic, not an oracle and not on the timed path.
"""

from __future__ import annotations

import dataclasses
import math

VSA_TILE = 64
VSA_CUBE = (4, 4, 4)
FASTH3_SPARSITY = 0.9


@dataclasses.dataclass(frozen=True)
class Segment:
    kind: str
    start: int
    end: int


@dataclasses.dataclass(frozen=True)
class PackedLayout:
    """Text, then stereo audio rows (channel-major), then the video patches."""

    segments: tuple[Segment, ...]
    latent_frames: int
    latent_height: int
    latent_width: int
    audio_frames: int

    @staticmethod
    def text_to_video(text_tokens: int, latent_frames: int, latent_height: int,
                      latent_width: int, audio_frames: int) -> "PackedLayout":
        audio_end = text_tokens + 2 * audio_frames
        video = latent_frames * (latent_height // 2) * (latent_width // 2)
        return PackedLayout(
            segments=(
                Segment("text", 0, text_tokens),
                Segment("audio", text_tokens, audio_end),
                Segment("video", audio_end, audio_end + video),
            ),
            latent_frames=latent_frames,
            latent_height=latent_height,
            latent_width=latent_width,
            audio_frames=audio_frames,
        )

    def __len__(self) -> int:
        return self.segments[-1].end

    def segment(self, kind: str) -> Segment:
        return next(segment for segment in self.segments if segment.kind == kind)


@dataclasses.dataclass(frozen=True)
class VsaPlan:
    """The packed sequence cut into tiles of at most 64 tokens, with the video in cube order."""

    tile_starts: tuple[int, ...]
    tile_lengths: tuple[int, ...]
    prefix_tiles: int
    video_start: int
    # For each video token in the reordered sequence, its index among the video tokens in the
    # packed layout.
    video_order: tuple[int, ...]

    @staticmethod
    def for_layout(layout: PackedLayout) -> "VsaPlan":
        starts: list[int] = []
        lengths: list[int] = []
        for segment in layout.segments:
            if segment.kind == "video":
                continue
            for start in range(segment.start, segment.end, VSA_TILE):
                starts.append(start)
                lengths.append(min(segment.end - start, VSA_TILE))
        prefix_tiles = len(starts)
        video = layout.segment("video")
        grid = (layout.latent_frames, layout.latent_height // 2, layout.latent_width // 2)
        if grid[0] * grid[1] * grid[2] != video.end - video.start:
            raise ValueError("the video segment does not match the latent grid")
        order: list[int] = []
        start = video.start
        for frame_tile in range(0, grid[0], VSA_CUBE[0]):
            for row_tile in range(0, grid[1], VSA_CUBE[1]):
                for column_tile in range(0, grid[2], VSA_CUBE[2]):
                    before = len(order)
                    for frame in range(frame_tile, min(frame_tile + VSA_CUBE[0], grid[0])):
                        for row in range(row_tile, min(row_tile + VSA_CUBE[1], grid[1])):
                            base = (frame * grid[1] + row) * grid[2]
                            order.extend(
                                base + column
                                for column in range(column_tile,
                                                    min(column_tile + VSA_CUBE[2], grid[2]))
                            )
                    length = len(order) - before
                    starts.append(start)
                    lengths.append(length)
                    start += length
        return VsaPlan(tuple(starts), tuple(lengths), prefix_tiles, video.start, tuple(order))

    @property
    def tiles(self) -> int:
        return len(self.tile_starts)

    @property
    def video_tiles(self) -> int:
        return self.tiles - self.prefix_tiles

    def kept_video_tiles(self, sparsity: float) -> int:
        """Video tiles each video query tile keeps at `sparsity`."""
        tiles = self.video_tiles
        return min(max(math.ceil((1.0 - sparsity) * tiles), 1), max(tiles, 1))

    def sequence_order(self, tokens: int) -> list[int]:
        """The packed sequence position of each position of the reordered sequence."""
        video_end = self.video_start + len(self.video_order)
        return (
            list(range(self.video_start))
            + [self.video_start + index for index in self.video_order]
            + list(range(video_end, tokens))
        )

    def expected_selected_fraction(self, kept: int) -> float:
        """Mean fraction of tiles a query tile attends token by token (closed form)."""
        prefix, video, tiles = self.prefix_tiles, self.video_tiles, self.tiles
        if kept >= video:
            return 1.0
        return (prefix * tiles + video * (prefix + kept)) / (tiles * tiles)
