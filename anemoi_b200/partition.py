"""Ragged 2-D block partition of one video frame (host side, cached).

A frame of ``height x width`` tokens is covered by exactly
``ceil(height * width / capacity)`` four-connected blocks whose real-token counts
differ by at most one.  Two families of covers are searched and the one with the
smaller shape cost wins:

* *stripe covers*: the frame is cut into full-width row bands (a dynamic program
  picks the band heights and block counts), and every band is cut along a
  column-wise boustrophedon walk; the same is tried on the transposed frame;
* *two-level covers*: blocks are first grouped into roughly square ragged bands
  along a row-wise boustrophedon walk of the whole frame, then each band is cut
  along a perpendicular walk of its own cells.

The shape cost is the lexicographic tuple (total perimeter, bounding-box waste,
second spatial moment, |log aspect|).

Behaviour follows the reference's ``make_ragged_2d_partition``
(anemoi/layers/attention/mpa/ragged_2d.py:448-525) bit for bit - the floating
point sums below are evaluated in the same order so that ties resolve the same
way - and is pinned by the reference's SHA-256 vectors
(tests/test_mpa_ragged_2d.py:85-146) in this repository's tests.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

Block = tuple[int, ...]
Cover = tuple[Block, ...]


@dataclass(frozen=True)
class Ragged2DPartition:
    """Exact cover of a ``height x width`` raster by connected balanced blocks."""

    height: int
    width: int
    capacity: int
    blocks: Cover
    token_to_block: tuple[int, ...]
    adjacency: tuple[tuple[bool, ...], ...] | None

    @property
    def block_count(self) -> int:
        return len(self.blocks)

    @property
    def counts(self) -> tuple[int, ...]:
        return tuple(len(block) for block in self.blocks)


# --------------------------------------------------------------------------
# shape cost
# --------------------------------------------------------------------------
def _shape_terms(block: Block, width: int) -> tuple[int, int, float, float]:
    """(perimeter, bounding-box waste, moment, aspect error) of one block."""
    cells = {divmod(token, width) for token in block}
    ys = [y for y, _ in cells]
    xs = [x for _, x in cells]
    box_h = max(ys) - min(ys) + 1
    box_w = max(xs) - min(xs) + 1
    edge = 0
    for y, x in cells:
        for other in ((y - 1, x), (y + 1, x), (y, x - 1), (y, x + 1)):
            edge += other not in cells
    mean_y = sum(ys) / len(ys)
    mean_x = sum(xs) / len(xs)
    moment = sum((y - mean_y) ** 2 + (x - mean_x) ** 2 for y, x in cells)
    return edge, box_h * box_w - len(block), moment, abs(math.log(box_w / box_h))


def _cover_cost(cover: Cover, width: int) -> tuple[float, float, float, float, int]:
    per_block = [_shape_terms(block, width) for block in cover]
    return (
        float(sum(t[0] for t in per_block)),
        float(sum(t[1] for t in per_block)),
        sum(t[2] for t in per_block),
        sum(t[3] for t in per_block),
        1,
    )


def _cost_sum(a, b):
    return (
        round(a[0] + b[0], 12),
        round(a[1] + b[1], 12),
        round(a[2] + b[2], 12),
        round(a[3] + b[3], 12),
        a[4] + b[4],
    )


# --------------------------------------------------------------------------
# walks and cuts
# --------------------------------------------------------------------------
def _balanced_sizes(tokens: int, parts: int) -> tuple[int, ...]:
    small, extra = divmod(tokens, parts)
    return (small + 1,) * extra + (small,) * (parts - extra)


def _cut(walk: tuple[int, ...], sizes) -> Cover:
    out = []
    start = 0
    for size in sizes:
        out.append(walk[start : start + size])
        start += size
    return tuple(out)


def _column_walk_cover(height: int, width: int, parts: int) -> Cover:
    """Cut a full ``height x width`` band along its column-wise snake."""
    walk = []
    for x in range(width):
        ys = range(height) if x % 2 == 0 else range(height - 1, -1, -1)
        walk.extend(y * width + x for y in ys)
    return _cut(tuple(walk), _balanced_sizes(height * width, parts))


def _is_connected(block: Block, width: int) -> bool:
    todo = set(block)
    stack = [todo.pop()]
    while stack:
        token = stack.pop()
        y, x = divmod(token, width)
        near = []
        if y:
            near.append(token - width)
        if x:
            near.append(token - 1)
        if x + 1 < width:
            near.append(token + 1)
        near.append(token + width)
        for other in near:
            if other in todo:
                todo.remove(other)
                stack.append(other)
    return not todo


def _transpose_cover(cover: Cover, height: int, width: int) -> Cover:
    """Map a cover of the ``width x height`` transposed frame back to raster ids."""
    return tuple(
        tuple((token % height) * width + token // height for token in block) for block in cover
    )


# --------------------------------------------------------------------------
# stripe covers (dynamic program over row bands)
# --------------------------------------------------------------------------
def _stripe_cover(height: int, width: int, capacity: int, parts: int) -> Cover:
    small, extra = divmod(height * width, parts)
    if small + bool(extra) > capacity:
        raise RuntimeError("balanced block size exceeds physical capacity")
    bands: dict[tuple[int, int], tuple[Cover, tuple]] = {}
    best: dict[tuple[int, int], tuple] = {(0, 0): ((0.0, 0.0, 0.0, 0.0, 0), 0, ())}
    for top in range(height):
        for used in range(parts + 1):
            here = best.get((top, used))
            if here is None:
                continue
            cost, centre, chosen = here
            for band_h in range(1, height - top + 1):
                band_tokens = band_h * width
                rows_left = height - top - band_h
                lo = math.ceil(band_tokens / (small + 1))
                hi = min(band_tokens // small, parts - used)
                for band_parts in range(lo, hi + 1):
                    band_extra = band_tokens - band_parts * small
                    if not 0 <= band_extra <= band_parts:
                        continue
                    parts_left = parts - used - band_parts
                    extra_left = rows_left * width - parts_left * small
                    if not 0 <= extra_left <= parts_left:
                        continue
                    entry = bands.get((band_h, band_parts))
                    if entry is None:
                        local = _column_walk_cover(band_h, width, band_parts)
                        entry = (local, _cover_cost(local, width))
                        bands[(band_h, band_parts)] = entry
                    bottom = top + band_h
                    trial = (
                        _cost_sum(cost, entry[1]),
                        centre + (abs(2 * bottom - height) if bottom < height else 0),
                        chosen + ((band_h, band_parts),),
                    )
                    key = (bottom, used + band_parts)
                    if key not in best or trial < best[key]:
                        best[key] = trial
    final = best.get((height, parts))
    if final is None:
        raise RuntimeError("stripe DP failed to find the capacity-minimum cover")
    cover = []
    top = 0
    for band_h, band_parts in final[2]:
        for block in bands[(band_h, band_parts)][0]:
            cover.append(tuple((t // width + top) * width + t % width for t in block))
        top += band_h
    return tuple(cover)


# --------------------------------------------------------------------------
# two-level covers
# --------------------------------------------------------------------------
def _bit_patterns(length: int, ones: int) -> tuple[tuple[int, ...], ...]:
    """A constant-size family of 0/1 arrangements with ``ones`` ones."""
    if not 0 <= ones <= length:
        raise ValueError("ones must be within the binary-pattern length")
    if ones in (0, length):
        return ((1 if ones else 0,) * length,)
    spread = tuple((i + 1) * ones // length - i * ones // length for i in range(length))
    family = {
        (1,) * ones + (0,) * (length - ones),
        (0,) * (length - ones) + (1,) * ones,
        spread,
        spread[::-1],
    }
    return tuple(sorted(family))


def _two_level_cover(height: int, width: int, sizes, band_parts) -> Cover | None:
    outer = []
    for y in range(height):
        xs = range(width) if y % 2 == 0 else range(width - 1, -1, -1)
        outer.extend(y * width + x for x in xs)
    outer = tuple(outer)
    cover: list[Block] = []
    token_at = 0
    part_at = 0
    for count in band_parts:
        band_sizes = sizes[part_at : part_at + count]
        band_tokens = sum(band_sizes)
        cells = set(outer[token_at : token_at + band_tokens])
        column_rows: list[list[int]] = [[] for _ in range(width)]
        for token in cells:
            y, x = divmod(token, width)
            column_rows[x].append(y)
        for rows in column_rows:
            rows.sort()
        winner = None
        for right_to_left in (False, True):
            columns = range(width - 1, -1, -1) if right_to_left else range(width)
            for phase in (0, 1):
                walk = tuple(
                    y * width + x
                    for position, x in enumerate(columns)
                    for y in (
                        column_rows[x]
                        if (position + phase) % 2 == 0
                        else reversed(column_rows[x])
                    )
                )
                pieces = []
                start = 0
                for size in band_sizes:
                    piece = walk[start : start + size]
                    if not _is_connected(piece, width):
                        break
                    pieces.append(piece)
                    start += size
                if len(pieces) != count:
                    continue
                pieces = tuple(pieces)
                trial = (_cover_cost(pieces, width), right_to_left, phase, pieces)
                if winner is None or trial < winner:
                    winner = trial
        if winner is None:
            return None
        cover.extend(winner[3])
        token_at += band_tokens
        part_at += count
    if token_at != height * width or part_at != len(sizes):
        raise RuntimeError("compact band construction did not consume the exact grid")
    return tuple(cover)


def _best_two_level_cover(height: int, width: int, capacity: int, parts: int) -> Cover | None:
    small, extra = divmod(height * width, parts)
    if small + bool(extra) > capacity:
        raise RuntimeError("balanced block size exceeds physical capacity")
    winner = None
    for flipped in (False, True):
        h, w = (width, height) if flipped else (height, width)
        ideal = math.sqrt(parts * h / w)
        band_numbers = {
            max(1, min(h, parts, math.floor(ideal))),
            max(1, min(h, parts, math.ceil(ideal))),
        }
        for bands in sorted(band_numbers):
            per_band, fat_bands = divmod(parts, bands)
            for band_bits in _bit_patterns(bands, fat_bands):
                band_parts = tuple(per_band + bit for bit in band_bits)
                for size_bits in _bit_patterns(parts, extra):
                    sizes = tuple(small + bit for bit in size_bits)
                    cover = _two_level_cover(h, w, sizes, band_parts)
                    if cover is None:
                        continue
                    if flipped:
                        cover = _transpose_cover(cover, height, width)
                    trial = (_cover_cost(cover, width), flipped, bands, band_parts, sizes, cover)
                    if winner is None or trial < winner:
                        winner = trial
    return None if winner is None else winner[5]


def _adjacency(height: int, width: int, owner: list[int], parts: int):
    touch = [[False] * parts for _ in range(parts)]
    for i in range(parts):
        touch[i][i] = True
    for y in range(height):
        for x in range(width):
            a = owner[y * width + x]
            if x + 1 < width:
                b = owner[y * width + x + 1]
                touch[a][b] = touch[b][a] = True
            if y + 1 < height:
                b = owner[(y + 1) * width + x]
                touch[a][b] = touch[b][a] = True
    return tuple(tuple(row) for row in touch)


@lru_cache(maxsize=128)
def make_ragged_2d_partition(
    height: int,
    width: int,
    capacity: int = 64,
    *,
    include_adjacency: bool = True,
) -> Ragged2DPartition:
    """Partition one ``height x width`` frame into balanced connected blocks."""
    if any(type(v) is not int or v <= 0 for v in (height, width)):
        raise ValueError("height and width must be positive integers")
    if type(capacity) is not int or capacity <= 0:
        raise ValueError("capacity must be a positive integer")
    if type(include_adjacency) is not bool:
        raise TypeError("include_adjacency must be a built-in bool")

    parts = math.ceil(height * width / capacity)
    if height == 1 or width == 1:
        chosen = _column_walk_cover(1, height * width, parts)
    else:
        across = _stripe_cover(height, width, capacity, parts)
        down = _transpose_cover(_stripe_cover(width, height, capacity, parts), height, width)
        stripe = (
            across
            if (_cover_cost(across, width), False) <= (_cover_cost(down, width), True)
            else down
        )
        nested = _best_two_level_cover(height, width, capacity, parts)
        chosen = (
            nested
            if nested is not None and _cover_cost(nested, width) < _cover_cost(stripe, width)
            else stripe
        )
    blocks = tuple(tuple(sorted(block)) for block in chosen)

    owner = [-1] * (height * width)
    for index, block in enumerate(blocks):
        if not block or len(block) > capacity:
            raise RuntimeError("ragged block violates physical K capacity")
        for token in block:
            if not 0 <= token < height * width:
                raise RuntimeError("ragged block contains an invalid token")
            if owner[token] != -1:
                raise RuntimeError("ragged partition assigned a token twice")
            owner[token] = index
    if min(owner) < 0:
        raise RuntimeError("ragged partition did not cover the complete grid")
    if len(blocks) != parts:
        raise RuntimeError("ragged partition did not reach the capacity lower bound")
    return Ragged2DPartition(
        height=height,
        width=width,
        capacity=capacity,
        blocks=blocks,
        token_to_block=tuple(owner),
        adjacency=_adjacency(height, width, owner, parts) if include_adjacency else None,
    )


__all__ = ["Ragged2DPartition", "make_ragged_2d_partition"]
