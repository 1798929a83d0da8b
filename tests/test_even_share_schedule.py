"""CPU: the arithmetic of the even-share schedule of the persistent decode kernels, restated in Python.

The device code (anna_b200/csrc/balanced_schedule.cuh) lets every work unit derive its tile range, the slot of each
partial it writes and the number of partials each stream will receive from three numbers (tiles per row, units,
scratch capacity).  The properties the fused merge relies on are checked here for many ragged batches: every tile is
covered exactly once, slots of a stream are 0 .. partials-1 without gaps or repeats, and no stream needs more slots
than the scratch holds."""
from __future__ import annotations

import random

import pytest

TILE = 16


def share_of(total: int, units: int, max_tiles: int, capacity: int, min_tiles: int) -> int:
    share = (total + units - 1) // units
    share = max(share, min_tiles)
    return max(share, (max_tiles + capacity - 2) // (capacity - 1))


def segments(lengths: list[int], streams_per_row: int, units: int, capacity: int, min_tiles: int):
    """(unit, row, stream, first tile, tiles, slot, partials) for every piece, walking the line like the kernel."""
    tiles_row = [(n + TILE - 1) // TILE for n in lengths]
    prefix = [0]
    for n in tiles_row:
        prefix.append(prefix[-1] + n * streams_per_row)
    total = prefix[-1]
    if total == 0:
        return [], 0
    share = share_of(total, units, max(tiles_row), capacity, min_tiles)
    out = []
    for unit in range(units):
        pos, end = min(unit * share, total), min((unit + 1) * share, total)
        while pos < end:
            row = max(b for b in range(len(lengths)) if prefix[b] <= pos and tiles_row[b] > 0)
            n = tiles_row[row]
            stream = (pos - prefix[row]) // n
            tile = (pos - prefix[row]) - stream * n
            seg = min(n - tile, end - pos)
            stream_first = prefix[row] + stream * n
            first_unit = stream_first // share
            out.append((unit, row, stream, tile, seg, unit - first_unit,
                        (stream_first + n - 1) // share - first_unit + 1))
            pos += seg
    return out, share


@pytest.mark.parametrize("seed", range(12))
def test_even_share_covers_every_tile_once_with_dense_slots(seed):
    rng = random.Random(seed)
    batch = rng.choice([1, 2, 7, 32, 100])
    lengths = [rng.choice([0, 1, 15, 16, 17, rng.randint(1, 9000)]) for _ in range(batch)]
    if seed % 4 == 0:
        lengths[rng.randrange(batch)] = 40000          # one long row among short ones
    streams_per_row = rng.choice([1, 2, 8])
    units = rng.choice([4, 444, 1776])
    capacity = rng.choice([2, 3, 16, 64])
    min_tiles = rng.choice([1, 4])
    pieces, share = segments(lengths, streams_per_row, units, capacity, min_tiles)
    covered: dict[tuple[int, int], list[int]] = {}
    slots: dict[tuple[int, int], list[tuple[int, int]]] = {}
    for unit, row, stream, tile, seg, slot, partials in pieces:
        assert seg >= 1 and 0 <= slot < partials <= capacity
        covered.setdefault((row, stream), []).extend(range(tile, tile + seg))
        slots.setdefault((row, stream), []).append((slot, partials))
    for row, n in enumerate(lengths):
        tiles = (n + TILE - 1) // TILE
        for stream in range(streams_per_row):
            if tiles == 0:
                assert (row, stream) not in covered
                continue
            assert sorted(covered[(row, stream)]) == list(range(tiles))
            got = sorted(s for s, _ in slots[(row, stream)])
            partials = slots[(row, stream)][0][1]
            assert got == list(range(partials)) and all(p == partials for _, p in slots[(row, stream)])
    if pieces:
        work = {}
        for unit, *_rest in pieces:
            work[unit] = work.get(unit, 0) + _rest[3]
        assert max(work.values()) <= share


FUSED_MAX_CHUNKS = 512  # kFusedMaxChunks: weights per head that the fused merge stages in shared memory


@pytest.mark.parametrize("capacity", [600, 4096])
def test_even_share_never_exceeds_the_fused_merge_limit(capacity):
    """A caller may hand in a scratch larger than the fused merge can stage; the kernel clamps the capacity it gives
    to the schedule to 512, so one very long row beside short ones still gets at most 512 partials."""
    lengths = [512 * 1024] + [1] * 7           # ~586 partials with an unclamped capacity and 592 units
    pieces, _ = segments(lengths, 1, 592, min(capacity, FUSED_MAX_CHUNKS), 4)
    assert pieces
    assert max(partials for *_head, partials in pieces) <= FUSED_MAX_CHUNKS
    unclamped, _ = segments(lengths, 1, 592, capacity, 4)
    assert max(partials for *_head, partials in unclamped) > FUSED_MAX_CHUNKS  # the case the clamp is for
