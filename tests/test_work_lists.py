"""The work lists of the prompt attention kernels (host code): every token of every entry
lies in exactly one tile or unit, the parts of one together hold all its key blocks once, the
split ones are numbered without gaps, and the list is sorted the way the kernels take it."""
import random

import pytest

from mini_llm_b200.kernels import ops


def random_step(rng):
    n_items = rng.randint(1, 6)
    counts = [rng.choice([1, 2, 7, 64, 127, 128, 129, 255, 256, 257, 300, 700, 1024]) for _ in range(n_items)]
    starts = [rng.choice([0, 0, 1, 63, 128, 500, 1000, 3000]) for _ in range(n_items)]
    offsets, total = [], 0
    for count in counts:
        offsets.append(total)
        total += count
    return offsets, counts, starts


def check_list(records, n_split, most, offsets, counts, starts, rows_per_record):
    by_place = {}
    for item, first_row, rows, position, part, parts, number, blocks in records:
        assert 1 <= rows <= rows_per_record and 0 <= part < parts <= ops.ATTENTION_MAX_PARTS and blocks >= 0
        assert position - starts[item] == first_row - offsets[item], "position and row do not belong together"
        by_place.setdefault((item, first_row), []).append((rows, position, part, parts, number, blocks))
    # rows: each entry is tiled without gap or overlap
    for item, (offset, count) in enumerate(zip(offsets, counts)):
        firsts = sorted(first for (it, first) in by_place if it == item)
        at = offset
        for first in firsts:
            assert first == at
            at += by_place[(item, first)][0][0]
        assert at == offset + count
    # parts: 0 .. parts - 1 once each, the same rows, all key blocks once
    numbers = []
    for (item, first_row), held in by_place.items():
        rows, position, _, parts, number, _ = held[0]
        assert sorted(h[2] for h in held) == list(range(parts))
        assert all(h[0] == rows and h[1] == position and h[3] == parts and h[4] == number for h in held)
        assert sum(h[5] for h in held) == (position + rows - 1) // ops.ATTENTION_TILE + 1
        if parts > 1:
            numbers.append(number)
        else:
            assert number == 0
    assert sorted(numbers) == list(range(n_split))
    assert most == max([h[0][3] for h in by_place.values()] + [1])
    assert [r[7] for r in records] == sorted((r[7] for r in records), reverse=True)


@pytest.mark.parametrize("seed", range(20))
def test_tiles_cover_every_row_and_key_block_once(seed):
    rng = random.Random(seed)
    offsets, counts, starts = random_step(rng)
    for split in (None, True, False):
        records, n_split, most = ops.attention_tiles(offsets, counts, starts, split=split)
        check_list(records, n_split, most, offsets, counts, starts, ops.ATTENTION_TILE)
        if split is False:
            assert n_split == 0 and most == 1


@pytest.mark.parametrize("seed", range(20))
def test_units_cover_every_row_and_key_block_once_and_stay_within_the_sms(seed):
    rng = random.Random(100 + seed)
    offsets, counts, starts = random_step(rng)
    for n_heads, n_sms in ((12, 148), (1, 148), (25, 132), (16, 10 ** 6), (12, 1)):
        records, n_split, most = ops.attention_units(offsets, counts, starts, n_heads, n_sms)
        check_list(records, n_split, most, offsets, counts, starts, ops.ATTENTION_UNIT)
        n_units = sum(-(-count // ops.ATTENTION_UNIT) for count in counts)
        # parts are added only while the records of all heads still fit the SMs
        assert len(records) == n_units or len(records) * n_heads <= n_sms
        for record in records:
            if record[5] > 1:                      # a unit is not cut below two key blocks a part
                whole = (record[3] + record[2] - 1) // ops.ATTENTION_TILE + 1
                assert -(-whole // (record[5] - 1)) >= 3
