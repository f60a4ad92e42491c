"""The step description's work lists, without a GPU: the attention planner's tiles, single
tokens and work items (every tile covered exactly once, long tiles in parts whose slots are
consecutive, longest first, one round of CTAs where that is possible), the layout's room for
them, and the launch sizes a replayed step uses."""
import random

import numpy as np
import pytest

from pretrained_rstr_b200.engine.batch import BatchLayout, WorkPlanner, fill_host_buffer
from pretrained_rstr_b200.parts.attention import AttentionWork


def _fill(planner, lengths, starts, t_cap=None, b_cap=None):
    t_cap = t_cap or max(8, sum(lengths))
    b_cap = b_cap or max(1, len(lengths))
    arrays = {name: np.full(cap, fill, dtype=np.int32)
              for name, (cap, fill) in planner.arrays(t_cap, b_cap).items()}
    return arrays, planner.fill(arrays, lengths, starts)


def _check_items(planner, arrays, got, lengths, starts):
    n_tiles, n_items = got["tiles"], got["items"]
    part = int(arrays["part_blocks"][0])
    # the key blocks of every tile, as the kernel works them out
    spans = []
    t = 0
    for b, n in enumerate(lengths):
        if n > planner.SINGLE_MAX_Q:
            for r0 in range(0, n, planner.TILE):
                rows = min(planner.TILE, n - r0)
                pos0 = starts[b] + r0
                lo = max(0, pos0 - planner.window + 1) if planner.window else 0
                spans.append((lo // 64, (pos0 + rows - 1) // 64))
        t += n
    assert len(spans) == n_tiles
    seen = {i: [] for i in range(n_tiles)}
    sizes = []
    for i in range(n_items):
        tile, z, slot = (int(arrays[k][i]) for k in ("item_tile", "item_part", "item_slot"))
        first, last = spans[tile]
        if z < 0:
            seen[tile].append(("whole", first, last, None))
            sizes.append(last - first + 1)
        else:
            lo = max(first, (first // part + z) * part)
            hi = min(last, (first // part + z) * part + part - 1)
            assert lo <= hi
            seen[tile].append((z, lo, hi, slot))
            sizes.append(hi - lo + 1)
    assert sizes == sorted(sizes, reverse=True)                    # longest first
    used_slots = []
    for tile, pieces in seen.items():
        first, last = spans[tile]
        assert pieces, f"tile {tile} is in no item"
        if pieces[0][0] == "whole":
            assert len(pieces) == 1
            continue
        pieces.sort()
        assert [p[0] for p in pieces] == list(range(len(pieces)))    # parts 0 .. n-1, each once
        assert len(pieces) == last // part - first // part + 1
        assert len(pieces) <= 16
        assert pieces[0][1] == first and pieces[-1][2] == last
        for a, b in zip(pieces, pieces[1:]):
            assert b[1] == a[2] + 1                                  # no gap, no overlap
            assert b[3] == a[3] + 1                                  # consecutive slots
        used_slots += [p[3] for p in pieces]
    assert sorted(used_slots) == list(range(len(used_slots)))        # every slot once
    assert len(used_slots) <= planner.slot_cap()


@pytest.mark.parametrize("heads,window", [(12, None), (25, None), (4, 100), (2, 700)])
def test_attention_items_cover_every_tile_once(heads, window):
    rng = random.Random(heads)
    for trial in range(200):
        planner = AttentionWork()
        planner.note_mixer(heads, window, rng.choice([None, 8, 148, 1000]))
        if trial % 3 == 0:
            planner.MIN_PART = rng.choice([1, 2, 4])
        n_req = rng.randint(1, 6)
        lengths = [rng.choice([1, 2, 4, 5, 64, 100, 128, 129, 300, 512, 1000]) for _ in range(n_req)]
        starts = [rng.choice([0, 0, 7, 64, 500, 3000, 8000]) for _ in range(n_req)]
        arrays, got = _fill(planner, lengths, starts)
        assert got["singles"] == sum(n for n in lengths if n <= planner.SINGLE_MAX_Q)
        _check_items(planner, arrays, got, lengths, starts)


def test_attention_items_balance_a_long_prompt_step():
    """2 x 1,024 tokens at 12 heads on 148 SMs: 16 tiles of 2 to 16 key blocks become 24 items
    of at most 8, which with 12 heads are 288 CTAs, one round of two to an SM."""
    planner = AttentionWork()
    planner.note_mixer(12, None, 148)
    arrays, got = _fill(planner, [1024, 1024], [0, 0], t_cap=2048, b_cap=8)
    assert {k: got[k] for k in planner.counters} == {"tiles": 16, "singles": 0, "items": 24}
    assert int(arrays["part_blocks"][0]) == 8
    assert got["items"] * 12 <= 2 * 148
    # with 25 heads the tiles alone are more than a round: nothing is split
    planner.note_mixer(25, None, 148)
    arrays, got = _fill(planner, [1024, 1024], [0, 0], t_cap=2048, b_cap=8)
    assert got["items"] == 16 and (arrays["item_part"][:16] < 0).all()


def test_a_decode_step_plans_no_items():
    planner = AttentionWork()
    planner.note_mixer(12, None, 148)
    arrays, got = _fill(planner, [1] * 8, [900 + i for i in range(8)])
    assert {k: got[k] for k in planner.counters} == {"tiles": 0, "singles": 8, "items": 0}
    assert arrays["single_tokens"][:8].tolist() == list(range(8))
    assert got["_used"] == ["single_tokens"]            # nothing else need go to the device


class _Lists(WorkPlanner):
    """A planner of a test: one list of the requests with an even number of tokens."""
    key = "even"
    counters = ("evens",)
    launch_steps = {"evens": (4, "even_req")}

    def arrays(self, t_cap, b_cap):
        return {"even_req": (b_cap, -1)}

    def fill(self, arrays, lengths):
        hits = [b for b, n in enumerate(lengths) if n % 2 == 0]
        arrays["even_req"][:len(hits)] = hits
        return {"evens": len(hits)}


def test_layout_gives_planners_room_and_counters():
    planners = (AttentionWork(), _Lists())
    lay = BatchLayout(64, 8, 1, 16, planners)
    offsets = []
    for key, arrays in lay.work_arrays.items():
        for name, (off, words, _fill_value) in arrays.items():
            assert off % 4 == 0                              # 16-byte aligned
            offsets.append((off, off + words))
    offsets.sort()
    for a, b in zip(offsets, offsets[1:]):
        assert a[1] <= b[0]                                  # no two arrays overlap
    assert set(lay.work_counts["causal_attention"]) == {"tiles", "singles", "items"}
    assert set(lay.work_counts["even"]) == {"evens"}
    host = np.zeros(lay.size, dtype=np.int32)
    tokens = [[1, 2], [3], [4, 5, 6, 7], [8] * 6]
    counts = fill_host_buffer(host, lay, tokens, [0, 5, 9, 100], [0, 1, 2, 3], [True] * 4,
                              [[[0, 1], [2], [3, 4, 5, 6], list(range(7, 13))]],
                              [[[0] * 16 for _ in range(4)]], [[0, 0, 0, 0]], [1, 2])
    assert counts["even"] == {"evens": 3}
    off = lay.work_arrays["even"]["even_req"][0]
    assert host[off:off + 4].tolist() == [0, 2, 3, -1]
    assert counts["causal_attention"]["singles"] == 2 + 1 + 4 and counts["causal_attention"]["tiles"] == 1
    assert host[lay.work_counts["even"]["evens"]] == 3
    # the words a step copies to the device end behind the last array it uses: here the
    # other planner's list (it names no arrays, so all of them count)
    assert counts["_words"] == off + 8
    decode = fill_host_buffer(host, lay, [[1], [2], [3]], [7, 8, 9], [0, 1, 2], [False] * 3,
                              [[[0], [1], [2]]], [[[0] * 16 for _ in range(3)]], [[0, 0, 0]], [0, 1, 2])
    assert decode["_words"] == off + 8


def test_a_decode_step_is_described_like_any_other():
    """One token per request takes a shorter way through fill_host_buffer, and block tables
    may come as rows in their device form: the words are those of the long way."""
    lay = BatchLayout(8, 4, 2, 6, (AttentionWork(),))
    tables = [[[3, 1, 4], [5], [9, 2]], [[7, -1, 8], [0], [6, 11]]]
    rows = [np.full((3, 6), -1, dtype=np.int32) for _ in range(2)]
    for g in range(2):
        for b, table in enumerate(tables[g]):
            rows[g][b, :len(table)] = table
    slots = [[[3 * 16 + 2], [5 * 16 + 1], [2 * 16 + 15]], [[8 * 16 + 2], [1], [11 * 16 + 15]]]
    args = ([[17], [4], [250]], [130, 1, 31], [2, 0, 1], [False, True, False])
    a = np.full(lay.size, 77, dtype=np.int32)
    b = np.full(lay.size, 77, dtype=np.int32)
    ca = fill_host_buffer(a, lay, *args, slots, tables, [[0, 0, 0], [64, 0, 0]], [0, 1, 2])
    cb = fill_host_buffer(b, lay, *args, slots, rows, [[0, 0, 0], [64, 0, 0]], [0, 1, 2])
    assert ca == cb and np.array_equal(a[:ca["_words"]], b[:cb["_words"]])
    assert a[lay.tokens:lay.tokens + 4].tolist() == [17, 4, 250, 0]
    assert a[lay.positions:lay.positions + 4].tolist() == [130, 1, 31, 0]
    assert a[lay.seq_of_token:lay.seq_of_token + 4].tolist() == [0, 1, 2, -1]
    assert a[lay.q_start:lay.q_start + 5].tolist() == [0, 1, 2, 3, 3]
    assert a[lay.kv_len:lay.kv_len + 4].tolist() == [131, 2, 32, 0]
    assert a[lay.state_slot:lay.state_slot + 4].tolist() == [2, 0, 1, 0]
    assert a[lay.fresh:lay.fresh + 4].tolist() == [0, 1, 0, 0]
    assert a[lay.slots[1]:lay.slots[1] + 4].tolist() == [130, 1, 191, -1]
    assert a[lay.first_pos[1]:lay.first_pos[1] + 4].tolist() == [64, 0, 0, 0]
    assert a[lay.block_table[1]:lay.block_table[1] + 24].reshape(4, 6).tolist() == \
        [[7, -1, 8, -1, -1, -1], [0, -1, -1, -1, -1, -1], [6, 11, -1, -1, -1, -1], [-1] * 6]
    assert a[lay.counts:lay.counts + 2].tolist() == [3, 3]
    # the same requests with two tokens for one of them go the long way
    c = np.full(lay.size, 77, dtype=np.int32)
    slots2 = [[[50], [81, 82], [47]], [[130], [1, 2], [191]]]
    fill_host_buffer(c, lay, [[17], [4, 5], [250]], [130, 1, 31], [2, 0, 1], [False, True, False],
                     slots2, rows, [[0, 0, 0], [64, 0, 0]], [0, 2, 3])
    assert c[lay.positions:lay.positions + 5].tolist() == [130, 1, 2, 31, 0]
    assert c[lay.kv_len:lay.kv_len + 4].tolist() == [131, 3, 32, 0]
    assert np.array_equal(c[lay.block_table[0]:lay.block_table[0] + 24],
                          a[lay.block_table[0]:lay.block_table[0] + 24])
