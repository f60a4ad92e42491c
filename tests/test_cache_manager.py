"""The cache manager without a GPU: pages, block tables, transactions, windows,
sharing, copy-on-write, state slots, and random orders of requests."""
import random

import pytest

from pretrained_rstr_b200.cache import (CacheError, CacheManager, GroupSpec, OutOfPages,
                                        PageAllocator, SlotAllocator)

FULL = GroupSpec("full", (0, 1), 4, 16, None)
WIN = GroupSpec("win", (2,), 2, 16, 40)


def test_allocator_lowest_first_and_double_free():
    a = PageAllocator(4)
    assert [a.allocate() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        a.allocate()
    a.release(2)
    a.release(0)
    assert a.allocate() == 0
    with pytest.raises(CacheError, match="freed twice"):
        a.release(2)
    a.retain(1)
    assert a.release(1) is False and a.release(1) is True
    s = SlotAllocator(2)
    assert (s.allocate(), s.allocate()) == (0, 1)
    s.release(0)
    with pytest.raises(CacheError, match="freed twice"):
        s.release(0)


def test_slots_are_consecutive_and_invisible_until_commit():
    cm = CacheManager([FULL], 16, 8, 4, 128)
    cm.open("a")
    r = cm.reserve("a", 20)
    assert r.start == 0 and r.slots[0] == list(range(20))
    assert cm.length("a") == 0
    with pytest.raises(CacheError, match="pending"):
        cm.reserve("a", 1)
    cm.commit("a")
    assert cm.length("a") == 20 and cm.block_table("a", 0) == [0, 1]
    r = cm.reserve("a", 13)
    assert r.start == 20 and r.slots[0][:2] == [20, 21] and r.slots[0][-1] == 2 * 16
    cm.abort("a")
    assert cm.block_table("a", 0) == [0, 1] and cm.free_pages(0) == 6
    cm.check()
    cm.close("a")
    assert cm.free_pages(0) == 8 and cm.slots.free_count == 4
    with pytest.raises(CacheError, match="unknown request"):
        cm.close("a")


def test_pages_run_out_and_reserve_leaves_nothing_behind():
    cm = CacheManager([FULL], 16, 3, 4, 128)
    cm.open("a")
    cm.open("b")
    cm.reserve("a", 32)
    cm.commit("a")
    with pytest.raises(OutOfPages):
        cm.reserve("b", 17)
    cm.check()
    assert cm.free_pages(0) == 1 and cm.block_table("b", 0) == []
    with pytest.raises(CacheError, match="exceed"):
        cm.reserve("a", 128)


def test_window_group_gives_pages_back():
    cm = CacheManager([FULL, WIN], 16, [8, 6], 4, 128)
    cm.open("a")
    for n in (50, 30, 20, 28):
        cm.reserve("a", n)
        cm.commit("a")
        cm.check()
    assert cm.length("a") == 128
    table = cm.block_table("a", 1)
    # next query at position 128 would see keys > 88: pages 0..4 are passed
    assert table[:5] == [-1] * 5 and all(p >= 0 for p in table[5:])
    assert cm.first_visible("a", 1) == 80
    assert all(p >= 0 for p in cm.block_table("a", 0))
    assert cm.stats["window_released"] == 5
    cm.close("a")
    assert cm.free_pages(0) == 8 and cm.free_pages(1) == 6


def test_fork_shares_and_copies_on_write():
    cm = CacheManager([FULL], 16, 8, 4, 128)
    cm.open("root")
    cm.reserve("root", 40)
    cm.commit("root")
    cm.fork("root", "child", 36)
    assert cm.block_table("child", 0) == cm.block_table("root", 0) == [0, 1, 2]
    assert cm.allocators[0].refcount[:3] == [2, 2, 2]
    r = cm.reserve("child", 2)                  # tail page is shared and partly filled
    assert r.copies == [(0, 2, 3)] and r.slots[0] == [3 * 16 + 4, 3 * 16 + 5]
    assert cm.block_table("root", 0) == [0, 1, 2]          # the root is untouched
    cm.abort("child")                            # abort undoes the copy
    assert cm.block_table("child", 0) == [0, 1, 2] and cm.allocators[0].refcount[3] == 0
    cm.check()
    r = cm.reserve("child", 2)
    cm.commit("child")
    assert cm.block_table("child", 0) == [0, 1, 3] and cm.allocators[0].refcount[2] == 1
    r = cm.reserve("root", 1)                    # root's tail is its own again: no copy
    assert r.copies == []
    cm.commit("root")
    cm.fork("root", "edge", 32)                  # fork at a page boundary shares only full pages
    assert cm.block_table("edge", 0) == [0, 1]
    assert cm.reserve("edge", 1).copies == []
    cm.commit("edge")
    cm.check()
    for rid in ("root", "child", "edge"):
        cm.close(rid)
    assert cm.free_pages(0) == 8


def test_prefix_pages_are_found_again_and_evicted_when_needed():
    cm = CacheManager([FULL], 4, 6, 4, 64, share_prefixes=True)
    prompt = list(range(100, 111))               # 11 tokens: two full pages + 3
    cm.open("a")
    assert cm.match_prefix("a", prompt) == 0
    cm.reserve("a", 11)
    cm.commit("a", prompt)
    cm.close("a")
    assert cm.free_pages(0) == 4                 # two full pages stay, held by the index
    cm.open("b")
    assert cm.match_prefix("b", prompt) == 8
    assert cm.block_table("b", 0) == [0, 1] and cm.stats["prefix_hits"] == 2
    cm.open("c")
    assert cm.match_prefix("c", prompt[:8]) == 4      # never the page of the last prompt token
    assert cm.match_prefix("c", [1, 2, 3]) == 4       # only an empty request may match
    cm.close("c")
    cm.open("d")
    assert cm.match_prefix("d", [100, 101, 102, 999, 104, 105, 106, 107, 108]) == 0
    cm.close("d")
    cm.close("b")
    cm.check()
    cm.open("big")                               # needs all six pages: cached ones are evicted
    cm.reserve("big", 24)
    cm.commit("big", list(range(24)))
    assert cm.stats["evicted"] == 2
    cm.check()


def test_admission_promises_pages():
    cm = CacheManager([FULL], 16, 6, 4, 96)
    cm.open("a", reserve_tokens=64)              # promised 4 pages, none taken yet
    assert cm.available(0) == 2
    with pytest.raises(OutOfPages):
        cm.open("b", reserve_tokens=48)
    assert "b" not in cm.requests and cm.slots.free_count == 3
    cm.open("b", reserve_tokens=32)
    cm.open("c")                                 # no promise: may not eat into others'
    with pytest.raises(OutOfPages):
        cm.reserve("c", 1)
    cm.reserve("a", 64)
    cm.commit("a")
    cm.reserve("b", 32)
    cm.commit("b")
    cm.close("a")
    assert cm.available(0) == 4
    with pytest.raises(CacheError, match="positions"):
        cm.open("d", reserve_tokens=97)
    cm.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    """Open, append (commit or abort), fork and close in random order: after every
    operation no page is lost, held twice or freed twice; at the end all are free."""
    rng = random.Random(seed)
    groups = [FULL, WIN] if seed % 2 else [FULL]
    cm = CacheManager(groups, 8, [24, 10][:len(groups)], 5, 96,
                      share_prefixes=(seed % 2 == 0))
    live, counter = {}, 0
    for _ in range(400):
        op = rng.random()
        try:
            if op < 0.2 and len(live) < 5:
                rid = f"r{counter}"
                counter += 1
                if live and rng.random() < 0.3 and len(groups) == 1:
                    src = rng.choice(list(live))
                    cm.fork(src, rid, rng.randint(0, cm.length(src)))
                    live[rid] = list(live[src][:cm.length(rid)])
                else:
                    cm.open(rid)
                    live[rid] = []
                    if rng.random() < 0.5:
                        prompt = [rng.randrange(3) for _ in range(rng.randint(1, 30))]
                        got = cm.match_prefix(rid, prompt)
                        live[rid] = prompt[:got]
            elif op < 0.8 and live:
                rid = rng.choice(list(live))
                n = rng.randint(1, 20)
                if cm.length(rid) + n > 96:
                    continue
                cm.reserve(rid, n)
                if rng.random() < 0.2:
                    cm.abort(rid)
                else:
                    toks = [rng.randrange(3) for _ in range(n)]
                    cm.commit(rid, toks)
                    live[rid] += toks
                assert cm.length(rid) == len(live[rid])
            elif live:
                rid = rng.choice(list(live))
                cm.close(rid)
                del live[rid]
        except OutOfPages:
            pass
        cm.check()
    for rid in list(live):
        cm.close(rid)
    cm.check()
    while cm._evict_one(0):
        pass
    for gi, alloc in enumerate(cm.allocators):
        assert alloc.free_count == alloc.num_pages
    assert cm.slots.free_count == 5


def test_state_keeping_models_share_no_prefix_and_fork_with_their_state():
    """A model whose parts keep fixed-size state per request: a request that took over cached
    pages would skip their tokens and never run their state updates, so sharing is off; a fork
    copies the source's state row, and is refused at any length but the source's present one."""
    copied = []
    cm = CacheManager([FULL], 16, 8, 4, 128, share_prefixes=True, has_state=True,
                      copy_state=lambda src, dst: copied.append((src, dst)))
    assert cm.share_prefixes is False
    cm.open("a")
    cm.reserve("a", 40)
    cm.commit("a", list(range(40)))
    cm.open("b")
    assert cm.match_prefix("b", list(range(40))) == 0 and cm.is_fresh("b")
    cm.close("b")
    with pytest.raises(CacheError, match="present length"):
        cm.fork("a", "c", 32)
    assert "c" not in cm.requests
    slot = cm.fork("a", "c")
    assert copied == [(cm.slot("a"), slot)] and cm.length("c") == 40 and not cm.is_fresh("c")
    empty = cm.fork("a", "d", 0)                      # nothing to copy: it starts fresh
    assert len(copied) == 1 and cm.is_fresh("d") and empty != slot
    cm.check()
    bare = CacheManager([FULL], 16, 8, 4, 128, has_state=True)
    bare.open("a")
    bare.reserve("a", 5)
    bare.commit("a")
    with pytest.raises(CacheError, match="no state copy"):
        bare.fork("a", "b")


def test_block_tables_keep_their_device_form():
    """Each table's row (padded with -1, by state slot) follows appends, copy-on-write
    swaps, aborted reservations, pages a window has passed, forks and the request's end."""
    groups = [GroupSpec("all", (0,), 2, 16), GroupSpec("near", (1,), 2, 16, window=20)]
    cm = CacheManager(groups, page_size=16, num_pages=[12, 12], num_slots=3, max_positions=96)
    sa = cm.open("a")
    cm.reserve("a", 40)
    assert cm.table_rows[0][sa].tolist() == cm.block_table("a", 0) + [-1] * 3
    cm.abort("a")
    assert cm.table_rows[0][sa].tolist() == [-1] * 6
    cm.reserve("a", 40)
    cm.commit("a")
    cm.check()
    assert cm.table_rows[1][sa].tolist()[:3] == cm.block_table("a", 1) and \
        cm.table_rows[1][sa][0] == -1                      # the window has passed page 0
    sb = cm.fork("a", "b")
    assert cm.table_rows[0][sb].tolist() == cm.table_rows[0][sa].tolist()
    cm.reserve("b", 1)                                      # copies the shared, partly filled page
    cm.commit("b")
    assert cm.table_rows[0][sb][2] != cm.table_rows[0][sa][2]
    assert cm.table_rows[0][sb].tolist()[:3] == cm.block_table("b", 0)
    cm.check()
    cm.close("a")
    assert cm.table_rows[0][sa].tolist() == [-1] * 6 and cm.table_rows[1][sa].tolist() == [-1] * 6
    cm.check()
    cm.close("b")
    cm.check()
