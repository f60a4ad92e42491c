"""The cache manager: pages, block tables, groups of layers, and state slots.

Pure bookkeeping, no tensors: it decides *which* page holds which tokens; device
memory lives in :mod:`pretrained_rstr_b200.cache.storage`.  The vocabulary follows
the reference's page pool (``src/pretrained/continuation/page_pool.clj``):

* a **page** holds ``page_size`` consecutive tokens of one request for every layer of
  one group (``page_pool.clj:4-6``); free pages are handed out lowest index first
  (``:513-524``) and carry a reference count (``:296-303``);
* a request's **block table** lists its pages in position order (the reference's
  *route*, ``:670-674``); the device form is padded with -1 (``:1423-1446``);
* a new token's **slot** is ``page * page_size + offset`` (``paged_append.clj:44-57``);
* appending is a transaction: :meth:`CacheManager.reserve` hands out slots and is
  invisible until :meth:`commit`; :meth:`abort` gives back what it took
  (``page_pool.clj:902-973, 1003-1023, 1031-1061``);
* a request may **fork** another at any length and shares the covering pages
  (``:679-724``); the first append into a shared, partly filled page copies it first
  (copy-on-write, ``:926-944``);
* full pages of a prompt are found again through a chained hash of their tokens
  (``continuation/chunk.clj:33-51``); a hit is confirmed by comparing the tokens.

Beyond the reference: **groups**.  Layers with different needs (all keys, or only a
window of them) form groups with page pools and block tables of their own; a windowed
group gives pages back as soon as the window has passed them.  And **state slots**:
fixed-size per-request state, one slot per live request, for parts that keep a state
instead of (or beside) keys and values.
"""
from __future__ import annotations

import hashlib
import heapq
import struct
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """No free page is left in a group (after evicting what may be evicted)."""


@dataclass(frozen=True)
class GroupSpec:
    """Layers that share one page pool.

    ``layers``   cache-layer indices stored in this group, in storage order.
    ``window``   None: every key is kept.  w: token i needs keys j with i-w < j <= i.
    """

    name: str
    layers: Tuple[int, ...]
    kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def elements_per_token(self) -> int:
        return self.kv_heads * self.head_dim


class PageAllocator:
    """Free set (lowest first) and reference counts of one group's pages."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages))
        heapq.heapify(self._free)
        self.refcount = [0] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = heapq.heappop(self._free)
        assert self.refcount[page] == 0, f"page {page} handed out while held"
        self.refcount[page] = 1
        return page

    def retain(self, page: int) -> None:
        if self.refcount[page] <= 0:
            raise CacheError(f"retain of free page {page}")
        self.refcount[page] += 1

    def release(self, page: int) -> bool:
        """Drop one reference; True when the page became free."""
        if self.refcount[page] <= 0:
            raise CacheError(f"page {page} freed twice")
        self.refcount[page] -= 1
        if self.refcount[page] == 0:
            heapq.heappush(self._free, page)
            return True
        return False


class SlotAllocator:
    """Fixed number of per-request state slots, lowest first."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots))
        heapq.heapify(self._free)
        self._held = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise CacheError("no free state slot")
        slot = heapq.heappop(self._free)
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"state slot {slot} freed twice")
        self._held.remove(slot)
        heapq.heappush(self._free, slot)


class _Table(list):
    """A block table (pages by logical index, -1 for a page given back) that keeps its
    device form up to date: ``row``, the same pages padded with -1 to the longest table a
    request can have.  A step copies rows; it does not rebuild them."""

    __slots__ = ("row", "held")

    def __init__(self, row: np.ndarray, pages: Sequence[int] = ()):
        super().__init__(pages)
        self.row = row
        self.held = sum(1 for p in self if p >= 0)      # pages not given back
        row[:] = -1
        if len(self):
            row[:len(self)] = self

    def append(self, page: int) -> None:
        self.row[len(self)] = page
        self.held += 1 if page >= 0 else 0
        super().append(page)

    def pop(self) -> int:                  # the last page only
        page = super().pop()
        self.held -= 1 if page >= 0 else 0
        self.row[len(self)] = -1
        return page

    def __setitem__(self, index: int, page: int) -> None:
        self.held += (1 if page >= 0 else 0) - (1 if self[index] >= 0 else 0)
        super().__setitem__(index, page)
        self.row[index] = page


@dataclass
class _Pending:
    count: int
    new_pages: List[Tuple[int, int, int]]          # (group, logical index, page)
    swapped: List[Tuple[int, int, int, int]]       # (group, logical index, old page, new page)


@dataclass
class Reservation:
    """What :meth:`CacheManager.reserve` hands to the step function."""

    start: int                                     # position of the first new token
    count: int
    slots: List[List[int]]                         # [group][token] physical slot
    copies: List[Tuple[int, int, int]]             # (group, source page, destination page)


@dataclass
class _Request:
    rid: Hashable
    slot: int
    length: int = 0                                # committed tokens
    tables: List[List[int]] = field(default_factory=list)   # [group][logical page] or -1
    tokens: List[int] = field(default_factory=list)         # committed token ids (for the index)
    pending: Optional[_Pending] = None
    fresh: bool = True                             # no step has run for it yet
    promise: List[int] = field(default_factory=list)        # pages promised at admission, per group
    indexed_pages: int = 0                         # full pages already offered to the index
    chain: bytes = b""                             # hash chain up to indexed_pages

    def held(self, group: int) -> int:
        return self.tables[group].held


def chain_hash(parent: bytes, tokens: Sequence[int]) -> bytes:
    """Hash of one full page given its parent's hash: domain tag, parent, count and the
    token ids as fixed-width big-endian integers (``continuation/chunk.clj:33-51``)."""
    h = hashlib.sha256()
    h.update(b"pretrained-rstr-b200/page/v1")
    h.update(struct.pack(">I", len(parent)))
    h.update(parent)
    h.update(struct.pack(">q", len(tokens)))
    h.update(struct.pack(f">{len(tokens)}q", *tokens))
    return h.digest()


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int,
                 num_pages: Sequence[int] | int, num_slots: int,
                 max_positions: int, share_prefixes: bool = False, has_state: bool = False,
                 copy_state=None):
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        self.allocators = [PageAllocator(n) for n in num_pages]
        self.slots = SlotAllocator(num_slots)
        self.max_positions = max_positions
        self.max_pages_per_request = -(-max_positions // page_size)
        self.requests: Dict[Hashable, _Request] = {}
        # the block tables in their device form, by group: one row per state slot
        self.table_rows = [np.full((num_slots, self.max_pages_per_request), -1, dtype=np.int32)
                           for _ in self.groups]
        # Sharing full prompt pages needs every group to keep all its pages, and a model
        # without fixed-size state per request: a request that takes over shared pages skips
        # their tokens, so a part that keeps a state would never see them
        # (``doc/serving-architecture.md:76-79``: per-request state is no reusable attention
        # state).
        self.has_state = bool(has_state)
        self.copy_state = copy_state           # (source slot, destination slot) -> None
        self.share_prefixes = share_prefixes and not self.has_state and \
            all(g.window is None for g in self.groups)
        # chain hash -> (pages per group, tokens of that page); LRU order.
        self._index: "OrderedDict[bytes, Tuple[Tuple[int, ...], Tuple[int, ...]]]" = OrderedDict()
        # which pages the index names, and how many of them nobody else holds (what an
        # admission may count on besides the free pages), kept up to date where reference
        # counts change: asking must not cost a walk over the index
        self._indexed = [bytearray(a.num_pages) for a in self.allocators]
        self._cached = [0] * len(self.groups)
        self.stats = {"allocated": 0, "released": 0, "window_released": 0, "cow_copies": 0,
                      "prefix_hits": 0, "evicted": 0}

    # ------------------------------------------------------------------ capacity
    def pages_needed(self, group: int, total_tokens: int, longest_step: int = 1) -> int:
        """Pages of ``group`` a request of ``total_tokens`` can hold at once."""
        g = self.groups[group]
        full = -(-total_tokens // self.page_size)
        if g.window is None:
            return full
        span = g.window + max(1, longest_step) - 1
        return min(full, -(-span // self.page_size) + 1)

    def available(self, group: int) -> int:
        """Pages that could be handed out now: free ones plus those only the prefix index
        holds, minus what admissions were promised."""
        alloc = self.allocators[group]
        outstanding = 0
        for r in self.requests.values():
            short = r.promise[group] - r.tables[group].held
            if short > 0:
                outstanding += short
        return alloc.free_count + self._cached[group] - outstanding

    # ------------------------------------------------------------------ requests
    def open(self, rid: Hashable, reserve_tokens: Optional[int] = None,
             longest_step: int = 1) -> int:
        """Register a request and give it a state slot.  With ``reserve_tokens`` the pages
        it may need are promised to it now (``page_pool.clj:567-611``) and the call
        raises :class:`OutOfPages`, changing nothing, if they cannot be."""
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already open")
        reserved = [0] * len(self.groups)
        if reserve_tokens is not None:
            if reserve_tokens > self.max_positions:
                raise CacheError(
                    f"request {rid!r} wants {reserve_tokens} tokens; the model holds "
                    f"{self.max_positions} positions")
            for gi in range(len(self.groups)):
                need = self.pages_needed(gi, reserve_tokens, longest_step)
                if need > self.allocators[gi].num_pages:
                    raise CacheError(
                        f"request {rid!r} needs {need} pages of group "
                        f"{self.groups[gi].name!r}; the pool has {self.allocators[gi].num_pages}")
                if need > self.available(gi):
                    raise OutOfPages(
                        f"group {self.groups[gi].name!r}: {need} pages wanted, "
                        f"{self.available(gi)} available")
                reserved[gi] = need
        if self.slots.free_count == 0:
            raise CacheError("no free state slot")
        slot = self.slots.allocate()
        self.requests[rid] = _Request(rid=rid, slot=slot,
                                      tables=[_Table(rows[slot]) for rows in self.table_rows],
                                      promise=reserved)
        return slot

    def close(self, rid: Hashable) -> None:
        """The request is finished: every page and its state slot are given back."""
        req = self._get(rid)
        if req.pending is not None:
            self.abort(rid)
        for gi, table in enumerate(req.tables):
            for page in table:
                if page >= 0:
                    self._release(gi, page)
        for rows in self.table_rows:
            rows[req.slot] = -1
        self.slots.release(req.slot)
        del self.requests[rid]

    def fork(self, source: Hashable, rid: Hashable, length: Optional[int] = None) -> int:
        """Open ``rid`` as a copy of the first ``length`` tokens of ``source``: the covering
        pages are shared, not copied (``page_pool.clj:679-724``)."""
        src = self._get(source)
        if src.pending is not None:
            raise CacheError("cannot fork a request with a pending append")
        length = src.length if length is None else length
        if not 0 <= length <= src.length:
            raise CacheError(f"fork length {length} outside [0, {src.length}]")
        for g in self.groups:
            if self._first_live_page(g, length) < self._first_live_page(g, src.length):
                raise CacheError("fork point lies before a page the window already released")
        if self.has_state and length > 0:
            # the state slot holds the state after the source's last token and no other
            if length != src.length:
                raise CacheError(
                    f"the model keeps per-request state: request {source!r} can be forked at its "
                    f"present length {src.length} only, not at {length}")
            if self.copy_state is None:
                raise CacheError("the model keeps per-request state and no state copy was given: "
                                 "it cannot be forked")
        slot = self.open(rid)
        req = self.requests[rid]
        if self.has_state and length > 0:
            self.copy_state(src.slot, slot)
        req.fresh = False if length > 0 else True
        n_pages = -(-length // self.page_size)
        for gi in range(len(self.groups)):
            req.tables[gi] = _Table(self.table_rows[gi][slot], src.tables[gi][:n_pages])
            for page in req.tables[gi]:
                if page >= 0:
                    self._retain(gi, page)
        req.length = length
        req.tokens = list(src.tokens[:length])
        return slot

    # -------------------------------------------------------------- prefix index
    def match_prefix(self, rid: Hashable, prompt: Sequence[int]) -> int:
        """Share every indexed full page that matches the start of ``prompt``; returns
        the number of tokens the request now holds.  The page that will receive the
        prompt's last token is never shared: that token has to be computed."""
        req = self._get(rid)
        if not self.share_prefixes or req.length or req.pending:
            return req.length
        ps = self.page_size
        chain = b""
        shared = 0
        while (shared + 1) * ps < len(prompt):
            tokens = tuple(prompt[shared * ps:(shared + 1) * ps])
            key = chain_hash(chain, tokens)
            hit = self._index.get(key)
            if hit is None or hit[1] != tokens:
                break
            self._index.move_to_end(key)
            for gi, page in enumerate(hit[0]):
                self._retain(gi, page)
                req.tables[gi].append(page)
            chain = key
            shared += 1
            self.stats["prefix_hits"] += 1
        req.length = shared * ps
        req.tokens = list(prompt[:req.length])
        req.indexed_pages = shared
        req.chain = chain
        if shared:
            req.fresh = False
        return req.length

    def page_keys(self, prompt: Sequence[int]) -> List[bytes]:
        """The chained hashes under which the prompt's full pages would be found in the prefix
        index, in order (none where nothing is shared; never the page that holds the prompt's
        last token, which is always computed)."""
        if not self.share_prefixes:
            return []
        ps = self.page_size
        keys: List[bytes] = []
        chain = b""
        while (len(keys) + 1) * ps < len(prompt):
            chain = chain_hash(chain, tuple(prompt[len(keys) * ps:(len(keys) + 1) * ps]))
            keys.append(chain)
        return keys

    def is_indexed(self, key: bytes) -> bool:
        return key in self._index

    def _offer_full_pages(self, req: _Request) -> None:
        ps = self.page_size
        while (req.indexed_pages + 1) * ps <= req.length and \
                len(req.tokens) >= (req.indexed_pages + 1) * ps:
            i = req.indexed_pages
            tokens = tuple(req.tokens[i * ps:(i + 1) * ps])
            key = chain_hash(req.chain, tokens)
            if key not in self._index:
                pages = tuple(req.tables[gi][i] for gi in range(len(self.groups)))
                for gi, page in enumerate(pages):
                    self._retain(gi, page)
                    self._indexed[gi][page] = 1          # (held by the request too: not counted)
                self._index[key] = (pages, tokens)
            else:
                self._index.move_to_end(key)
            req.chain = key
            req.indexed_pages += 1

    def _evict_one(self, group: int) -> bool:
        """Drop the least recently used index entry that only the index holds."""
        for key, (pages, _) in self._index.items():
            if all(self.allocators[gi].refcount[p] == 1 for gi, p in enumerate(pages)):
                del self._index[key]
                for gi, p in enumerate(pages):
                    self._indexed[gi][p] = 0
                    self._cached[gi] -= 1
                    self._release(gi, p)
                self.stats["evicted"] += 1
                return True
        return False

    # ---------------------------------------------------------------- appending
    def reserve(self, rid: Hashable, count: int) -> Reservation:
        """Slots for the next ``count`` tokens of ``rid``.  Nothing is visible to others
        until :meth:`commit`; :meth:`abort` undoes it."""
        req = self._get(rid)
        if req.pending is not None:
            raise CacheError(f"request {rid!r} already has a pending append")
        if count <= 0:
            raise CacheError("reserve needs a positive token count")
        if req.length + count > self.max_positions:
            raise CacheError(
                f"request {rid!r}: {req.length}+{count} tokens exceed {self.max_positions} positions")
        ps = self.page_size
        pending = _Pending(count=count, new_pages=[], swapped=[])
        slots: List[List[int]] = []
        copies: List[Tuple[int, int, int]] = []
        try:
            for gi in range(len(self.groups)):
                table = req.tables[gi]
                group_slots: List[int] = []
                pos, end = req.length, req.length + count
                while pos < end:                       # page by page, not token by token
                    li, off = divmod(pos, ps)
                    if li == len(table):
                        page = self._allocate(gi, req)
                        table.append(page)
                        pending.new_pages.append((gi, li, page))
                    else:
                        page = table[li]
                        if page < 0:
                            raise CacheError("append into a released page")
                        if pos == req.length and self.allocators[gi].refcount[page] > 1:
                            # shared, partly filled tail: copy before the first write
                            new = self._allocate(gi, req)
                            copies.append((gi, page, new))
                            pending.swapped.append((gi, li, page, new))
                            table[li] = new
                            self.stats["cow_copies"] += 1
                    n = min(ps - off, end - pos)
                    first = table[li] * ps + off
                    group_slots.extend(range(first, first + n))
                    pos += n
                slots.append(group_slots)
        except Exception:
            req.pending = pending
            self.abort(rid)
            raise
        req.pending = pending
        return Reservation(start=req.length, count=count, slots=slots, copies=copies)

    def commit(self, rid: Hashable, tokens: Optional[Sequence[int]] = None) -> None:
        """The reserved tokens now belong to the request.  Shared pages a copy replaced
        lose this request's reference; pages a window has passed are given back."""
        req = self._get(rid)
        if req.pending is None:
            raise CacheError(f"request {rid!r} has nothing to commit")
        for gi, _li, old, _new in req.pending.swapped:
            self._release(gi, old)
        if tokens is not None:
            if len(tokens) != req.pending.count:
                raise CacheError("commit: token count differs from the reservation")
            if len(req.tokens) == req.length:
                req.tokens.extend(tokens if type(tokens) is list else [int(t) for t in tokens])
        req.length += req.pending.count
        req.pending = None
        req.fresh = False
        if self.share_prefixes:
            self._offer_full_pages(req)
        self._release_passed(req)

    def abort(self, rid: Hashable) -> None:
        req = self._get(rid)
        if req.pending is None:
            return
        for gi, li, old, new in reversed(req.pending.swapped):
            req.tables[gi][li] = old
            self._release(gi, new)
        for gi, li, page in reversed(req.pending.new_pages):
            assert req.tables[gi][-1] == page and len(req.tables[gi]) == li + 1
            req.tables[gi].pop()
            self._release(gi, page)
        req.pending = None

    # ------------------------------------------------------------------ windows
    def _first_live_page(self, group: GroupSpec, length: int) -> int:
        """Index of the first page a request of ``length`` committed tokens still needs:
        the next query sits at position ``length`` and sees keys j > length - window."""
        if group.window is None:
            return 0
        first_needed = max(0, length - group.window + 1)
        return first_needed // self.page_size

    def _release_passed(self, req: _Request) -> None:
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            table = req.tables[gi]
            for li in range(min(self._first_live_page(g, req.length), len(table))):
                if table[li] >= 0:
                    self._release(gi, table[li])
                    table[li] = -1
                    self.stats["window_released"] += 1

    # ------------------------------------------------------------------ queries
    def length(self, rid: Hashable) -> int:
        return self._get(rid).length

    def peek(self, rid: Hashable) -> _Request:
        """The request's record, to read ``slot``, ``length`` and ``fresh`` from in one
        look-up; not to be changed by the caller."""
        return self._get(rid)

    def slot(self, rid: Hashable) -> int:
        return self._get(rid).slot

    def is_fresh(self, rid: Hashable) -> bool:
        return self._get(rid).fresh

    def block_table(self, rid: Hashable, group: int) -> List[int]:
        """Pages of ``rid`` in ``group`` by logical index, as they are now (a pending
        append included: the step attends over what it is about to write)."""
        return list(self._get(rid).tables[group])

    def first_visible(self, rid: Hashable, group: int) -> int:
        """Lowest position whose page the request still holds in ``group``."""
        req = self._get(rid)
        return self._first_live_page(self.groups[group], req.length) * self.page_size

    def free_pages(self, group: int = 0) -> int:
        return self.allocators[group].free_count

    def check(self) -> None:
        """Invariant: every page's reference count equals the number of block tables and
        index entries that name it; free pages are named by nobody."""
        for gi, alloc in enumerate(self.allocators):
            counts = [0] * alloc.num_pages
            for req in self.requests.values():
                seen = set()
                for page in req.tables[gi]:
                    if page >= 0:
                        if page in seen:
                            raise CacheError(f"page {page} twice in one block table")
                        seen.add(page)
                        counts[page] += 1
                if req.pending is not None:
                    for g2, _li, old, _new in req.pending.swapped:
                        if g2 == gi:
                            counts[old] += 1
            for pages, _ in self._index.values():
                counts[pages[gi]] += 1
            if counts != alloc.refcount:
                raise CacheError(f"group {gi}: reference counts {alloc.refcount} != uses {counts}")
            free = sorted(alloc._free)
            if len(set(free)) != len(free):
                raise CacheError("a page is twice in the free set")
            if any(alloc.refcount[p] for p in free):
                raise CacheError("a held page is in the free set")
            if len(free) + sum(1 for c in alloc.refcount if c) != alloc.num_pages:
                raise CacheError("a page is lost")
            named = bytearray(alloc.num_pages)
            for pages, _ in self._index.values():
                named[pages[gi]] = 1
            if named != self._indexed[gi]:
                raise CacheError(f"group {gi}: the record of indexed pages differs from the index")
            alone = sum(1 for pages, _ in self._index.values() if alloc.refcount[pages[gi]] == 1)
            if alone != self._cached[gi]:
                raise CacheError(f"group {gi}: {self._cached[gi]} pages counted as held by the index "
                                 f"alone, {alone} are")
            rows = self.table_rows[gi]
            held_slots = set()
            for req in self.requests.values():
                held_slots.add(req.slot)
                table = req.tables[gi]
                if table.held != sum(1 for p in table if p >= 0):
                    raise CacheError(f"request {req.rid!r}: held-page count differs from the table")
                if rows[req.slot, :len(table)].tolist() != list(table) or \
                        bool((rows[req.slot, len(table):] != -1).any()):
                    raise CacheError(f"request {req.rid!r}: the device form of its block table "
                                     f"differs from the table")
            for slot in range(rows.shape[0]):
                if slot not in held_slots and bool((rows[slot] != -1).any()):
                    raise CacheError(f"state slot {slot} is free and its block table row is not empty")

    # ----------------------------------------------------------------- internals
    def _get(self, rid: Hashable) -> _Request:
        try:
            return self.requests[rid]
        except KeyError:
            raise CacheError(f"unknown request {rid!r}") from None

    def _allocate(self, gi: int, req: _Request) -> int:
        alloc = self.allocators[gi]
        promised = req.promise[gi] > req.held(gi)
        if not promised and self.available(gi) <= 0:
            # Not covered by an admission promise: may not eat into others' promises.
            raise OutOfPages(
                f"group {self.groups[gi].name!r}: no page left for request {req.rid!r}")
        while alloc.free_count == 0:
            if not self._evict_one(gi):
                raise OutOfPages(
                    f"group {self.groups[gi].name!r}: no page left for request {req.rid!r}")
        page = alloc.allocate()
        self.stats["allocated"] += 1
        return page

    def _retain(self, gi: int, page: int) -> None:
        alloc = self.allocators[gi]
        alloc.retain(page)
        if self._indexed[gi][page] and alloc.refcount[page] == 2:
            self._cached[gi] -= 1                        # no longer the index's alone

    def _release(self, gi: int, page: int) -> None:
        alloc = self.allocators[gi]
        alloc.release(page)
        if self._indexed[gi][page] and alloc.refcount[page] == 1:
            self._cached[gi] += 1                        # only the index holds it now
        self.stats["released"] += 1
