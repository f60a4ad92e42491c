"""Causal attention over the paged cache as a mixer.

Order inside a layer follows the reference's paged decoder
(``src/pretrained/continuation/paged_decoder.clj:266-278``): project Q, K, V; write the
new keys and values to their slots; attend over the block table, the step's own
tokens included; project the result and add it to the residual stream.

Sizes and constants are parameters: width, number of query heads and of key/value
heads (groups), head size, score scale, window, whether the projections have biases,
and the checkpoint's weight layout.  The fused QKV matrix has columns [Q | K | V]
(``dev/examples/gpt2.clj:186-194``); head h owns columns h*head_dim..(h+1)*head_dim of
its part.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from ..engine.batch import WorkPlanner
from ..settings import SETTINGS
from .interfaces import KVSpec, LayerCache, Mixer, PositionEncoding
from .linear import Linear
from .registry import register_part


class AttentionWork(WorkPlanner):
    """How the attention kernels cut a step: portions of prompts go in tiles of up to
    ``TILE`` queries of one request to the prompt kernels; decoded tokens and portions of
    up to ``SINGLE_MAX_Q`` tokens go token by token to the decode kernels.

    For the tensor-memory prompt kernel the tiles are also listed as work ITEMS, longest
    first: a tile as a whole, or, where that balances the step better, a tile's keys in parts
    of ``part_blocks`` blocks of ``KEY_BLOCK`` absolute positions, a CTA each, merged by the
    last to finish.  A tile's time goes with its number of key blocks (plus about four
    blocks' worth of set-up), a late tile of a long prompt has many times an early one's, and
    a launch lasts as long as its longest CTA: 2 x 1,024 tokens of GPT-2 small are 192 (tile,
    head) CTAs of 2 to 16 blocks, 25 us a launch, where 360 CTAs of at most 6 blocks need 15.
    The list holds exactly the CTAs that have work: CTAs that find nothing to do and leave
    at once do not give their place on an SM to a waiting CTA until much later (measured)."""

    key = "causal_attention"
    counters = ("tiles", "singles", "items")
    wants_starts = True
    # CTAs that find nothing to do keep a waiting CTA from its place on an SM for
    # microseconds: a replayed step launches the items it has (rounded up), not the capacity
    launch_steps = {"items": (8, "item_tile")}
    TILE = 128
    SINGLE_MAX_Q = 4
    KEY_BLOCK = 64
    MAX_PARTS = 8                       # most parts of one tile
    MIN_PART = 4                        # blocks: a part costs about as much as four besides its own

    def __init__(self):
        self.heads = 1                  # most query heads of the mixers that use the lists
        self.window: Optional[int] = None
        self.sm_count = 148             # (set from the device when a mixer is built on one)

    def note_mixer(self, heads: int, window: Optional[int], sm_count: Optional[int]) -> None:
        """What a mixer that uses the lists needs them planned for."""
        self.heads = int(heads)
        self.window = window or None
        if sm_count:
            self.sm_count = int(sm_count)

    def absorb(self, other: "AttentionWork") -> None:
        """The mixers of a model share one planner: the lists are balanced for the most heads
        any of them has, and parts are planned for one window (the first mixer's; a mixer with
        another window has its tiles' chunks taken by grid index instead)."""
        self.heads = max(self.heads, other.heads)
        if other.sm_count != 148:
            self.sm_count = other.sm_count

    def slot_cap(self) -> int:
        """Most part slots (parts of split tiles) a step may use."""
        return max(16, 4 * self.sm_count // self.heads)

    def arrays(self, t_cap: int, b_cap: int):
        tile_cap = t_cap // self.TILE + b_cap
        item_cap = tile_cap + self.slot_cap()
        # (the single tokens first: a decode step uses nothing of what follows, and what a
        # step does not use is not copied to the device)
        return {"single_tokens": (min(t_cap, b_cap * self.SINGLE_MAX_Q), 0),
                "tile_req": (tile_cap, -1), "tile_row0": (tile_cap, 0), "tile_rows": (tile_cap, 0),
                "part_blocks": (1, 0),
                "item_tile": (item_cap, 0), "item_part": (item_cap, -1), "item_slot": (item_cap, 0)}

    def fill(self, arrays: Dict[str, np.ndarray], lengths: Sequence[int],
             starts: Optional[Sequence[int]] = None) -> Dict[str, int]:
        treq, trow, tnum = arrays["tile_req"], arrays["tile_row0"], arrays["tile_rows"]
        sing = arrays["single_tokens"]
        n_tiles = n_sing = 0
        t = 0
        spans = []                      # (first key block, last key block) of every tile
        if max(lengths) == 1:           # a decode step: every token is a single one
            n_sing = len(lengths)
            sing[:n_sing] = np.arange(n_sing, dtype=np.int32)
            lengths = ()
        for b, n in enumerate(lengths):
            if n <= self.SINGLE_MAX_Q:
                sing[n_sing:n_sing + n] = np.arange(t, t + n, dtype=np.int32)
                n_sing += n
            else:
                for r0 in range(0, n, self.TILE):
                    rows = min(self.TILE, n - r0)
                    treq[n_tiles] = b
                    trow[n_tiles] = t + r0
                    tnum[n_tiles] = rows
                    pos0 = (starts[b] if starts is not None else 0) + r0
                    lo = max(0, pos0 - self.window + 1) if self.window else 0
                    spans.append((lo // self.KEY_BLOCK, (pos0 + rows - 1) // self.KEY_BLOCK))
                    n_tiles += 1
            t += n
        n_items = self._items(arrays, spans) if spans and "item_tile" in arrays else 0
        used = (["single_tokens"] if n_sing else []) + \
            (["tile_req", "tile_row0", "tile_rows", "part_blocks", "item_tile", "item_part", "item_slot"]
             if n_tiles else [])
        return {"tiles": n_tiles, "singles": n_sing, "items": n_items, "_used": used}

    def _split(self, spans, blocks, part):
        """The items for parts of ``part`` blocks: (blocks of the item, tile, part or -1, slot)."""
        items, slots = [], 0
        for tile in sorted(range(len(spans)), key=lambda i: -blocks[i]):
            first, last = spans[tile]
            n_parts = last // part - first // part + 1
            if blocks[tile] < part + 2 or n_parts < 2 or slots + n_parts > self.slot_cap():
                items.append((blocks[tile], tile, -1, 0))
                continue
            for z in range(n_parts):
                lo = max(first, (first // part + z) * part)
                hi = min(last, (first // part + z) * part + part - 1)
                items.append((hi - lo + 1, tile, z, slots + z))
            slots += n_parts
        return items

    def _items(self, arrays, spans) -> int:
        """The tiles as work items, longest first, the long ones in parts: the smallest parts
        (of at least ``MIN_PART`` blocks) with which all CTAs still run at once, two to an SM
        (every part costs its CTA a set-up and a merge, so a second round of short CTAs is
        dearer than a first round of longer ones)."""
        itile, ipart, islot = arrays["item_tile"], arrays["item_part"], arrays["item_slot"]
        blocks = [last - first + 1 for first, last in spans]
        longest = max(blocks, default=0)
        part = max(self.MIN_PART, -(-longest // self.MAX_PARTS))
        items = self._split(spans, blocks, part)
        while part < longest and (len(items) * self.heads > 2 * self.sm_count or len(items) > len(itile)):
            part += 1
            items = self._split(spans, blocks, part)
        if len(items) > len(itile):
            items = [(blocks[i], i, -1, 0) for i in range(len(spans))]
        items.sort(key=lambda it: -it[0])
        for i, (_n, tile, z, slot) in enumerate(items):
            itile[i], ipart[i], islot[i] = tile, z, slot
        arrays["part_blocks"][0] = part
        return len(items)


class CausalAttention(Mixer):
    graph_safe = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself
    def __init__(self, qkv: Linear, out: Linear, width: int, n_head: int, n_kv_head: int,
                 head_dim: int, scale: float, window: Optional[int], runtime,
                 position=None):
        if n_head % n_kv_head != 0:
            raise ValueError(f"causal_attention: {n_head} query heads are not a multiple of "
                             f"{n_kv_head} key/value heads")
        self.q_width = n_head * head_dim
        self.kv_width = n_kv_head * head_dim
        if qkv.n_out != self.q_width + 2 * self.kv_width or qkv.n_in != width:
            raise ValueError("causal_attention: fused QKV matrix has the wrong shape")
        if out.n_in != self.q_width or out.n_out != width:
            raise ValueError("causal_attention: output projection has the wrong shape")
        self.qkv, self.out = qkv, out
        self.width, self.n_head, self.n_kv_head, self.head_dim = width, n_head, n_kv_head, head_dim
        self.scale, self.window = float(scale), window
        self.runtime = runtime
        self.position = position
        self.work_plan = AttentionWork()
        self.work_plan.note_mixer(n_head, window, ops.sm_count() if torch.cuda.is_available() else None)

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.n_kv_head, self.head_dim, self.window)

    def work_planners(self):
        return [self.work_plan]

    def forward(self, ctx, h, x, cache: LayerCache) -> None:
        t = x.shape[0]
        dtype = self.runtime.dtype
        qkv = ctx.scratch("attn_qkv", (ctx.token_capacity, self.qkv.n_out), dtype)[:t]
        group = ctx.groups[cache.group]
        # With no rotation of keys to wait for, the decode-time product may write the new
        # keys and values to their cache slots itself.
        rotates = self.position is not None and \
            type(self.position).rotate is not PositionEncoding.rotate
        # (a step without single tokens reads keys and values from the cache alone: the product
        # need not store those columns beside the queries as well)
        singles = ctx.work[AttentionWork.key].host_counts.get("singles")
        scatter = (cache.k, cache.v, group.slots, self.q_width, singles == 0) \
            if cache.writes and not rotates else None
        appended = self.qkv.forward(ctx, h, qkv, kv_scatter=scatter)
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if rotates:
            self.position.rotate(ctx, q, k)
        if cache.writes and not appended:
            ops.kv_append(cache.k, cache.v, k, v, group.slots, t, ctx.status)
        o = ctx.scratch("attn_out", (ctx.token_capacity, self.q_width), dtype)[:t]
        # (the step's own keys and values lie beside the queries exactly as the cache got them)
        last = attend(ctx, o, q, cache, group, self.n_head, self.scale, self.window,
                      kv_new=(k, v) if cache.writes else None)
        # After the split-key decode kernel (hundreds of small CTAs, several to an SM) the
        # projection is launched the plain way: placed early, its CTAs take room beside them
        # on the SMs and the pair lasts longer (measured, a layer of GPT-2 small: 30.3 -> 29.5
        # us at 8 requests, 25.5 -> 24.1 us at one).
        with ops.plain_launch(last == "split"):
            self.out.forward(ctx, o, x, resid=x)


def prefill_key_parts(items: int, max_context: int, window: Optional[int]):
    """(blocks per part, most parts per item) for the tensor-memory prompt kernel; (0, 1):
    one CTA per item.  Splitting an item's keys over several CTAs costs each of them a
    part written and a merge (about 5 microseconds, as much as four blocks of keys), so it
    pays only while the items alone leave most SMs empty.  Measured on a B200, kernel alone:
    8 items of up to 16 blocks 17.4 -> 12.1 us in parts of 4, 128 items of up to 128 blocks
    128 -> 70 us in parts of 32, 192 items of up to 16 blocks 23.0 -> 26.9 us; in a GPT-2
    small step: 512 tokens at positions 512 to 1,023 (48 items) 0.991 -> 0.953 ms, a whole
    prompt of 1,024 (96 items) 1.07 -> 1.11 ms.  Hence: only up to 74 items (half the SMs)."""
    span = min(max_context, window + 128) if window else max_context
    blocks = -(-span // 64) + (1 if window else 0)
    sms = ops.sm_count()
    if SETTINGS.prefill_part >= 0:
        part = SETTINGS.prefill_part
    elif items > sms // 2 or blocks < 8:
        part = 0
    else:
        # about as many CTAs as run at a time (two per SM), parts of at least four blocks
        part = max(4, -(-items * blocks // (4 * sms)))
    if part <= 0 or part >= blocks:
        return 0, 1
    part = max(part, -(-blocks // (ops.PREFILL_MAX_PARTS - 1)))
    return part, -(-blocks // part) + (1 if window else 0)


def attend(ctx, out, q, cache: LayerCache, group, n_head: int, scale: float,
           window: Optional[int], kv_new=None) -> Optional[str]:
    """Attention of the step's tokens over their requests' cached keys and values.  Returns
    which kernel ran last: "ring", "split" (the split-key decode kernel) or None.

    float32 runtime: the 32-bit kernel for every token.  bfloat16 runtime: prompt
    portions go in tiles of up to 128 queries to a tensor-core kernel (tcgen05 for head
    size 64 and pages of a multiple of 64, else mma.sync), single tokens (decoded
    tokens, portions of a few tokens) to the split-key decode kernel; head sizes or page
    sizes those kernels do not take fall back to the 32-bit-arithmetic kernel."""
    t = out.shape[0]
    head_dim = cache.k.shape[3]
    fast = ctx.dtype == torch.bfloat16 and head_dim % 8 == 0 and head_dim <= 256 and \
        group.page_size >= 8 and ops.decode_split() % group.page_size == 0 and \
        ops.prefill_supports(head_dim)
    if not fast:
        ops.attention_generic(out, q, cache.k, cache.v, group.block_table, ctx.seq_of_token,
                              ctx.positions, t, n_head, scale, window, ctx.max_context, ctx.status)
        return
    work = ctx.work[AttentionWork.key]
    planner = work.planner
    tiles, singles = work.host_counts["tiles"], work.host_counts["singles"]
    tile_req, tile_row0, tile_rows = (work.arrays[n] for n in ("tile_req", "tile_row0", "tile_rows"))
    if tiles is None or tiles > 0:
        n_tiles = work.caps["tile_req"] if tiles is None else tiles
        if SETTINGS.attention_tcgen05 and ops.prefill_tc_supports(head_dim, group.page_size):
            if SETTINGS.prefill_part < 0 and "item_tile" in work.arrays and planner is not None \
                    and planner.window == (window or None):
                # the planner's list: exactly the CTAs that have work, longest first, long
                # tiles in parts (a step that runs as a graph is planned with its capacities)
                items = work.host_counts["items"]
                n_items = work.launch.get("items", work.caps["item_tile"]) if items is None else items
                n_slots = planner.slot_cap()
                parts = (ctx.scratch("attn_part_o", (n_slots * n_head * 8192,), torch.float32),
                         ctx.scratch("attn_part_ml", (n_slots * n_head * 256,), torch.float32),
                         ctx.scratch_zero("attn_part_count", (n_slots * n_head,), torch.int32))
                ops.attention_prefill_tc(out, q, cache.k, cache.v, group.block_table, ctx.positions,
                                         tile_req, tile_row0, tile_rows, work.counts["tiles"],
                                         n_tiles, n_head, scale, window, ctx.status, parts=parts,
                                         items=(work.arrays["item_tile"], work.arrays["item_part"],
                                                work.arrays["item_slot"], work.counts["items"],
                                                work.arrays["part_blocks"], n_items, n_slots))
            else:
                # (a forced chunk size, or a mixer whose heads or window the planner did not
                # plan for: chunks by grid index)
                parts = None
                part_blocks, max_parts = prefill_key_parts(n_tiles * n_head, ctx.max_context, window)
                if part_blocks:
                    units = 1 << max(6, (n_tiles * n_head - 1).bit_length())
                    parts = (ctx.scratch("attn_part_o2", (units * max_parts * 8192,), torch.float32),
                             ctx.scratch("attn_part_ml2", (units * max_parts * 256,), torch.float32),
                             ctx.scratch_zero("attn_part_count2", (units,), torch.int32))
                ops.attention_prefill_tc(out, q, cache.k, cache.v, group.block_table, ctx.positions,
                                         tile_req, tile_row0, tile_rows, work.counts["tiles"],
                                         n_tiles, n_head, scale, window, ctx.status,
                                         part_blocks=part_blocks, max_parts=max_parts, parts=parts)
        else:
            ops.attention_prefill(out, q, cache.k, cache.v, group.block_table, ctx.positions,
                                  tile_req, tile_row0, tile_rows, work.counts["tiles"],
                                  n_tiles, n_head, scale, window, ctx.status)
    if singles is None or singles > 0:
        n_list = work.caps["single_tokens"] if singles is None else singles
        cap = ctx.runtime.max_requests * AttentionWork.SINGLE_MAX_Q
        ring = SETTINGS.decode_ring
        if ring is None:
            ring = ops.decode_ring_prefers(n_list, n_head, ctx.max_context)
        if ring and cap <= ops.decode_ring_max_list() and \
                ops.decode_ring_supports(head_dim, group.page_size):
            ws = ctx.scratch("attn_ring_ws", (ops.decode_ring_workspace(cap, n_head, head_dim),),
                             torch.float32)
            counters = ctx.scratch_zero("attn_decode_counters", (cap * n_head,), torch.int32)
            ops.attention_decode_ring(out, q, cache.k, cache.v, group.block_table,
                                      ctx.seq_of_token, ctx.positions, work.arrays["single_tokens"],
                                      work.counts["singles"], n_list, n_head, scale, window, ws,
                                      counters, ctx.status, new_keys=AttentionWork.SINGLE_MAX_Q,
                                      max_context=ctx.max_context, kv_new=kv_new)
            return "ring"
        split_keys, max_splits = decode_splits(n_list * n_head, ctx.max_context, group.page_size)
        # room for the shortest splits any step may choose
        splits_cap = -(-ctx.max_positions // ops.decode_split())
        ws = ctx.scratch("attn_decode_ws", (cap * n_head * splits_cap * (head_dim + 4),),
                         torch.float32)
        counters = ctx.scratch_zero("attn_decode_counters", (cap * n_head,), torch.int32)
        ops.attention_decode(out, q, cache.k, cache.v, group.block_table, ctx.seq_of_token,
                             ctx.positions, work.arrays["single_tokens"], work.counts["singles"],
                             n_list, n_head, scale, window, ws, counters, max_splits, ctx.status,
                             split_keys=split_keys)
        return "split"
    return None


def decode_splits(pairs: int, max_context: int, page_size: int):
    """(keys per split, most splits per (token, head)) of the decode kernel for a launch of
    ``pairs`` (token, head) pairs over contexts of up to ``max_context`` keys.  The launch
    should have about five CTAs per SM: many pairs get fewer, longer splits, and one each when
    there are more pairs than that.  A split is a multiple of the kernel's granule and spans
    no more pages than the kernel holds page ids for."""
    granule = ops.decode_split()
    target = SETTINGS.decode_ctas or 768 * ops.sm_count() // 148
    most = -(-max_context // granule)
    pairs = max(1, pairs)
    wanted = -(-target // pairs) if pairs < target else 1
    wanted = max(1, min(most, wanted))
    split_keys = -(-max_context // wanted // granule) * granule
    longest = ops.decode_max_split_pages() * page_size // granule * granule
    split_keys = max(granule, min(split_keys, longest))
    return split_keys, -(-max_context // split_keys)


def _causal_attention(p, store, rt) -> CausalAttention:
    width, nh, nkv, dh = p["width"], p["n_head"], p["n_kv_head"], p["head_dim"]
    layout = p.get("weight_layout", "out_in")
    qkv = Linear.from_store(store, p["weights"]["qkv"], layout, width, (nh + 2 * nkv) * dh,
                            p.get("bias", False), rt)
    out = Linear.from_store(store, p["weights"]["out"], layout, nh * dh, width,
                            p.get("bias", False), rt)
    return CausalAttention(qkv, out, width, nh, nkv, dh, p["scale"], p.get("window"), rt)


register_part("mixer", "causal_attention", _causal_attention)
