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

import os

from typing import Optional

import torch

from ..csrc import ops
from ..engine.batch import SINGLE_MAX_Q
from .interfaces import KVSpec, LayerCache, Mixer, PositionEncoding
from .linear import Linear
from .registry import register_part


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

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.n_kv_head, self.head_dim, self.window)

    def forward(self, ctx, h, x, cache: LayerCache) -> None:
        t = x.shape[0]
        dtype = self.runtime.dtype
        qkv = ctx.scratch("attn_qkv", (ctx.token_capacity, self.qkv.n_out), dtype)[:t]
        group = ctx.groups[cache.group]
        # With no rotation of keys to wait for, the decode-time product may write the new
        # keys and values to their cache slots itself.
        rotates = self.position is not None and \
            type(self.position).rotate is not PositionEncoding.rotate
        scatter = (cache.k, cache.v, group.slots, self.q_width) \
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
        attend(ctx, o, q, cache, group, self.n_head, self.scale, self.window)
        self.out.forward(ctx, o, x, resid=x)


DECODE_CTAS = int(os.environ.get("PRB200_DECODE_CTAS", "768"))
USE_TC = os.environ.get("PRB200_ATTN_TC", "1") != "0"


PREFILL_PART = int(os.environ.get("PRB200_PREFILL_PART", "-1"))     # blocks per key part; -1: choose


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
    if PREFILL_PART >= 0:
        part = PREFILL_PART
    elif items > 74 or blocks < 8:
        part = 0
    else:
        # about as many CTAs as run at a time (two per SM), parts of at least four blocks
        part = max(4, -(-items * blocks // (2 * 296)))
    if part <= 0 or part >= blocks:
        return 0, 1
    part = max(part, -(-blocks // (ops.PREFILL_MAX_PARTS - 1)))
    return part, -(-blocks // part) + (1 if window else 0)


def attend(ctx, out, q, cache: LayerCache, group, n_head: int, scale: float,
           window: Optional[int]) -> None:
    """Attention of the step's tokens over their requests' cached keys and values.

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
    lay = ctx.layout
    if ctx.n_tiles is None or ctx.n_tiles > 0:
        n_tiles = lay.tile_cap if ctx.n_tiles is None else ctx.n_tiles
        if USE_TC and ops.prefill_tc_supports(head_dim, group.page_size):
            # (a step that runs as a graph is planned with its capacities: the most tiles and
            # the longest context it may have)
            parts = None
            part_blocks, max_parts = prefill_key_parts(n_tiles * n_head, ctx.max_context, window)
            if part_blocks:
                units = 1 << max(6, (n_tiles * n_head - 1).bit_length())
                parts = (ctx.scratch("attn_part_o", (units * max_parts * 8192,), torch.float32),
                         ctx.scratch("attn_part_ml", (units * max_parts * 256,), torch.float32),
                         ctx.scratch_zero("attn_part_count", (units,), torch.int32))
            ops.attention_prefill_tc(out, q, cache.k, cache.v, group.block_table, ctx.positions,
                                     ctx.tile_req, ctx.tile_row0, ctx.tile_rows, ctx.counts[0:1],
                                     n_tiles, n_head, scale, window, ctx.status,
                                     part_blocks=part_blocks, max_parts=max_parts, parts=parts)
        else:
            ops.attention_prefill(out, q, cache.k, cache.v, group.block_table, ctx.positions,
                                  ctx.tile_req, ctx.tile_row0, ctx.tile_rows, ctx.counts[0:1],
                                  n_tiles, n_head, scale, window, ctx.status)
    if ctx.n_singles is None or ctx.n_singles > 0:
        n_list = lay.single_cap if ctx.n_singles is None else ctx.n_singles
        # about five CTAs per SM (the kernel's leaner instance fits six): many (token, head)
        # pairs get fewer, longer splits, and one each when there are more pairs than that
        granule = ops.decode_split()
        most = -(-ctx.max_context // granule)
        pairs = max(1, n_list * n_head)
        if pairs < DECODE_CTAS:
            wanted = -(-DECODE_CTAS // pairs)
        else:
            wanted = 1
        wanted = max(1, min(most, wanted))
        split_keys = -(-ctx.max_context // wanted // granule) * granule
        max_splits = -(-ctx.max_context // split_keys)
        cap = ctx.runtime.max_requests * SINGLE_MAX_Q
        ws = ctx.scratch("attn_decode_ws", (cap * n_head * ctx.max_splits_cap * (head_dim + 4),),
                         torch.float32)
        counters = ctx.scratch_zero("attn_decode_counters", (cap * n_head,), torch.int32)
        ops.attention_decode(out, q, cache.k, cache.v, group.block_table, ctx.seq_of_token,
                             ctx.positions, ctx.single_tokens, ctx.counts[1:2], n_list, n_head,
                             scale, window, ws, counters, max_splits, ctx.status,
                             split_keys=split_keys)


def _causal_attention(p, store, rt) -> CausalAttention:
    width, nh, nkv, dh = p["width"], p["n_head"], p["n_kv_head"], p["head_dim"]
    layout = p.get("weight_layout", "out_in")
    qkv = Linear.from_store(store, p["weights"]["qkv"], layout, width, (nh + 2 * nkv) * dh,
                            p.get("bias", False), rt)
    out = Linear.from_store(store, p["weights"]["out"], layout, nh * dh, width,
                            p.get("bias", False), rt)
    return CausalAttention(qkv, out, width, nh, nkv, dh, p["scale"], p.get("window"), rt)


register_part("mixer", "causal_attention", _causal_attention)
