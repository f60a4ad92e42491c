"""Puts a model together from a configuration's layer specifications.

Nothing here is specific to one architecture: the configuration says, as data, which
parts each layer has (``layer_specs()``), in which order layers run and whose cache
each run reads (``run_order()``), and which embedding, position encoding, final norm
and head surround them.  The reference assembles its decoders from descriptors in the
same spirit (``src/pretrained/arch/llama.clj:22-45``,
``src/pretrained/decoder_gpu.clj:122-133``).

Cache groups are derived here: every cache layer whose mixer keeps keys and values
declares (kv heads, head size, window); layers with equal needs share a group, i.e. a
page pool and block tables of their own
(``src/pretrained/continuation/attention_state.clj:52-84`` declares slabs the same way).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..cache.manager import GroupSpec
from ..parts import build_part, part_factory
from ..parts.interfaces import LayerCache, StateSpec
from ..parts.linear import LazyNorm


class Model:
    def __init__(self, config, runtime, embedding, position, blocks, order, final_norm, head,
                 width: int, vocab: int):
        self.config, self.runtime = config, runtime
        self.embedding, self.position = embedding, position
        self.blocks, self.order = blocks, order
        self.final_norm, self.head = final_norm, head
        self.width, self.vocab = width, vocab
        self.max_positions = config.max_positions
        # cache layout
        self.group_specs: List[GroupSpec] = []
        self.layer_group: Dict[int, Tuple[int, int]] = {}     # cache layer -> (group, index)
        self.state_specs: Dict[Tuple[int, str], StateSpec] = {}
        self._derive_cache_layout()
        self._caches: List[LayerCache] = []
        # a step can be replayed as a CUDA graph only if every part launches the same
        # kernels whatever the step holds (parts say so with ``graph_safe = True``)
        parts = [embedding, position, final_norm, head]
        for blk in blocks:
            parts += [blk, blk.mixer, blk.feed_forward, *blk.norms.values()]
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in parts)
        # work lists the parts want in every step's description, one planner per key
        self.planners = []
        for part in parts:
            for planner in getattr(part, "work_planners", lambda: [])():
                kept = [have for have in self.planners if have.key == planner.key]
                if not kept:
                    self.planners.append(planner)
                elif kept[0] is not planner:
                    kept[0].absorb(planner)

    # ---------------------------------------------------------------- cache layout
    def _derive_cache_layout(self) -> None:
        writers = {e.cache_layer for e in self.order if e.writes_cache}
        for e in self.order:
            if e.cache_layer not in writers:
                raise ValueError(f"run order: layer {e.layer} reads the cache of layer "
                                 f"{e.cache_layer}, which no entry writes")
        keyed: Dict[Tuple[int, int, object], List[int]] = {}
        for layer in sorted(writers):
            mixer = self.blocks[layer].mixer
            spec = mixer.kv_spec()
            if spec is not None:
                keyed.setdefault((spec.kv_heads, spec.head_dim, spec.window), []).append(layer)
            for st in mixer.state_specs():
                self.state_specs[(layer, st.name)] = st
        for (kv_heads, head_dim, window), layers in sorted(
                keyed.items(), key=lambda kv: kv[1][0]):
            name = "full" if window is None else f"window{window}"
            gi = len(self.group_specs)
            self.group_specs.append(GroupSpec(f"{name}.{gi}", tuple(layers), kv_heads, head_dim,
                                              window))
            for idx, layer in enumerate(layers):
                self.layer_group[layer] = (gi, idx)
        for e in self.order:
            reader = self.blocks[e.layer].mixer.kv_spec()
            if reader is not None and e.cache_layer in self.layer_group:
                g = self.group_specs[self.layer_group[e.cache_layer][0]]
                if (reader.kv_heads, reader.head_dim) != (g.kv_heads, g.head_dim):
                    raise ValueError(f"run order: layer {e.layer} cannot read the cache of layer "
                                     f"{e.cache_layer}: head counts or sizes differ")

    def attach_storage(self, storage) -> None:
        """Bind every run entry to the pages and state tensors of its cache layer."""
        self._caches = []
        for e in self.order:
            cache = LayerCache(writes=e.writes_cache)
            if e.cache_layer in self.layer_group:
                gi, idx = self.layer_group[e.cache_layer]
                cache.group = gi
                cache.k, cache.v = storage.layer_pages(gi, idx)
            cache.state = {name: t for (layer, name), t in storage.state.items()
                           if layer == e.cache_layer}
            self._caches.append(cache)

    # --------------------------------------------------------------------- forward
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's tokens through the model; returns float32 logits [rows, vocab]
        for ``ctx.logit_rows`` (a view of scratch memory whose rows are padded to a multiple
        of 32 elements: copy it to keep it)."""
        t = ctx.launch_tokens
        x = ctx.scratch("residual", (ctx.token_capacity, self.width), torch.float32)[:t]
        self.embedding.forward(ctx, self.position, x)
        for entry, cache in zip(self.order, self._caches):
            self.blocks[entry.layer].forward(ctx, x, cache)
        r = ctx.launch_rows
        if r == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=x.device)
        hn = ctx.scratch("final_normed", (ctx.row_capacity(r), self.width), self.runtime.dtype)[:r]
        # (a head that can norm its few rows itself does: the norm then is no kernel of its own)
        lazy = getattr(self.head, "accepts_lazy_norm", False)
        h_in = LazyNorm(ctx, self.final_norm, x, hn, rows=ctx.logit_rows) if lazy else hn
        if not lazy:
            self.final_norm.forward(ctx, x, hn, rows=ctx.logit_rows)
        # rows 128 bytes apart at least: a vocabulary that is no multiple of 4 (GPT-2's 50,257)
        # would otherwise put every row at an odd address, which the products' epilogues can
        # only store element by element
        pitch = -(-self.vocab // 32) * 32
        logits = ctx.scratch("logits", (ctx.row_capacity(r), pitch), torch.float32)[:r, :self.vocab]
        self.head.forward(ctx, h_in, logits)
        return logits


def build_model(config, store, runtime) -> Model:
    specs = config.layer_specs()
    blocks = []
    for spec in specs:
        mixer = build_part("mixer", spec.mixer, store, runtime)
        ff = build_part("feed_forward", spec.feed_forward, store, runtime)
        norms = {name: build_part("norm", ns, store, runtime) for name, ns in spec.norms.items()}
        blocks.append(part_factory("arrangement", spec.arrangement)(mixer, ff, norms, spec.width,
                                                                    runtime))
    position = build_part("position", config.position_spec(), store, runtime)
    for block in blocks:                      # rotary-style encodings act inside the mixer
        if hasattr(block.mixer, "position") and block.mixer.position is None:
            block.mixer.position = position
    embedding = build_part("embedding", config.embedding_spec(), store, runtime)
    final_norm = build_part("norm", config.final_norm_spec(), store, runtime)
    head = build_part("head", config.head_spec(), store, runtime)
    order = config.run_order()
    for e in order:
        if not (0 <= e.layer < len(blocks)) or not (0 <= e.cache_layer < len(blocks)):
            raise ValueError(f"run order names layer {e.layer}/{e.cache_layer}; "
                             f"the model has {len(blocks)}")
    emb = config.embedding_spec().params
    return Model(config, runtime, embedding, position, blocks, order, final_norm, head,
                 width=emb["width"], vocab=config.head_spec().params["vocab"])
