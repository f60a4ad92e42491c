"""pretrained_rstr_b200: a small, whole GPT-2 inference engine for one B200.

The task API follows the reference's ``pretrained.lm`` (``src/pretrained/lm.clj``):

    m = load_lm("/path/to/model", gpu=True)           # (load-lm k dir {:gpu? true})
    ids = generate_ids(m, prompt_ids, 20)             # (generate-ids m ids n)
    ids = generate_ids(m, prompt_ids, 20, {"temperature": 0.8, "top_k": 40, "seed": 7})
    out = generate_text(m, prompt, 20)                # (generate-text m prompt n)

Everything runs on the CUDA device through this package's own kernels; there is no
CPU path (``gpu=False`` is refused).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

__version__ = "0.1.0"


class LM:
    """A loaded language model with its engine (the reference's model map with
    ``::mode :gpu`` and a bound decoder, ``lm.clj:103-115``)."""

    def __init__(self, loaded, engine, eos_ids=(), tokenizer=None):
        self.loaded = loaded
        self.engine = engine
        self.config = loaded.config
        self.eos_ids = tuple(eos_ids)
        self.tokenizer = tokenizer

    def stats(self):
        return self.engine.stats()


def _eos_ids(folder: str) -> tuple:
    """``generation_config.json``'s ``eos_token_id`` when the folder has one
    (``src/pretrained/chat.clj:94-120``); a folder of random weights has none."""
    import json
    import os
    path = os.path.join(folder, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    with open(path, "r", encoding="utf-8") as fh:
        eos = json.load(fh).get("eos_token_id")
    if eos is None:
        return ()
    return tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))


def load_lm(path: str, opts: Optional[Dict] = None, *, gpu: bool = True,
            dtype: str = "bfloat16", device_id: str = "cuda:0", maxpos: Optional[int] = None,
            page_size: int = 64, max_lanes: int = 64, max_batched_tokens: int = 2048,
            prefill_chunk: int = 512, max_tokens: Optional[int] = None,
            share_prefixes: bool = True) -> LM:
    """Load the model folder ``path`` (``config.json`` + ``model.safetensors``); the model
    class is chosen by ``config.json``.  Options, by the reference's names where it has
    them (``lm.clj:94-115``): ``gpu`` (must be true), ``device_id``, ``maxpos``: the most
    tokens a request may hold (default and upper bound: the model's positions).  ``opts``
    may give the same options as a dict (``{"gpu?": True, "maxpos": 2048}``)."""
    from .engine.engine import Engine
    from .engine.loading import load_model
    from .engine.scheduler import SchedulerOptions
    if opts:
        gpu = bool(opts.get("gpu?", opts.get("gpu", gpu)))
        device_id = opts.get("device-id", opts.get("device_id", device_id))
        maxpos = opts.get("maxpos", maxpos)
        dtype = opts.get("dtype", dtype)
    if not gpu:
        raise ValueError("pretrained_rstr_b200 has no CPU path: load_lm(..., gpu=True) only")
    from .config.registry import read_config
    _arch, config = read_config(path)
    per_request = config.max_positions if maxpos is None else min(int(maxpos), config.max_positions)
    if max_tokens is None:
        max_tokens = max_lanes * (-(-per_request // page_size) * page_size)
    loaded = load_model(path, dtype=dtype, device=device_id, page_size=page_size,
                        max_batched_tokens=max_batched_tokens, max_requests=max_lanes,
                        max_tokens=max_tokens, share_prefixes=share_prefixes)
    engine = Engine(loaded, SchedulerOptions(
        max_batched_tokens=max_batched_tokens, max_lanes=max_lanes,
        prefill_chunk=min(prefill_chunk, max_batched_tokens),
        minimum_prefill_tokens=1 if max_lanes > 1 else 0))
    return LM(loaded, engine, eos_ids=_eos_ids(path))


def _sampling(opts: Optional[Dict]):
    from .engine.scheduler import SamplingParams
    if not opts:                        # empty options = greedy (sampling.clj:37-38)
        return SamplingParams()
    known = {"temperature", "top_k", "top-k", "top_p", "top-p", "seed"}
    unknown = set(opts) - known
    if unknown:
        raise ValueError(f"unknown sampling options {sorted(unknown)}; known: {sorted(known)}")
    return SamplingParams(
        temperature=float(opts.get("temperature", 1.0)),
        top_k=opts.get("top_k", opts.get("top-k")),
        top_p=opts.get("top_p", opts.get("top-p")),
        seed=opts.get("seed"))


def generate_ids(m: LM, prompt_ids: Sequence[int], n: int, opts: Optional[Dict] = None) -> List[int]:
    """Prompt token ids -> the n generated ids.  ``opts``: ``temperature``, ``top_k``,
    ``top_p``, ``seed``; empty = greedy (``lm.clj:117-124``, ``sampling.clj:31-43``).
    Generation stops early at a stop token (kept in the output) or when the model's
    positions are used up (``decoder_gpu.clj:1293-1295``)."""
    return m.engine.generate([list(prompt_ids)], n, _sampling(opts), m.eos_ids)[0]


def generate_batch(m: LM, prompts: Sequence[Sequence[int]], n: int,
                   opts: Optional[Dict] = None) -> List[List[int]]:
    """Several prompts at once through the continuous-batching scheduler."""
    return m.engine.generate([list(p) for p in prompts], n, _sampling(opts), m.eos_ids)


def generate_text(m: LM, prompt: Union[str, Sequence[int]], n: int,
                  opts: Optional[Dict] = None):
    """Encode ``prompt``, generate n tokens, decode (``lm.clj:126-135``).  A model folder
    without tokenizer files takes and returns token ids."""
    if isinstance(prompt, str):
        if m.tokenizer is None:
            raise ValueError("this model folder has no tokenizer; pass token ids")
        ids = m.tokenizer.encode(prompt)
        return m.tokenizer.decode(generate_ids(m, ids, n, opts))
    return generate_ids(m, prompt, n, opts)


__all__ = ["LM", "load_lm", "generate_ids", "generate_batch", "generate_text"]
