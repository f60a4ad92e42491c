"""Sampling options and the launch of the kernel that chooses tokens.

Options and their order of operations are the reference's (``src/pretrained/sampling.clj:31-64``):
``temperature`` <= 0 (or no options at all) is greedy, the first largest logit winning;
otherwise the ``top_k`` largest logits (default 40) are kept, softmax of logit / temperature
over them in double precision, the smallest prefix whose cumulative probability reaches
``top_p`` (default 1.0), and a draw from ``java.util.Random(seed)``.  All of it runs on the
device, one block per row; only the chosen ids come back.

The generator's state belongs to the request, not to the cache (``doc/serving-architecture.md:76-79``):
it lives in the request's state slot (``rng_states[slot]``) and is seeded when the request
samples for the first time.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional

import torch

from ..csrc import ops


@dataclass
class SamplingParams:
    """Options of the reference's sampler (``src/pretrained/sampling.clj:31-43``):
    ``temperature`` <= 0 is greedy; otherwise ``top_k`` defaults to 40 and ``top_p`` to
    1.0, and draws come from a generator seeded with ``seed``."""

    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature is None or self.temperature <= 0.0

    def validate(self, vocab: int, max_top_k: int) -> None:
        if self.greedy:
            return
        k = 40 if self.top_k is None else int(self.top_k)
        if k < 1:
            raise ValueError("top_k must be >= 1")
        if min(k, vocab) > max_top_k:
            raise ValueError(f"top_k={k} exceeds the sampling kernel's limit of {max_top_k}")
        p = 1.0 if self.top_p is None else float(self.top_p)
        if not 0.0 < p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")


class Sampler:
    """Host side of the sampling kernel for up to ``rows`` rows a step: pinned staging and
    device copies of the per-row options (two sets, used in turn, so that the set of the step
    in flight is not overwritten), and the per-slot generator states."""

    def __init__(self, rows: int, device, slot_of):
        self.rows = rows
        self.slot_of = slot_of                         # request id -> state slot
        self.rng_states = torch.zeros(rows, dtype=torch.int64, device=device)
        # scratch of the launches that give a row to several CTAs (and their counter)
        self._workspace = torch.zeros(ops.sample_workspace_words(), dtype=torch.int32, device=device)
        self.started: Dict[Hashable, bool] = {}
        self.max_top_k = ops.max_top_k()

        def option_buffers():
            # one pinned buffer and one device buffer hold all six arrays, so that a step's
            # options go to the device in ONE copy; numpy views for the host side (writing
            # tensor elements one by one costs a microsecond each)
            words = rows * (2 + 5)                       # seeds are 8 bytes, the rest 4
            host = torch.zeros(words, dtype=torch.int32, pin_memory=True)
            dev = torch.zeros(words, dtype=torch.int32, device=device)
            names = ("temperature", "top_p", "top_k", "fresh", "slots")
            dtypes = (torch.float32, torch.float32, torch.int32, torch.int32, torch.int32)
            views = {"seeds": (host[:2 * rows].view(torch.int64).numpy(),
                               dev[:2 * rows].view(torch.int64))}
            for j, (name, dtype) in enumerate(zip(names, dtypes)):
                lo = (2 + j) * rows
                views[name] = (host[lo:lo + rows].view(dtype).numpy(), dev[lo:lo + rows].view(dtype))
            return host, dev, views
        self._sets = [option_buffers(), option_buffers()]
        self._sent = [None, None]                      # what each set's device copy holds
        self._turn = 0

    def forget(self, rid: Hashable) -> None:
        """The request has ended; a later request in its slot seeds the generator anew."""
        self.started.pop(rid, None)

    def launch(self, out: torch.Tensor, logits: torch.Tensor, requests: List,
               publish=None) -> None:
        """Launch the kernel that chooses a token for every row (row i belongs to
        ``requests[i]``); nothing synchronises.  ``publish`` = (host address, source, words):
        the kernel also writes these words (the chosen ids among them) to pinned host memory."""
        n = len(requests)
        if all(r.sampling.greedy for r in requests):
            ops.sample(out, logits, n, publish=publish, workspace=self._workspace)
            return
        self._turn ^= 1
        host, dev, p = self._sets[self._turn]
        for i, r in enumerate(requests):
            sp = r.sampling
            p["temperature"][0][i] = 0.0 if sp.greedy else float(sp.temperature)
            p["top_p"][0][i] = 1.0 if sp.top_p is None else float(sp.top_p)
            p["top_k"][0][i] = 40 if sp.top_k is None else int(sp.top_k)
            started = self.started.get(r.rid, False)
            p["fresh"][0][i] = 0 if started else 1
            if not started and not sp.greedy:
                self.started[r.rid] = True
            p["slots"][0][i] = self.slot_of(r.rid)
            if started:
                seed = 0                       # (read only when the generator is seeded)
            elif sp.seed is None:              # unseeded, like java.util.Random() without a seed
                seed = int.from_bytes(os.urandom(6), "little")
            else:
                seed = int(sp.seed)
            p["seeds"][0][i] = seed
        # decoding the same requests, a step's options are the last step's: the device copy of
        # this set is still right and a copy of more than a kilobyte (7 us) is saved
        now = host.numpy().tobytes()
        if self._sent[self._turn] != now:
            dev.copy_(host, non_blocking=True)
            self._sent[self._turn] = now
        ops.sample(out, logits, n, temperature=p["temperature"][1], top_k=p["top_k"][1],
                   top_p=p["top_p"][1], seeds=p["seeds"][1], fresh=p["fresh"][1],
                   slots=p["slots"][1], rng_states=self.rng_states, publish=publish,
                   workspace=self._workspace)
