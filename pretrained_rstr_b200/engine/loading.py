"""From a model folder to a model that can be stepped: configuration and architecture
from ``config.json`` through the registry, weights by name, parts, cache, runner.
The path of the reference's ``from-pretrained`` (``src/pretrained/loader.clj:80-97``)."""
from __future__ import annotations

import contextlib
import shutil
import tempfile
from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.registry import read_config
from ..csrc import ops
from ..settings import SETTINGS
from ..weights.loader import load_weights
from .batch import Runtime
from .runner import ModelRunner

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


@contextlib.contextmanager
def random_model_folder(size: str, seed: int, dtype="bfloat16"):
    """A temporary model folder of a named size with seeded random weights, stored in the
    element type it will run in; removed when the block ends (the weights are on the device
    by then)."""
    from ..config.registry import named_size
    from ..weights.loader import make_random_model
    _arch, config = named_size(size)
    folder = tempfile.mkdtemp(prefix="prb200_random_")
    try:
        make_random_model(folder, config, int(seed), parse_dtype(dtype))
        yield folder
    finally:
        shutil.rmtree(folder, ignore_errors=True)


@dataclass
class LoadedModel:
    folder: str
    architecture: object
    config: object
    runtime: Runtime
    model: object
    cache: CacheManager
    storage: CacheStorage
    runner: ModelRunner


def load_model(folder: str, dtype="bfloat16", device="cuda:0", page_size: int = 64,
               max_batched_tokens: int = 2048, max_requests: int = 64,
               max_tokens: Optional[int] = None, num_pages: Optional[int] = None,
               share_prefixes: bool = False) -> LoadedModel:
    """``max_tokens``: the most tokens live requests hold at any time, each request's
    count rounded up to whole pages; the page pools are made for that many.  Default:
    ``max_requests`` requests of full length."""
    ops.require_cuda()
    ops.lib()                                   # build / load now, fail loudly here
    ops.set_pdl(SETTINGS.pdl)
    dtype = parse_dtype(dtype)
    device = torch.device(device)
    torch.cuda.set_device(device)
    arch, config = read_config(folder)
    runtime = Runtime(device=device, dtype=dtype, page_size=page_size,
                      max_batched_tokens=max_batched_tokens, max_requests=max_requests,
                      use_graphs=SETTINGS.graphs)
    store = load_weights(folder, arch.expected_tensors(config), device,
                         strip_prefixes=arch.strip_prefixes, ignorable=arch.ignorable)
    model = arch.build(config, store, runtime)
    store.release()
    if num_pages is None:
        if max_tokens is None:
            max_tokens = max_requests * (-(-config.max_positions // page_size) * page_size)
        num_pages = max(1, -(-max_tokens // page_size))
    pages = [num_pages] * len(model.group_specs)
    storage = CacheStorage(model.group_specs, pages, page_size, dtype, device,
                           model.state_specs, max_requests)
    # A model whose parts keep state of fixed size per request cannot skip shared prompt
    # tokens (their state updates would never run), and a fork has to copy the state rows.
    cache = CacheManager(model.group_specs, page_size, pages if pages else 1, max_requests,
                         config.max_positions, share_prefixes=share_prefixes,
                         has_state=bool(model.state_specs), copy_state=storage.copy_state)
    runner = ModelRunner(model, runtime, cache, storage)
    return LoadedModel(folder, arch, config, runtime, model, cache, storage, runner)
