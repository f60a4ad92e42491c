"""One registry from an architecture's name to its configuration class and model.

Mirrors the reference's architecture registry (``src/pretrained/loader.clj:26-46``):
handlers are registered under their Hugging Face identifiers; lookup tries every
entry of ``architectures[]`` first and ``model_type`` after that; on a miss the
bundled architecture modules are imported once and the lookup is retried
(``loader.clj:69-78, 88-93``); a final miss raises an error that lists what is
registered.
"""
from __future__ import annotations

import importlib
import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Tuple, Type

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Type[ModelConfig]
    #: ``build(config, weight_store, runtime) -> Model``
    build: Callable[..., Any]
    #: ``expected_tensors(config) -> {name: TensorExpectation}``
    expected_tensors: Callable[[ModelConfig], Dict[str, Any]]
    #: ``random_tensors(config, seed, dtype) -> {name: torch.Tensor}``
    random_tensors: Callable[..., Dict[str, Any]]
    #: leading tensor-name parts a checkpoint may carry and the loader removes
    strip_prefixes: Tuple[str, ...] = ()
    #: ``ignorable(name) -> bool``: tensors that may be present without being parameters
    ignorable: Callable[[str], bool] = lambda name: False
    #: named sizes for random-weight models: name -> raw ``config.json`` dict
    named_sizes: Dict[str, Dict[str, Any]] = None


_REGISTRY: Dict[str, Architecture] = {}
_BUNDLED = ("pretrained_rstr_b200.models.gpt2",)
_bundled_loaded = False


def register_architecture(identifiers, architecture: Architecture) -> None:
    """Register ``architecture`` under one identifier or several."""
    if isinstance(identifiers, str):
        identifiers = (identifiers,)
    for ident in identifiers:
        _REGISTRY[ident] = architecture


def registered() -> List[str]:
    _ensure_bundled()
    return sorted(_REGISTRY)


def _ensure_bundled() -> None:
    global _bundled_loaded
    if not _bundled_loaded:
        _bundled_loaded = True
        for module in _BUNDLED:
            importlib.import_module(module)


def dispatch_keys(raw: Dict[str, Any]) -> List[str]:
    """Identifiers to try, in order: ``architectures[]`` entries, then ``model_type``."""
    keys: List[str] = []
    archs = raw.get("architectures") or []
    if isinstance(archs, str):
        archs = [archs]
    keys.extend(str(a) for a in archs)
    if raw.get("model_type"):
        keys.append(str(raw["model_type"]))
    return keys


def lookup(raw: Dict[str, Any]) -> Architecture:
    keys = dispatch_keys(raw)
    for attempt in range(2):
        for key in keys:
            if key in _REGISTRY:
                return _REGISTRY[key]
        if attempt == 0:
            _ensure_bundled()
    raise ConfigError(
        f"No architecture registered for {keys or '<no architectures/model_type key>'}; "
        f"known: {sorted(_REGISTRY)}")


def named_sizes() -> Dict[str, Dict[str, Any]]:
    """Every named size of every registered architecture: name -> raw ``config.json`` dict
    (with its ``architectures`` key), for models made from a size's name and a seed."""
    _ensure_bundled()
    out: Dict[str, Dict[str, Any]] = {}
    for arch in {id(a): a for a in _REGISTRY.values()}.values():
        for name, raw in (arch.named_sizes or {}).items():
            out[name] = dict(raw)
    return out


def named_size(name: str) -> Tuple[Architecture, ModelConfig]:
    sizes = named_sizes()
    if name not in sizes:
        raise ConfigError(f"no size named {name!r}; known: {sorted(sizes)}")
    arch = lookup(sizes[name])
    return arch, arch.config_class.from_dict(sizes[name])


def read_config(folder: str) -> Tuple[Architecture, ModelConfig]:
    """Read ``folder/config.json`` and return (architecture, typed configuration)."""
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path, "r", encoding="utf-8") as fh:
        raw = json.load(fh)
    arch = lookup(raw)
    return arch, arch.config_class.from_dict(raw)
