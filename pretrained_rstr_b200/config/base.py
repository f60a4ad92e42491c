"""Typed model configurations and the data that describes how layers are arranged.

A configuration class reads the architecture's own ``config.json`` keys once, applies
defaults in one place and validates them (the reference normalises hyper-parameters
the same way: ``src/pretrained/decoder.clj:36-56``).  Everything downstream takes its
sizes and constants from the configuration object; no size lives in code.

Besides sizes, a configuration answers two structural questions as *data*:

``layer_specs()``
    one :class:`LayerSpec` per layer: which mixer, feed-forward, norm and arrangement
    that layer uses, each with its own parameters, so different layers of one model
    may be built from different parts.

``run_order()``
    a list of :class:`RunEntry`: which layer runs when, and whose cache it uses.  A
    layer may appear twice, and an entry may read another layer's cache.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the chosen architecture."""


@dataclass(frozen=True)
class PartSpec:
    """Names a registered part (``kind``) and gives its parameters."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts, their parameters, and how the block arranges them.

    ``prefix`` is the tensor-name prefix of the layer's weights (``"h.3."``).
    ``arrangement`` names a registered block arrangement (``"pre_norm"``).
    ``norms`` are the layer's norms by the names its arrangement asks for: ``pre_norm``
    wants ``"mixer"`` and ``"feed_forward"``; a block with sandwich norms would name four,
    a parallel block one.  ``width`` is the width of the residual stream.
    """

    prefix: str
    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    width: int


@dataclass(frozen=True)
class RunEntry:
    """One position in the execution order.

    ``layer``       index into ``layer_specs()`` (weights).
    ``cache_layer`` index of the layer whose cache this entry attends over.
    ``writes_cache`` False when the entry only reads a cache another entry filled.
    """

    layer: int
    cache_layer: int
    writes_cache: bool = True


class ModelConfig:
    """Base of all typed configurations."""

    #: HF identifiers this configuration answers to (``architectures[]`` entries and
    #: ``model_type``), used by the registry.
    identifiers: tuple = ()

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    # --- structure as data -------------------------------------------------
    def layer_specs(self) -> List[LayerSpec]:
        raise NotImplementedError

    def run_order(self) -> List[RunEntry]:
        return [RunEntry(i, i, True) for i in range(len(self.layer_specs()))]

    def embedding_spec(self) -> PartSpec:
        raise NotImplementedError

    def position_spec(self) -> PartSpec:
        return PartSpec("none")

    def final_norm_spec(self) -> PartSpec:
        raise NotImplementedError

    def head_spec(self) -> PartSpec:
        raise NotImplementedError

    @property
    def max_positions(self) -> int:
        raise NotImplementedError

    # --- helpers -------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str) -> "ModelConfig":
        with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2, sort_keys=True)
            fh.write("\n")


def _require_int(raw: Dict[str, Any], key: str, default: Optional[int] = None,
                 minimum: int = 1) -> int:
    value = raw.get(key, default)
    if value is None:
        raise ConfigError(f"config.json: missing required key '{key}'")
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {value}")
    return value


def _require_float(raw: Dict[str, Any], key: str, default: float) -> float:
    value = raw.get(key, default)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
    return float(value)


def _require_bool(raw: Dict[str, Any], key: str, default: bool) -> bool:
    value = raw.get(key, default)
    if not isinstance(value, bool):
        raise ConfigError(f"config.json: '{key}' must be true or false, got {value!r}")
    return value


def replace(config, **changes):
    """``dataclasses.replace`` that re-validates."""
    return type(config).from_dict({**config.to_dict(), **changes})


__all__ = ["ConfigError", "PartSpec", "LayerSpec", "RunEntry", "ModelConfig",
           "replace", "dataclasses"]
