"""Registries of parts.  A part is chosen by the ``kind`` of a
:class:`~pretrained_rstr_b200.config.base.PartSpec` and built from that spec's
parameters; nothing in a part says which model it is in.

Categories and what a factory returns (interfaces in :mod:`.interfaces`):

``mixer``         :class:`Mixer`        factory(params, store, runtime)
``feed_forward``  :class:`FeedForward`  factory(params, store, runtime)
``norm``          :class:`Norm`         factory(params, store, runtime)
``position``      :class:`PositionEncoding`  factory(params, store, runtime)
``embedding``     :class:`Embedding`    factory(params, store, runtime)
``head``          :class:`Head`         factory(params, store, runtime)
``arrangement``   :class:`Block`        factory(mixer, feed_forward, norms by name, width, runtime);
                                        the block keeps ``mixer``, ``feed_forward`` and ``norms``
"""
from __future__ import annotations

from typing import Any, Callable, Dict

_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "embedding", "head", "arrangement")
_PARTS: Dict[str, Dict[str, Callable[..., Any]]] = {c: {} for c in _CATEGORIES}


def register_part(category: str, kind: str, factory: Callable[..., Any]) -> None:
    if category not in _PARTS:
        raise KeyError(f"unknown part category {category!r}; known: {list(_CATEGORIES)}")
    _PARTS[category][kind] = factory


def part_factory(category: str, kind: str) -> Callable[..., Any]:
    try:
        return _PARTS[category][kind]
    except KeyError:
        raise KeyError(f"no {category} part registered as {kind!r}; "
                       f"known: {sorted(_PARTS.get(category, {}))}") from None


def build_part(category: str, spec, store, runtime):
    return part_factory(category, spec.kind)(spec.params, store, runtime)


def registered_parts(category: str):
    return sorted(_PARTS[category])
