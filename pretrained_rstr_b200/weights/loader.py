"""Weights by tensor name: checking, loading, and a random-weights mode.

The reference looks tensors up by their Hugging Face names and has no shape check
(a missing tensor becomes a later null dereference in ``dev/examples/gpt2.clj:180``;
its lazy reader throws "Tensor not found" one name at a time,
``src/pretrained/safetensors.clj:141-143``).  Here the whole file is checked against
what the architecture expects *before* anything is copied, and every problem is
reported in one error: missing tensors, unexpected tensors, wrong shapes.

Storage precision: a tensor stored in 16-bit floating point is kept in bfloat16, a
tensor stored in 32-bit floating point stays 32-bit, integer tables become int32.
Parts decide at build time which precision their kernels read.
"""
from __future__ import annotations

import os
import re
import zlib
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile, save_file


class WeightError(ValueError):
    """The tensors of a model folder do not match what its configuration needs."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{where}: tensors do not match the configuration"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorExpectation:
    shape: Tuple[int, ...]
    kind: str = "float"          # "float" or "int"


def _stored_dtype(dtype: torch.dtype, kind: str) -> torch.dtype:
    """Element type a tensor is kept in until a part binds it: integer tables int32, 32-bit
    (and wider) floats float32, bfloat16 bfloat16, and float16 as it is: the part converts it
    to the runtime's type in one step, so a float32 runtime loses none of its bits."""
    if kind == "int":
        return torch.int32
    if dtype in (torch.float32, torch.float64):
        return torch.float32
    if dtype == torch.float16:
        return torch.float16
    return torch.bfloat16


class WeightStore:
    """Tensors by name on one device.  ``get`` returns the tensor as stored;
    ``get(name, dtype)`` a cached copy in ``dtype``."""

    def __init__(self, tensors: Dict[str, torch.Tensor], device: torch.device):
        self.device = device
        self._tensors = tensors
        self._casts: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def names(self) -> List[str]:
        return sorted(self._tensors)

    def __contains__(self, name: str) -> bool:
        return name in self._tensors

    def get(self, name: str, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if name not in self._tensors:
            raise KeyError(f"weight store has no tensor {name!r}")
        t = self._tensors[name]
        if dtype is None or t.dtype == dtype:
            return t
        key = (name, dtype)
        if key not in self._casts:
            self._casts[key] = t.to(dtype)
        return self._casts[key]

    def release(self) -> None:
        """Drop the store's own references; parts keep what they bound."""
        self._tensors = {}
        self._casts = {}


def _canonical(name: str, strip_prefixes: Iterable[str]) -> str:
    for p in strip_prefixes:
        if name.startswith(p):
            return name[len(p):]
    return name


def load_weights(folder: str, expected: Dict[str, TensorExpectation], device,
                 strip_prefixes: Iterable[str] = (),
                 ignorable: Callable[[str], bool] = lambda name: False,
                 filename: str = "model.safetensors") -> WeightStore:
    """Check ``folder/model.safetensors`` against ``expected`` and copy it to ``device``.

    ``strip_prefixes``: leading name parts that may be present and are removed (the
    reference strips ``model.`` the same way, ``src/pretrained/decoder.clj:40-45``).
    ``ignorable(name)``: tensors that may be present without being parameters.
    """
    path = os.path.join(folder, filename)
    if not os.path.isfile(path):
        raise WeightError(path, sorted(expected), [], ["file does not exist"])
    f = SafetensorsFile(path)
    found: Dict[str, str] = {}
    unexpected: List[str] = []
    for stored_name in f.names():
        name = _canonical(stored_name, strip_prefixes)
        if name in expected:
            found[name] = stored_name
        elif not ignorable(name):
            unexpected.append(stored_name)
    missing = sorted(n for n in expected if n not in found)
    wrong: List[str] = []
    for name, stored_name in sorted(found.items()):
        exp = expected[name]
        shape = f.shape(stored_name)
        dtype = f.dtype(stored_name)
        if tuple(shape) != tuple(exp.shape):
            wrong.append(f"{stored_name}: expected {list(exp.shape)}, found {list(shape)}")
        elif exp.kind == "float" and not dtype.is_floating_point:
            wrong.append(f"{stored_name}: expected a floating-point tensor, found {dtype}")
        elif exp.kind == "int" and (dtype.is_floating_point or dtype == torch.bool):
            wrong.append(f"{stored_name}: expected an integer tensor, found {dtype}")
    if missing or unexpected or wrong:
        raise WeightError(path, missing, sorted(unexpected), wrong)
    device = torch.device(device)
    tensors: Dict[str, torch.Tensor] = {}
    for name, stored_name in found.items():
        t = f.tensor(stored_name)
        target = _stored_dtype(t.dtype, expected[name].kind)
        tensors[name] = t.to(device=device, dtype=target, copy=True)
    f.close()
    return WeightStore(tensors, device)


# --------------------------------------------------------------------------- random
def tensor_generator(seed: int, name: str) -> torch.Generator:
    """A CPU generator that depends only on (seed, tensor name), so a tensor's values
    do not depend on which other tensors are made or in which order (the reference's
    tests seed per name too: ``test/pretrained/decoder_gpu_oracle_test.clj:149-171``)."""
    g = torch.Generator(device="cpu")
    g.manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63))
    return g


def normal(seed: int, name: str, shape, std: float, mean: float = 0.0) -> torch.Tensor:
    g = tensor_generator(seed, name)
    return torch.randn(tuple(shape), generator=g, dtype=torch.float32) * std + mean


def write_model_folder(folder: str, config, tensors: Dict[str, torch.Tensor],
                       dtype: torch.dtype = torch.float32) -> None:
    """Write ``config.json`` and ``model.safetensors``; floating tensors are stored in
    ``dtype`` (float32 or bfloat16)."""
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    out = {}
    for name, t in tensors.items():
        out[name] = t.to(dtype) if t.dtype.is_floating_point else t
    save_file(out, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt"})


def make_random_model(folder: str, config, seed: int,
                      dtype: torch.dtype = torch.float32) -> None:
    """Random-weights mode: a complete model folder from a configuration and a seed."""
    from ..config.registry import lookup
    arch = lookup(config.to_dict())
    write_model_folder(folder, config, arch.random_tensors(config, seed), dtype)


_LAYER_RE = re.compile(r"\.(\d+)\.")


def layer_of(name: str) -> Optional[int]:
    m = _LAYER_RE.search(name)
    return int(m.group(1)) if m else None
