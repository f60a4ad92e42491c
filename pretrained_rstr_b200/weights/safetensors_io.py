"""safetensors reading and writing.

File layout (``src/pretrained/safetensors.clj:24-37, 88-107``): an unsigned 64-bit
little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``
(the ``__metadata__`` entry is skipped), and the raw little-endian tensor bytes.
The file is memory-mapped (privately, so views are writable without touching the
file); each tensor is a view into the map until it is copied.
Unlike the reference, which widens every dtype to 32-bit floats
(``safetensors.clj:47-78``), tensors keep the dtype they are stored in.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A memory-mapped safetensors file; ``tensor(name)`` returns a CPU view."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._fh = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds file size {size}")
        try:
            header = json.loads(self._fh.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON ({exc})") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, dict] = header
        self._data_start = 8 + header_len
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        for name, entry in self.entries.items():
            if entry.get("dtype") not in _DTYPES:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has unsupported dtype {entry.get('dtype')!r}")
            begin, end = entry["data_offsets"]
            if not (0 <= begin <= end <= size - self._data_start):
                raise SafetensorsError(f"{path}: tensor {name!r} lies outside the file")

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.entries:
            raise SafetensorsError(
                f"{self.path}: tensor not found: {name!r}; available: {sorted(self.entries)[:8]}...")
        entry = self.entries[name]
        dtype = _DTYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        shape = tuple(entry["shape"])
        count = 1
        for s in shape:
            count *= s
        itemsize = torch.empty((), dtype=dtype).element_size()
        if count * itemsize != end - begin:
            raise SafetensorsError(
                f"{self.path}: tensor {name!r}: shape {shape} needs {count * itemsize} bytes, "
                f"file holds {end - begin}")
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=count,
                                offset=self._data_start + begin)
        return flat.view(shape)

    def close(self) -> None:
        # Views handed out by tensor() keep the map alive; only drop our handle.
        try:
            self._fh.close()
        except Exception:
            pass


def load_file(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of ``path`` as independent CPU copies."""
    f = SafetensorsFile(path)
    out = {name: f.tensor(name).clone() for name in f.names()}
    f.close()
    return out


def save_file(tensors: Dict[str, torch.Tensor], path: str,
              metadata: Dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file; names are
    written in sorted order and each tensor starts on an 8-byte boundary like the
    header itself."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order: Iterable[str] = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * ((8 - len(head) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(head)))
        fh.write(head)
        for raw in blobs:
            fh.write(raw)
    os.replace(tmp, path)
