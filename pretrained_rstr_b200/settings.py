"""Measurement switches, all in one place.

None of them is needed to use the engine; they exist so that a measurement can turn one
mechanism off and see what it is worth.  Each is an environment variable read once, when
this module is first imported.

Python side (``SETTINGS``):

``PRB200_GRAPHS=0``        small steps are launched kernel by kernel instead of as CUDA graphs
``PRB200_PDL=0``           no programmatic dependent launch between the kernels of a step
``PRB200_ATTN_TC=0``       prompt attention on ``mma.sync`` even where the tcgen05 kernel applies
``PRB200_PREFILL_PART=N``  key blocks per part of the tcgen05 prompt attention (-1: the kernel's rule)
``PRB200_DECODE_CTAS=N``   CTAs a decode attention launch aims for (0: about five per SM)
``PRB200_DECODE_RING=0|1`` decode attention always by the split-key kernel (0) or, where its sizes
                           allow, always by the ring kernel (1); unset: whichever measured faster

Read by the CUDA library itself (``csrc/``): ``PRB200_DECODE_EARLY=1`` and
``PRB200_EARLY_SMALL=1`` let kernels of many small CTAs be placed on the SMs before their
predecessor has ended.  Read by the build (``csrc/build.py``): ``PRB200_NVCC_FLAGS`` (extra
compiler flags, e.g. ``-DPRB_TRACE`` for device-side timestamps) and ``PRB200_BUILD_DIR``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional


def _flag(name: str, default: bool) -> bool:
    value = os.environ.get(name)
    if value is None:
        return default
    return value.strip().lower() not in ("0", "false", "no", "off", "")


def _int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


@dataclass
class Settings:
    graphs: bool = True
    pdl: bool = True
    attention_tcgen05: bool = True
    prefill_part: int = -1
    decode_ctas: int = 0
    decode_ring: Optional[bool] = None
    step_words_by_kernel: bool = True

    @classmethod
    def from_environment(cls) -> "Settings":
        return cls(graphs=_flag("PRB200_GRAPHS", True), pdl=_flag("PRB200_PDL", True),
                   attention_tcgen05=_flag("PRB200_ATTN_TC", True),
                   prefill_part=_int("PRB200_PREFILL_PART", -1),
                   decode_ctas=_int("PRB200_DECODE_CTAS", 0),
                   decode_ring=(_flag("PRB200_DECODE_RING", True)
                                if "PRB200_DECODE_RING" in os.environ else None),
                   step_words_by_kernel=_flag("PRB200_STEP_WORDS_BY_KERNEL", True))


SETTINGS = Settings.from_environment()
