"""Choosing the next token: the options of the reference's sampler and the host side of the
device kernel that applies them (``csrc/sampling.cu``)."""
from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]
