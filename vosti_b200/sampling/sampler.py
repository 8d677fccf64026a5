"""Sampling from a step's logits on the device.

Greedy (temperature 0) is what the reference samples with: the argmax of the row, lowest
index on ties (python/vosti_kernels/kernels.py:1088-1104); its sampler is modelled as
(state, logits) -> (state', token) with an empty state (src/boundary/sampler.rs:7-19).
Temperature sampling keeps that shape with the state (seed, index of the token being
drawn): the uniform number comes from a counter-based generator keyed by that pair, so a
request's tokens do not depend on which other requests share its steps.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0


def uniform(seed: int, index: int) -> float:
    """The generator's value in [0, 1) with 24 bits, as the kernel computes it."""
    z = ((seed & _MASK) * 0x9E3779B97F4A7C15 + (index + 1) * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits; rows with temperature <= 0 are greedy."""
    return ops.sample(logits, temperature, seeds, counters, out=out)


def sampler_state_words(temperature: float, seed: int, index: int, position: int = 0):
    """The four 64-bit words of a request's sampler state as its slot keeps them: temperature
    as float32 bits, seed, index of the next token to draw, position (written by the kernel)."""
    bits = int(np.float32(temperature).view(np.uint32))
    signed = lambda v: int(np.uint64(v & _MASK).view(np.int64))
    return [bits, signed(seed), signed(index), int(position)]


def sample_from_slots(logits: torch.Tensor, slots: torch.Tensor, table: torch.Tensor,
                      positions: Optional[torch.Tensor], status: Optional[torch.Tensor],
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row; each row's (temperature, seed, index) is read from its request's slot
    of `table`, and the index is advanced there."""
    return ops.sample_slots(logits, slots, table, positions, status, out=out)


def sampling_arrays(temperatures: Sequence[float], seeds: Sequence[int], counters: Sequence[int]):
    """Host arrays in the layout the kernel reads; None if every row is greedy."""
    if not any(t > 0.0 for t in temperatures):
        return None
    as_signed = lambda v: np.asarray([x & _MASK for x in v], dtype=np.uint64).view(np.int64)
    return (np.asarray(temperatures, dtype=np.float32), as_signed(seeds), as_signed(counters))
