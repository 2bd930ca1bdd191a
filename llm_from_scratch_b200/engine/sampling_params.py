"""Per-request sampling parameters.

The reference's engine imports a ``SamplingParams`` module that it does not ship; the one it does
ship (utils/sampler.py:7-23) has ``temperature``, ``max_tokens`` and ``ignore_eos`` and forbids
greedy decoding, while engine/sequence.py:31-34 also reads ``max_model_length``.  This class has
all four fields; ``temperature == 0`` selects greedy decoding (argmax, first maximum), which the
benchmark configurations require.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 256
    ignore_eos: bool = False
    max_model_length: Optional[int] = None

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0 (0 = greedy)")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
