"""Token sampling (reference: utils/sampler.py:26-57).

The reference draws softmax(logits / T) divided by Exp(1) noise and takes the argmax: a sample of the
categorical distribution.  On the GPU that is one kernel (``ops.sample``: the same race in the log
domain, counter-based random numbers); the tensor-op form below is kept for CPU tensors and as the
definition.  The reference forbids T = 0; here a row with T = 0 is decoded greedily (argmax of the
raw logits, first maximum), which the benchmark configurations require.
"""
from __future__ import annotations

import torch
from torch import nn


class Sampler(nn.Module):
    def __init__(self, seed: int | None = None):
        super().__init__()
        self.seed = seed          # None: taken from torch.initial_seed() at the first draw
        self.calls = 0            # one random stream offset per call

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor | None) -> torch.Tensor:
        if logits.is_cuda and logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (torch.float32,
                                                                                               torch.bfloat16):
            from .. import ops
            if self.seed is None:
                self.seed = torch.initial_seed()
            self.calls += 1
            t = None if temperatures is None else temperatures.to(logits.device, torch.float32).contiguous()
            return ops.sample(logits, t, self.seed, self.calls)
        greedy = logits.argmax(dim=-1)
        if temperatures is None:
            return greedy
        t = temperatures.to(logits.device, torch.float32)
        safe = torch.where(t > 0, t, torch.ones_like(t))
        probs = torch.softmax(logits.float() / safe.unsqueeze(1), dim=-1)
        noise = torch.empty_like(probs).exponential_(1).clamp_min_(1e-10)
        sampled = (probs / noise).argmax(dim=-1)
        return torch.where(t > 0, sampled, greedy)
