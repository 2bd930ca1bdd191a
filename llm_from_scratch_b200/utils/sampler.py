"""Token sampling (reference: utils/sampler.py:26-57).

Temperature sampling is the reference's exponential-race form: softmax(logits / T) divided by
Exp(1) noise, then argmax.  The reference forbids T = 0; here a row with T = 0 is decoded greedily
(argmax of the raw logits, first maximum), which the benchmark configurations require.
"""
from __future__ import annotations

import torch
from torch import nn


class Sampler(nn.Module):
    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor | None) -> torch.Tensor:
        greedy = logits.argmax(dim=-1)
        if temperatures is None:
            return greedy
        t = temperatures.to(logits.device, torch.float32)
        safe = torch.where(t > 0, t, torch.ones_like(t))
        probs = torch.softmax(logits.float() / safe.unsqueeze(1), dim=-1)
        noise = torch.empty_like(probs).exponential_(1).clamp_min_(1e-10)
        sampled = (probs / noise).argmax(dim=-1)
        return torch.where(t > 0, sampled, greedy)
