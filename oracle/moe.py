"""CPU restatement of the per-expert loop of the reference's MoE inference path (test oracle only:
imported by tests/ and nothing else).

Follows MOE.moe_infer (model/architecture/moe.py:299-339): rows grouped by expert, expert e applied to
its contiguous row range; an expert is an MLP (model/architecture/mlp.py:61-67), w2(silu(w1 x) * w3 x),
each Linear rounding its output to the activation dtype.  Matrix products are taken in fp32 on the CPU
and rounded to bf16 where the bf16 tensor-op sequence would round.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def grouped_linear(x: torch.Tensor, w: torch.Tensor, offsets, bias: torch.Tensor | None, swiglu: bool) -> torch.Tensor:
    """x [rows, k] bf16 grouped by expert; expert e owns rows [offsets[e-1], offsets[e]).

    swiglu=False: out = x W_e^T (+ bias_e), w [E, n, k].
    swiglu=True:  w [E, 2n, k] = rows of w1 then of w3 (bias likewise): out = silu(h1) * h3 with
                  h = x W_e^T (+ bias_e); GEMM result, bias add, silu and product each rounded to bf16.
    """
    x, w = x.detach().cpu(), w.detach().cpu()
    bias = None if bias is None else bias.detach().cpu()
    E = w.shape[0]
    n_out = w.shape[1] // 2 if swiglu else w.shape[1]
    out = torch.zeros(x.shape[0], n_out, dtype=torch.bfloat16)
    lo = 0
    for e in range(E):
        hi = int(offsets[e])
        if hi > lo:
            h = (x[lo:hi].float() @ w[e].float().t()).to(torch.bfloat16)
            if bias is not None:
                h = h + bias[e]
            out[lo:hi] = F.silu(h[:, :n_out]) * h[:, n_out:] if swiglu else h
        lo = hi
    return out
