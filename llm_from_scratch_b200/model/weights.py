"""Random initialisation that reproduces the reference's parameters for a given seed.

"Random init (seed 0)" in the benchmark configurations means ``torch.manual_seed(0)`` followed by
constructing the reference's ``TransformerLM`` on the CPU (model/transformer.py:124-160).  The
parameters are drawn here with the same initialisers, shapes and ORDER, so the same seed yields
bit-identical weights without the reference's code:

  token_embeddings  trunc_normal_(std=1, a=-3, b=3)                    model/utils.py:28-33
  per layer: attention projections (nn.Linear default init, weight then bias), then the FFN
             (MLP w1, w3, w2 — or the routed experts in order, the gate's kaiming_uniform_, the shared
             expert), norms are ones and consume no randomness           GQA.py:34-40, MLA.py:54-81,
                                                                         mlp.py:56-58, moe.py:186-204
  lm_head           nn.Linear default init                               transformer.py:160

Names are the reference's state_dict names.  Always built on the CPU (the CUDA generator is a
different stream), then moved.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from .config import ModelConfig


def _linear(out: dict, name: str, fan_in: int, fan_out: int) -> None:
    lin = nn.Linear(fan_in, fan_out)          # kaiming_uniform_(a=sqrt(5)) weight, then uniform bias
    out[name + ".weight"] = lin.weight.detach()
    out[name + ".bias"] = lin.bias.detach()


def _mlp(out: dict, prefix: str, d_model: int, d_ff: int) -> None:
    _linear(out, prefix + ".w1", d_model, d_ff)
    _linear(out, prefix + ".w3", d_model, d_ff)
    _linear(out, prefix + ".w2", d_ff, d_model)


@torch.no_grad()
def init_reference_order(cfg: ModelConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    torch.manual_seed(seed)
    w: dict[str, torch.Tensor] = {}
    d, H, Hkv, hd = cfg.d_model, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    emb = torch.empty(cfg.vocab_size, d)
    nn.init.trunc_normal_(emb, mean=0.0, std=1.0, a=-3, b=3)
    w["token_embeddings.weight"] = emb
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        if cfg.attention_type == "GQA":
            _linear(w, p + ".att.q_proj", d, d)
            _linear(w, p + ".att.k_proj", d, Hkv * hd)
            _linear(w, p + ".att.v_proj", d, Hkv * hd)
            _linear(w, p + ".att.output_proj", d, d)
            w[p + ".att.q_norm.weight"] = torch.ones(d)
            w[p + ".att.k_norm.weight"] = torch.ones(Hkv * hd)
        else:
            r, rq, dr = cfg.kv_lora_rank, cfg.q_lora_rank, cfg.rope_dim
            _linear(w, p + ".att.q_down_proj", d, rq)
            _linear(w, p + ".att.q_up_proj_fused", rq, d + H * dr)
            _linear(w, p + ".att.kv_down_proj", d, r)
            _linear(w, p + ".att.kv_up_proj_fused", r, 2 * d)
            _linear(w, p + ".att.k_rope_proj", d, dr)
            w[p + ".att.q_norm.weight"] = torch.ones(rq)
            w[p + ".att.kv_norm.weight"] = torch.ones(r)
            _linear(w, p + ".att.output_proj", H * hd, d)
        if cfg.is_moe_layer(i):
            for e in range(cfg.n_routed_experts):
                _mlp(w, f"{p}.ffn.experts.{e}", d, cfg.d_ff)
            w[p + ".ffn.gate.expert_bias"] = torch.zeros(cfg.n_routed_experts)
            gate = torch.empty(cfg.n_routed_experts, d)
            nn.init.kaiming_uniform_(gate, a=math.sqrt(5))
            w[p + ".ffn.gate.weight"] = gate
            if cfg.n_shared_experts > 0:
                _mlp(w, p + ".ffn.shared_expert", d, cfg.d_ff)
        else:
            _mlp(w, p + ".ffn", d, cfg.d_ff)
        w[p + ".att_norm.weight"] = torch.ones(d)
        w[p + ".ffn_norm.weight"] = torch.ones(d)
    w["final_norm.weight"] = torch.ones(d)
    _linear(w, "lm_head", d, cfg.vocab_size)
    return w
