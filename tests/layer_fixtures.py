"""Rebuilds the weights and inputs of the layer-level bf16 fixtures (tests/golden/make_golden_layers.py).

The fixtures hold seeds, checksums and the reference's outputs; weights and inputs are drawn again
here and verified against the checksums, so a test that runs has the reference's exact operands."""
import os

import numpy as np
import torch

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

MOE_LAYER = dict(vocab_size=64, context_length=2048, d_model=1024, num_layers=1, num_heads=16, num_kv_heads=4,
                 d_ff=704, attention_type="GQA", use_moe=True, n_routed_experts=16, num_experts_per_tok=2,
                 n_shared_experts=1, rope_theta=10000.0)
MLA_LAYER = dict(vocab_size=64, context_length=512, d_model=2048, num_layers=1, num_heads=16, d_ff=64,
                 attention_type="MLA", kv_lora_rank=512, q_lora_rank=1024, rope_dim=64, use_moe=False,
                 rope_theta=10000.0)


def load(name):
    return np.load(os.path.join(G, name))


def from_bf16_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def seeded_input(seed: int, rows: int, dim: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, dim, generator=g).to(torch.bfloat16)


def layer_weights(cfg: dict, z, prefix: str) -> dict:
    """The reference's random initialisation for the fixture's seed, checked against its checksums."""
    from llm_from_scratch_b200.model import ModelConfig, init_reference_order
    w = init_reference_order(ModelConfig.from_dict(cfg), int(z["seed"]))
    if cfg.get("use_moe"):
        E = cfg["n_routed_experts"]
        w["layers.0.ffn.gate.expert_bias"] = ((torch.arange(E) % 5).float() - 2.0) * 0.03
    checked = 0
    for k in z.files:
        if k.startswith("sum::") and k[5:] in w:     # buffers of the module (expert_load) are not weights
            assert w[k[5:]].double().sum().item() == float(z[k]), f"weight {k[5:]} differs from the reference's draw"
            checked += 1
    assert checked > 0 and any(k.startswith("sum::" + prefix) for k in z.files)
    return w


def checked_input(z, seed_key: str, sum_key: str, rows: int, dim: int) -> torch.Tensor:
    x = seeded_input(int(z[seed_key]), rows, dim)
    assert x.double().sum().item() == float(z[sum_key]), "seeded input differs from the fixture's"
    return x


def rel_errors(got: torch.Tensor, want: torch.Tensor):
    """(max-abs, mean-relative) error of ``got`` against ``want`` in fp32."""
    g, w = got.float(), want.float()
    return (g - w).abs().max().item(), ((g - w).abs().mean() / w.abs().mean()).item()
