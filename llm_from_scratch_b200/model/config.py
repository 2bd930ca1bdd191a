"""Architecture fields of the reference's ``Config`` (model/config.py:97-252) that the decoder reads."""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional


@dataclass
class ModelConfig:
    vocab_size: int = 32000
    context_length: int = 2048
    d_model: int = 768
    num_layers: int = 12
    num_heads: int = 16
    d_ff: int = 3072
    attention_type: str = "GQA"          # "GQA" (MHA is GQA with num_kv_heads == num_heads) or "MLA"
    num_kv_heads: Optional[int] = None
    rope_theta: float = 10000.0
    rope_dim: Optional[int] = 16         # MLA
    q_lora_rank: Optional[int] = 128     # MLA
    kv_lora_rank: Optional[int] = 256    # MLA
    use_moe: bool = False
    moe_layers: Optional[list] = None
    n_routed_experts: int = 8
    num_experts_per_tok: int = 1
    n_shared_experts: int = 1
    rms_eps: float = 1e-5                # RMSNorm of the residual stream (model/utils.py:49)

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_heads
        if self.attention_type == "MHA":
            self.attention_type, self.num_kv_heads = "GQA", self.num_heads
        if self.attention_type not in ("GQA", "MLA"):
            raise ValueError(f"unsupported attention_type {self.attention_type!r}")
        if self.d_model % self.num_heads or self.num_heads % self.num_kv_heads:
            raise ValueError("d_model must divide by num_heads and num_heads by num_kv_heads")

    @property
    def head_dim(self) -> int:
        return self.d_model // self.num_heads

    def is_moe_layer(self, i: int) -> bool:
        return bool(self.use_moe and (self.moe_layers is None or i in self.moe_layers))

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        names = cls.__dataclass_fields__.keys()
        return cls(**{k: v for k, v in d.items() if k in names})
