"""Engine-mode decoder: the reference's layer arithmetic over flat ragged batches and paged caches."""
from .config import ModelConfig
from .weights import init_reference_order
from .transformer import EngineTransformerLM

__all__ = ["ModelConfig", "init_reference_order", "EngineTransformerLM"]
