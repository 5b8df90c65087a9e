"""cuteafd_b200: a Blackwell-datacenter-native attention/FFN-disaggregated MoE inference engine."""
from .config import ModelConfig, PRESETS, tiny_moe, qwen3_30b_a3b, deepseek_v3, deepseek_v32, kimi_k2, mixtral_8x7b, scaled_down

__version__ = "0.1.0"
__all__ = ["ModelConfig", "PRESETS", "tiny_moe", "qwen3_30b_a3b", "deepseek_v3", "deepseek_v32", "kimi_k2", "mixtral_8x7b", "scaled_down"]
