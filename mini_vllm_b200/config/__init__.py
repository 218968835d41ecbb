from .config import Config, gemma3_shape, qwen3_shape
from .sampling import SamplingParams

__all__ = ["Config", "SamplingParams", "qwen3_shape", "gemma3_shape"]
