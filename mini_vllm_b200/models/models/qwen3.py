from ..decoder import DecoderLM


class Qwen3ForCausalLM(DecoderLM):
    """Counterpart of minivllm/models/models/qwen3.py:Qwen3ForCausalLM."""
    family = "qwen3"
