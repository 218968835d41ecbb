from ..decoder import DecoderLM


class Gemma3ForCausalLM(DecoderLM):
    """Counterpart of minivllm/models/models/gemma3.py:Gemma3ForCausalLM."""
    family = "gemma3"
