"""B200 (sm_100a) kernels and host-side mirror for mini-vllm's ragged attention path."""

__version__ = "0.1.0"
