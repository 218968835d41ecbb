"""Stand-ins that answer the reference's literal imports with the CUDA kernels of this package."""
from __future__ import annotations

import sys


def install() -> None:
    """Register ``mini_flash_attention`` in ``sys.modules`` so that the reference's
    ``from mini_flash_attention import flash_attn_with_kvcache, flash_attn_varlen_func``
    (``minivllm/models/layers/attention.py:7``) binds to this package's kernels."""
    from . import mini_flash_attention
    sys.modules["mini_flash_attention"] = mini_flash_attention
