"""Model construction: weights from a safetensors directory, or seeded random weights when the
config carries no path (minivllm/models/loader.py:9-29 covers the first case only)."""
from __future__ import annotations

import os
from glob import glob

import torch

from .models import get_model_class


def _weights(path: str):
    import safetensors
    for file in sorted(glob(os.path.join(path, "*.safetensors"))):
        with safetensors.safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                yield name, f.get_tensor(name)


def load_model(config, device="cuda") -> torch.nn.Module:
    arch = config.hf_config.architectures[0]
    cls = get_model_class(arch)
    if cls is None:
        raise ValueError(f"Model architecture {arch} is not supported.")
    dtype = getattr(config.hf_config, "dtype", torch.bfloat16)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            model = cls(config.hf_config)
    finally:
        torch.set_default_dtype(prev)
    model.to(device)          # moves the CPU-built fp32 cos/sin tables; parameters are already there
    fuse = bool(getattr(config, "fuse_qk_norm", True))
    for module in model.modules():
        if hasattr(module, "fuse_qk_norm"):
            module.fuse_qk_norm = fuse
    if config.model is not None:
        model.load_weights(_weights(os.path.expanduser(config.model)))
    else:
        model.init_random(config.seed)
    return model.eval()
