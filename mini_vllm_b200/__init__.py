"""B200 (sm_100a) kernels and host-side mirror for mini-vllm's ragged attention path.

``LLM`` is the engine under the name offline-inference scripts usually give it: ``LLM(config).generate(prompts,
SamplingParams(...))`` is ``Engine.generate`` of ``minivllm/engine/engine.py:40-90``.  ``ReplicatedEngine`` puts the
same call in front of one engine process per GPU.
"""

__version__ = "0.2.0"

_LAZY = {
    "LLM": ("mini_vllm_b200.engine.engine", "Engine"),
    "Engine": ("mini_vllm_b200.engine.engine", "Engine"),
    "ReplicatedEngine": ("mini_vllm_b200.dispatcher", "ReplicatedEngine"),
    "Config": ("mini_vllm_b200.config", "Config"),
    "SamplingParams": ("mini_vllm_b200.config", "SamplingParams"),
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib
        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(f"module 'mini_vllm_b200' has no attribute {name!r}")
