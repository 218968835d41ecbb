"""The reference's own engine loop, driven on a device with a stand-in for its attention package.  TEST INFRASTRUCTURE.

What runs here is the reference's code, imported unmodified from the staged copy (``oracle/stage_reference.py``):
``Scheduler`` / ``KVCacheBlockManager`` (scheduler/scheduler.py, kvcache/block_manager.py), ``Executor`` with its
``_build_prefill_input`` / ``_build_decode_input`` / ``execute`` / ``sample`` (executor/executor.py:81-225), the
model classes (models/models/qwen3.py, gemma3.py) with their RoPE, norms, Triton ``store_kvcache`` and argmax
sampler, stepped exactly as ``Engine.step`` does (engine/engine.py:31-36).  Three things are supplied from outside,
because the reference cannot provide them on this machine:

* ``mini_flash_attention`` (requirements.txt:7, not vendored): a module of that name whose two functions are the
  fp32 gather-and-SDPA of ``oracle/attention.py`` - the definition the CUDA kernels are held to;
* weights: the reference loads safetensors from a model directory (models/loader.py:16-28); here the model class is
  built from a shape description and filled from a state dict with the reference's parameter names;
* ``Engine`` itself needs a tokenizer directory (engine/engine.py:17), so its four-line step loop is restated in
  ``generate``.

``torch.compile`` is switched off (``TORCHDYNAMO_DISABLE=1``) so that the decorated reference functions run their
eager arithmetic, and CUDA graphs are off because the stand-in attention reads lengths on the host.
"""
from __future__ import annotations

import os
import sys
import types
from types import SimpleNamespace

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import torch  # noqa: E402

from . import attention as oattn  # noqa: E402
from .stage_reference import DEST, staged_package  # noqa: E402


def available() -> bool:
    return staged_package() is not None


def _install_stubs() -> None:
    if "mini_flash_attention" not in sys.modules:
        stub = types.ModuleType("mini_flash_attention")

        def flash_attn_varlen_func(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, causal=True):
            return oattn.prefill(q, k, v, cu_seqlens_q, cu_seqlens_k)           # attention.py:84-87

        def flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens, block_table):
            return oattn.decode(q[:, 0], k_cache, v_cache, cache_seqlens, block_table).unsqueeze(1)   # :90-91

        stub.flash_attn_varlen_func = flash_attn_varlen_func
        stub.flash_attn_with_kvcache = flash_attn_with_kvcache
        sys.modules["mini_flash_attention"] = stub
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))


class ReferenceEngine:
    """``generate(prompts, max_tokens)`` through the reference's scheduler, executor and model on ``device``."""

    def __init__(self, hf_config, weights: dict, device, kv_cache_num_blocks: int = 256, max_num_batched_seqs: int = 64,
                 max_num_batched_tokens: int = 16384, kv_cache_block_size: int = 256, attention_functions=None):
        """``attention_functions``: ``(flash_attn_varlen_func, flash_attn_with_kvcache)`` to put where the
        reference's attention layer looks its two functions up; default: the fp32 gather-and-SDPA stand-in."""
        if not available():
            raise RuntimeError("the reference package has not been staged (python -m oracle.stage_reference)")
        _install_stubs()
        self.attention_functions = attention_functions
        import minivllm.executor.executor as ref_executor
        from minivllm.models.models import get_model_class
        from minivllm.scheduler.scheduler import Scheduler

        self.device = torch.device(device)
        self.config = SimpleNamespace(
            model=None, hf_config=hf_config, max_model_len=4096, max_num_batched_tokens=max_num_batched_tokens,
            max_num_batched_seqs=max_num_batched_seqs, eos_token_ids=set(), kv_cache_num_blocks=kv_cache_num_blocks,
            kv_cache_block_size=kv_cache_block_size, gpu_memory_utilization=0.9, use_cuda_graph=False)

        def load_model(config):                                  # stands in for models/loader.py:23-28
            model = get_model_class(hf_config.architectures[0])(hf_config)
            own = dict(model.state_dict())
            missing = [k for k in own if k not in weights and not (k == "lm_head.weight" and hf_config.tie_word_embeddings)]
            if missing:
                raise KeyError(f"no weights for {missing[:4]}")
            with torch.no_grad():
                for name, p in own.items():
                    if name in weights:
                        p.copy_(weights[name])
                if hf_config.tie_word_embeddings:
                    model.lm_head.weight.data = model.model.embed_tokens.weight.data     # qwen3.py:203-204
            return model

        self._Scheduler = Scheduler
        default_device, default_dtype = torch.get_default_device(), torch.get_default_dtype()
        if self.device.type == "cuda":
            saved = ref_executor.load_model
            ref_executor.load_model = load_model
            try:
                with torch.cuda.device(self.device):
                    self.executor = ref_executor.Executor(self.config)  # sets the default device / dtype itself
            finally:
                ref_executor.load_model = saved
                torch.set_default_device(default_device)
                torch.set_default_dtype(default_dtype)
            return
        # Without a GPU (small models, host-side tests) the constructor's CUDA calls and the Triton store cannot
        # run: the executor object is assembled by hand with the same fields (executor.py:13-60) and the KV write is
        # the restated copy of attention.py:24-33.  Packing, scheduling, model and sampler are still the reference's.
        import minivllm.models.layers.attention as ref_attention
        from minivllm.models.layers.sampler import Sampler
        from . import rope_kv
        ref_attention.store_kvcache = rope_kv.store_kvcache
        torch.set_default_dtype(hf_config.dtype)
        try:
            ex = object.__new__(ref_executor.Executor)
            ex.config, ex.model, ex.sampler = self.config, load_model(self.config), Sampler()
            head_dim = hf_config.head_dim
            ex.kv_cache = torch.zeros(2, hf_config.num_hidden_layers, kv_cache_num_blocks, kv_cache_block_size,
                                      hf_config.num_key_value_heads, head_dim)
            layer = 0
            for module in ex.model.modules():                     # executor.py:55-60
                if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
                    module.k_cache, module.v_cache = ex.kv_cache[0, layer], ex.kv_cache[1, layer]
                    layer += 1
            self.executor = ex
        finally:
            torch.set_default_dtype(default_dtype)

    def generate(self, prompts: list[list[int]], max_tokens: int):
        """Greedy tokens per prompt plus, per generated token, the two largest logits of the row it was taken from."""
        from minivllm.config.sampling import SamplingParams
        from minivllm.engine.request import Request
        sch = self._Scheduler(self.config)
        reqs = [Request(list(p), SamplingParams(max_tokens=max_tokens, ignore_eos=True)) for p in prompts]
        row_of = {r.id: i for i, r in enumerate(reqs)}
        top2 = [[] for _ in reqs]
        ex = self.executor
        plain_sample = ex.sample

        def recording_sample(logits, batch):
            best = torch.topk(logits.float(), 2, dim=-1).values.cpu()
            for r, pair in zip(batch.requests, best.tolist()):
                top2[row_of[r.id]].append(pair)
            return plain_sample(logits, batch)

        ex.sample = recording_sample
        import minivllm.models.layers.attention as ref_attention
        bound = (ref_attention.flash_attn_varlen_func, ref_attention.flash_attn_with_kvcache)
        if self.attention_functions is not None:      # the names the layer resolves at call time (attention.py:84-91)
            ref_attention.flash_attn_varlen_func, ref_attention.flash_attn_with_kvcache = self.attention_functions
        default_device, default_dtype = torch.get_default_device(), torch.get_default_dtype()
        torch.set_default_device(self.device)
        torch.set_default_dtype(self.config.hf_config.dtype)
        on_cpu = self.device.type == "cpu"
        plain_tensor, plain_cuda = torch.tensor, torch.Tensor.cuda
        if on_cpu:                                                # the packing code pins and uploads (executor.py:116-122)
            torch.tensor = lambda *a, **kw: plain_tensor(*a, **{k: v for k, v in kw.items() if k != "pin_memory"})
            torch.Tensor.cuda = lambda t, *a, **kw: t
        try:
            for r in reqs:
                sch.submit(r)
            guard = torch.cuda.device(self.device) if not on_cpu else _NullContext()
            with guard:
                while not sch.finished:                           # engine.py:31-36
                    batch = sch.schedule()
                    tokens = ex.execute(batch)
                    sch.update(batch, tokens)
        finally:
            ex.sample = plain_sample
            ref_attention.flash_attn_varlen_func, ref_attention.flash_attn_with_kvcache = bound
            torch.tensor, torch.Tensor.cuda = plain_tensor, plain_cuda
            torch.set_default_device(default_device)
            torch.set_default_dtype(default_dtype)
        return [r.completion_tokens for r in reqs], top2


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
