"""The reference's literal import seam: ``from mini_flash_attention import flash_attn_with_kvcache,
flash_attn_varlen_func`` (``minivllm/models/layers/attention.py:7``) answered by this package's kernels."""
import sys

import numpy as np
import pytest
import torch

from mini_vllm_b200 import compat, ops
from mini_vllm_b200.workloads import config1, generator, randn_bf16, table_tensor
from oracle import attention as oattn
from oracle import rope_kv
from tests.helpers import assert_close_attn


def test_llm_alias_and_module_registration():
    import mini_vllm_b200
    from mini_vllm_b200.engine.engine import Engine
    assert mini_vllm_b200.LLM is Engine
    saved = sys.modules.pop("mini_flash_attention", None)
    try:
        compat.install()
        from mini_flash_attention import flash_attn_varlen_func, flash_attn_with_kvcache   # the reference's import line
        assert callable(flash_attn_varlen_func) and callable(flash_attn_with_kvcache)
    finally:
        sys.modules.pop("mini_flash_attention", None)
        if saved is not None:
            sys.modules["mini_flash_attention"] = saved


@pytest.mark.gpu
def test_called_the_way_the_reference_calls_them(cuda):
    """Config 1 through the two functions with the reference's own keyword arguments (attention.py:84-91)."""
    from mini_vllm_b200.compat.mini_flash_attention import flash_attn_varlen_func, flash_attn_with_kvcache
    case, g = config1()
    lens = case.prefill_lens
    T = sum(lens)
    qkv = randn_bf16(g, T, (16 + 2 * 8) * 128)                     # q/k/v are views of one projection output
    q, k, v = (t.view(T, -1, 128) for t in qkv.split([16 * 128, 8 * 128, 8 * 128], dim=-1))
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    want = oattn.prefill(q, k, v, cu, cu, out_dtype=torch.float32)
    qd, kd, vd = (t.view(T, -1, 128) for t in qkv.to(cuda).split([16 * 128, 8 * 128, 8 * 128], dim=-1))
    o = flash_attn_varlen_func(qd, kd, vd, max_seqlen_q=max(lens), cu_seqlens_q=cu.to(cuda), max_seqlen_k=max(lens),
                               cu_seqlens_k=cu.to(cuda), causal=True)
    assert o.shape == (T, 16, 128)
    assert_close_attn(o, want, "flash_attn_varlen_func seam")

    k_cache = torch.zeros(64, 256, 8, 128, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    slot_map = torch.cat([torch.cat([torch.arange(256) + b * 256 for b in blocks])[:n]
                          for n, blocks in zip(lens, case.prefill_blocks)]).to(torch.int32)
    rope_kv.store_kvcache(k, v, k_cache, v_cache, slot_map)
    qdec = randn_bf16(g, len(lens), 16, 128)
    seqlens = torch.tensor(lens, dtype=torch.int32)
    bt = table_tensor(case.prefill_blocks)
    want = oattn.decode(qdec, k_cache, v_cache, seqlens, bt, out_dtype=torch.float32)
    o = flash_attn_with_kvcache(qdec.to(cuda).unsqueeze(1), k_cache.to(cuda), v_cache.to(cuda),
                                cache_seqlens=seqlens.to(cuda), block_table=bt.to(cuda))
    assert o.shape == (len(lens), 1, 16, 128)
    assert_close_attn(o[:, 0], want, "flash_attn_with_kvcache seam")

    # the prefix-cached call of the reference hands over the pool without a table: refused with the reason
    with pytest.raises(ValueError, match="no block_table"):
        flash_attn_varlen_func(qd, k_cache.to(cuda), v_cache.to(cuda), max_seqlen_q=max(lens), cu_seqlens_q=cu.to(cuda),
                               max_seqlen_k=max(lens), cu_seqlens_k=cu.to(cuda), causal=True)


@pytest.mark.gpu
def test_unmodified_reference_engine_runs_on_the_kernels_through_its_import_seam(cuda):
    """The reference's own scheduler, executor, model and attention LAYER (staged copy, unmodified), with the two
    names its layer imports bound to this package: its greedy tokens on the screened config-2 prompts equal the
    ones it produces with the fp32 stand-in (the committed fixture)."""
    from pathlib import Path
    from mini_vllm_b200.compat import mini_flash_attention as seam
    from mini_vllm_b200.config import Config, qwen3_shape
    from mini_vllm_b200.models.loader import load_model
    from oracle import reference_engine
    from oracle.model import reference_names
    if not reference_engine.available():
        pytest.skip("the reference package is not staged on this machine")
    z = np.load(Path(__file__).parent / "golden" / "config2_tokens.npz")
    cuts = np.concatenate([[0], np.cumsum(z["prompt_lens"])])
    prompts = [z["prompts_flat"][a:b].tolist() for a, b in zip(cuts[:-1], cuts[1:])][:6]
    hf = qwen3_shape()
    model = load_model(Config(hf_config=hf, seed=0), device=cuda)
    weights = reference_names({k: v.detach() for k, v in model.state_dict().items()}, "qwen3", hf)
    del model
    ref = reference_engine.ReferenceEngine(hf, weights, cuda, kv_cache_num_blocks=32, max_num_batched_seqs=8,
                                           attention_functions=(seam.flash_attn_varlen_func, seam.flash_attn_with_kvcache))
    tokens, _ = ref.generate(prompts, 32)
    assert np.array_equal(np.asarray(tokens, np.int32), z["ref_tokens"][:6])
