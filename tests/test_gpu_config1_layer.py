"""The single-layer correctness configuration, end to end at layer level: one Qwen3-0.6B attention layer, 8 sequences with prompt
lengths U[16,512] (seed 0), 64-block pool, block tables from a seeded permutation; RoPE (theta 1e6) + KV write +
causal varlen prefill, then 32 single-token decode steps with fresh N(0,1) q/k/v.  The attention layer (CUDA)
runs next to the CPU oracle: outputs within tolerance at every step, KV pool bit-identical at the end."""
import pytest
import torch

from mini_vllm_b200.executor.context import Context
from mini_vllm_b200.models.layers.attention import FlashAttention
from mini_vllm_b200.workloads import config1, randn_bf16, table_tensor
from oracle import attention as oattn
from oracle import packing as opack
from oracle import rope_kv
from tests.helpers import assert_close_attn

pytestmark = pytest.mark.gpu


def test_config1_prefill_then_32_decode_steps(cuda):
    case, g = config1()
    hq, hkv, d, bs = 16, 8, 128, 256
    lens, reserved = list(case.prefill_lens), case.prefill_blocks     # block lists sized for the 32 decode steps
    held = lambda: [b[:-(-n // 256)] for n, b in zip(lens, reserved)]     # the blocks a sequence owns right now
    table = rope_kv.cos_sin_table(d, 4096, 1e6)
    table_d = table.to(cuda)
    kc_ref, vc_ref = torch.zeros(64, bs, hkv, d, dtype=torch.bfloat16), torch.zeros(64, bs, hkv, d, dtype=torch.bfloat16)
    layer = FlashAttention(hq, d, d ** -0.5, hkv)
    layer.k_cache, layer.v_cache = kc_ref.to(cuda), vc_ref.to(cuda)

    # ---- prefill
    tokens = [[0] * n for n in lens]
    p = opack.build_prefill_input(tokens, held(), [0] * 8, bs)
    T = sum(lens)
    q, k, v = randn_bf16(g, T, hq, d), randn_bf16(g, T, hkv, d), randn_bf16(g, T, hkv, d)
    pos, slots, cu = torch.from_numpy(p["positions"]), torch.from_numpy(p["slot_mapping"]), torch.from_numpy(p["cu_seqlens_q"])
    q_ref, k_ref = rope_kv.apply_rope(pos, q, k, table)
    rope_kv.store_kvcache(k_ref, v, kc_ref, vc_ref, slots)
    want = oattn.prefill(q_ref, k_ref, v, cu, cu)
    ctx = Context(prefill=True, positions=pos.to(cuda), slot_mapping=slots.to(cuda), cu_seqlens_q=cu.to(cuda),
                  cu_seqlens_k=cu.to(cuda), max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    got = layer.forward_fused(ctx, q.to(cuda), k.to(cuda), v.to(cuda), ctx.positions, table_d)
    assert_close_attn(got, want, "config 1 prefill")

    # ---- 32 decode steps
    for step in range(32):
        lens = [n + 1 for n in lens]
        bt = table_tensor(held())
        pd = opack.build_decode_input([[0] * n for n in lens], held(), bs)
        q, k, v = randn_bf16(g, 8, hq, d), randn_bf16(g, 8, hkv, d), randn_bf16(g, 8, hkv, d)
        pos, slots = torch.from_numpy(pd["positions"]), torch.from_numpy(pd["slot_mapping"])
        seqlens = torch.from_numpy(pd["cache_seqlens"])
        q_ref, k_ref = rope_kv.apply_rope(pos, q, k, table)
        rope_kv.store_kvcache(k_ref, v, kc_ref, vc_ref, slots)
        want = oattn.decode(q_ref, kc_ref, vc_ref, seqlens, bt)
        ctx = Context(prefill=False, positions=pos.to(cuda), slot_mapping=slots.to(cuda), cache_seqlens=seqlens.to(cuda),
                      block_table=bt.to(cuda))
        got = layer.forward_fused(ctx, q.to(cuda), k.to(cuda), v.to(cuda), ctx.positions, table_d)
        assert got.shape == (8, 1, hq, d)
        assert_close_attn(got[:, 0], want, f"config 1 decode step {step}")
    torch.cuda.synchronize()
    assert torch.equal(layer.k_cache.cpu().view(torch.int16), kc_ref.view(torch.int16)), "K pool not bit-identical"
    assert torch.equal(layer.v_cache.cpu().view(torch.int16), vc_ref.view(torch.int16)), "V pool not bit-identical"
