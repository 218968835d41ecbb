"""Fused RoPE + KV write (CUDA) against the reference's golden vectors and the eager oracle: bit-exact."""
from pathlib import Path

import numpy as np
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import generator, randn_bf16
from oracle import rope_kv
from tests.helpers import poison_pool

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"


def bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.int16).cpu()


@pytest.mark.parametrize("name", ["qwen3", "gemma3_global", "gemma3_local"])
def test_rope_matches_reference_golden(cuda, name):
    z = np.load(GOLD / "rope.npz")
    hq, hkv, d, max_pos = z[f"{name}/meta"].tolist()
    theta = float(z[f"{name}/theta"][0])
    table = rope_kv.cos_sin_table(d, max_pos, theta)
    pos = torch.from_numpy(z[f"{name}/positions"])
    assert torch.equal(table[pos], torch.from_numpy(z[f"{name}/table_rows"]))   # same table as the reference
    q = torch.from_numpy(z[f"{name}/q"]).view(torch.bfloat16).to(cuda)
    k = torch.from_numpy(z[f"{name}/k"]).view(torch.bfloat16).to(cuda)
    v = torch.zeros_like(k)
    ops.rope_kv_write(q, k, v, pos.to(cuda), table.to(cuda), None, None, None, k_in_place=True)
    torch.cuda.synchronize()
    assert torch.equal(bits(q), torch.from_numpy(z[f"{name}/q_out"]))
    assert torch.equal(bits(k), torch.from_numpy(z[f"{name}/k_out"]))


# (the kernel gives a warp 1, 2 or 5 groups of 32 tasks depending on the token count: 301 / 1200 / 3000 tokens of
# the Qwen3 shape and 2500 of the Gemma3 shape cover the three variants)
@pytest.mark.parametrize("hq,hkv,d,T", [(16, 8, 128, 301), (4, 1, 256, 301), (2, 2, 64, 301), (16, 8, 128, 1200),
                                        (16, 8, 128, 3000), (4, 1, 256, 2500), (3, 1, 48, 700)])
def test_fused_write_bit_exact_with_strided_qkv(cuda, hq, hkv, d, T):
    """q/k/v are column slices of one packed GEMM output (row stride != heads*dim), some slots are -1."""
    g = generator(11)
    nblk, bs = -(-T // 256) + 4, 256
    max_pos = 2048
    table = rope_kv.cos_sin_table(d, max_pos, 1e6)
    qkv = randn_bf16(g, T, (hq + 2 * hkv) * d)
    pos = torch.randint(0, max_pos, (T,), generator=g)
    slots = torch.randperm(nblk * bs, generator=g)[:T].to(torch.int32)
    slots[::7] = -1
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.view(T, hq, d), k.view(T, hkv, d), v.view(T, hkv, d)
    q_ref, k_ref = rope_kv.apply_rope(pos, q, k, table)
    kc_ref, vc_ref = poison_pool(nblk, hkv, d, bs), poison_pool(nblk, hkv, d, bs)
    rope_kv.store_kvcache(k_ref, v, kc_ref, vc_ref, slots)

    qkv_d = qkv.to(cuda)
    qd, kd, vd = qkv_d.split([hq * d, hkv * d, hkv * d], dim=-1)
    qd, kd, vd = qd.view(T, hq, d), kd.view(T, hkv, d), vd.view(T, hkv, d)
    kc, vc = poison_pool(nblk, hkv, d, bs).to(cuda), poison_pool(nblk, hkv, d, bs).to(cuda)
    status = ops.new_status(cuda)
    ops.rope_kv_write(qd, kd, vd, pos.to(cuda), table.to(cuda), slots.to(cuda), kc, vc, k_in_place=True, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert torch.equal(bits(qd), bits(q_ref))
    assert torch.equal(bits(kd), bits(k_ref))
    assert torch.equal(bits(vd), bits(v))                      # v untouched
    assert torch.equal(bits(kc), bits(kc_ref))                 # NaN poison compares equal bit-wise
    assert torch.equal(bits(vc), bits(vc_ref))


def test_plain_store_without_rotation(cuda):
    """cos_sin=None is the reference's store_kvcache: a pure scatter of k and v."""
    g = generator(12)
    T, hkv, d, nblk, bs = 64, 8, 128, 2, 256
    k, v = randn_bf16(g, T, hkv, d), randn_bf16(g, T, hkv, d)
    slots = torch.randperm(nblk * bs, generator=g)[:T].to(torch.int32)
    kc_ref, vc_ref = poison_pool(nblk, hkv, d, bs), poison_pool(nblk, hkv, d, bs)
    rope_kv.store_kvcache(k, v, kc_ref, vc_ref, slots)
    kc, vc = poison_pool(nblk, hkv, d, bs).to(cuda), poison_pool(nblk, hkv, d, bs).to(cuda)
    ops.rope_kv_write(None, k.to(cuda), v.to(cuda), None, None, slots.to(cuda), kc, vc, k_in_place=False)
    torch.cuda.synchronize()
    assert torch.equal(bits(kc), bits(kc_ref)) and torch.equal(bits(vc), bits(vc_ref))


def test_out_of_range_slot_and_position_are_reported(cuda):
    g = generator(13)
    T, hq, hkv, d = 4, 2, 1, 128
    table = rope_kv.cos_sin_table(d, 16, 1e4).to(cuda)
    q, k, v = randn_bf16(g, T, hq, d).to(cuda), randn_bf16(g, T, hkv, d).to(cuda), randn_bf16(g, T, hkv, d).to(cuda)
    kc, vc = torch.zeros(1, 256, hkv, d, dtype=torch.bfloat16, device=cuda), torch.zeros(1, 256, hkv, d, dtype=torch.bfloat16, device=cuda)
    status = ops.new_status(cuda)
    ops.rope_kv_write(q, k, v, torch.tensor([0, 1, 2, 3], device=cuda), table,
                      torch.tensor([0, 1, 999, 3], dtype=torch.int32, device=cuda), kc, vc, status=status)
    torch.cuda.synchronize()
    assert status[0].item() == 1 and status[1].item() == 2
    status.zero_()
    ops.rope_kv_write(q, k, v, torch.tensor([0, 1, 2, 77], device=cuda), table, None, None, None, status=status)
    torch.cuda.synchronize()
    assert status[0].item() == 3 and status[1].item() == 3


@pytest.mark.parametrize("hq,hkv,d,unit_offset,T", [(16, 8, 128, False, 257), (4, 1, 256, True, 257), (8, 2, 128, True, 257),
                                                    (16, 8, 128, False, 1100), (16, 8, 128, False, 2600),
                                                    (4, 1, 256, True, 2400)])
def test_fused_qk_norm_rope_write_matches_unfused_sequence(cuda, hq, hkv, d, unit_offset, T):
    """norm -> bf16 -> RoPE -> cache, fused: equal to the oracle up to the summation order of the squares."""
    g = generator(21)
    nblk, bs, max_pos, eps = -(-T // 256) + 3, 256, 4096, 1e-6
    table = rope_kv.cos_sin_table(d, max_pos, 1e6)
    qkv = randn_bf16(g, T, (hq + 2 * hkv) * d) * 3
    qw, kw = randn_bf16(g, d) * 0.5 + (0 if unit_offset else 1), randn_bf16(g, d) * 0.5 + (0 if unit_offset else 1)
    pos = torch.randint(0, max_pos, (T,), generator=g)
    slots = torch.randperm(nblk * bs, generator=g)[:T].to(torch.int32)
    slots[::5] = -1
    q, k, v = (t.view(T, -1, d) for t in qkv.split([hq * d, hkv * d, hkv * d], dim=-1))
    qn, kn = rope_kv.qk_norm(q, qw, eps, unit_offset), rope_kv.qk_norm(k, kw, eps, unit_offset)
    q_ref, k_ref = rope_kv.apply_rope(pos, qn, kn, table)
    kc_ref, vc_ref = torch.zeros(nblk, bs, hkv, d, dtype=torch.bfloat16), torch.zeros(nblk, bs, hkv, d, dtype=torch.bfloat16)
    rope_kv.store_kvcache(k_ref, v, kc_ref, vc_ref, slots)

    qkv_d = qkv.to(cuda)
    qd, kd, vd = (t.view(T, -1, d) for t in qkv_d.split([hq * d, hkv * d, hkv * d], dim=-1))
    kc, vc = torch.zeros_like(kc_ref, device=cuda), torch.zeros_like(vc_ref, device=cuda)
    status = ops.new_status(cuda)
    ops.qk_norm_rope_kv_write(qd, kd, vd, qw.to(cuda), kw.to(cuda), eps, unit_offset, pos.to(cuda), table.to(cuda),
                              slots.to(cuda), kc, vc, k_in_place=True, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert torch.equal(bits(vc), bits(vc_ref)) and torch.equal(bits(vd), bits(v))          # V is a pure copy
    for got, want, name in ((qd, q_ref, "q"), (kd, k_ref, "k"), (kc, kc_ref, "k_cache")):
        got, want = got.float().cpu(), want.float()
        same = (got == want).float().mean().item()
        rel = ((got - want).abs() / want.abs().clamp_min(1.0)).max().item()      # one bf16 ulp of O(1) values
        assert same >= 0.995 and rel <= 2 ** -6, f"{name}: {same:.5f} equal, max rel diff {rel:.4g}"
