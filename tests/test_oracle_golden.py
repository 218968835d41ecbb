"""The CPU oracle pinned against vectors produced by the reference's own code (tests/golden/make_golden.py)."""
import json
from pathlib import Path

import numpy as np
import torch

from oracle import packing as opack
from oracle import rope_kv
from oracle import attention as oattn
from oracle import sampler as osamp

GOLD = Path(__file__).parent / "golden"
BS = 256


def _split(flat, counts):
    out, cur = [], 0
    for c in counts:
        out.append(list(map(int, flat[cur:cur + c])))
        cur += c
    return out


def test_packing_oracle_matches_reference_executor():
    z = np.load(GOLD / "packing.npz")
    for name in ("plain", "edges", "prefix", "single"):
        pre = f"{name}/prefill/"
        tokens = _split(z[pre + "tokens_flat"], z[pre + "tok_len"])
        blocks = _split(z[pre + "blocks_flat"], z[pre + "nblocks"])
        got = opack.build_prefill_input(tokens, blocks, z[pre + "cached"].tolist(), BS)
        for key in ("input_ids", "positions", "slot_mapping", "cu_seqlens_q", "cu_seqlens_k"):
            assert got[key].dtype == z[pre + key].dtype and np.array_equal(got[key], z[pre + key]), (name, key)
        assert [got["max_seqlen_q"], got["max_seqlen_k"]] == z[pre + "max_seqlen"].tolist()
        if pre + "block_table" in z:
            assert np.array_equal(got["block_table"], z[pre + "block_table"])
        else:
            assert got["block_table"] is None
        pre = f"{name}/decode/"
        n = z[pre + "tok_len"]
        tokens = [[0] * (int(k) - 1) + [int(t)] for k, t in zip(n, z[pre + "last_token"])]
        blocks = _split(z[pre + "blocks_flat"], z[pre + "nblocks"])
        got = opack.build_decode_input(tokens, blocks, BS)
        for key in ("input_ids", "positions", "slot_mapping", "cache_seqlens", "block_table"):
            assert got[key].dtype == z[pre + key].dtype and np.array_equal(got[key], z[pre + key]), (name, key)


def test_rope_oracle_matches_reference_rotary_bitwise():
    z = np.load(GOLD / "rope.npz")
    for name in ("qwen3", "gemma3_global", "gemma3_local"):
        hq, hkv, d, max_pos = z[f"{name}/meta"].tolist()
        table = rope_kv.cos_sin_table(d, max_pos, float(z[f"{name}/theta"][0]))
        pos = torch.from_numpy(z[f"{name}/positions"])
        assert torch.equal(table[pos], torch.from_numpy(z[f"{name}/table_rows"]))
        q = torch.from_numpy(z[f"{name}/q"]).view(torch.bfloat16)
        k = torch.from_numpy(z[f"{name}/k"]).view(torch.bfloat16)
        q2, k2 = rope_kv.apply_rope(pos, q, k, table)
        assert np.array_equal(q2.view(torch.int16).numpy(), z[f"{name}/q_out"])
        assert np.array_equal(k2.view(torch.int16).numpy(), z[f"{name}/k_out"])


def test_store_kvcache_skips_minus_one():
    k = torch.arange(3 * 2 * 4, dtype=torch.float32).view(3, 2, 4).to(torch.bfloat16)
    kc, vc = torch.zeros(2, 4, 2, 4, dtype=torch.bfloat16), torch.zeros(2, 4, 2, 4, dtype=torch.bfloat16)
    rope_kv.store_kvcache(k, k + 1, kc, vc, torch.tensor([5, -1, 0], dtype=torch.int32))
    assert torch.equal(kc.view(8, 2, 4)[5], k[0]) and torch.equal(kc.view(8, 2, 4)[0], k[2])
    assert kc.view(8, 2, 4)[[1, 2, 3, 4, 6, 7]].abs().sum() == 0
    assert torch.equal(vc.view(8, 2, 4)[5], k[0] + 1)


def test_attention_oracle_paged_equals_dense_and_decode_equals_last_prefill_row():
    g = torch.Generator().manual_seed(0)
    hq, hkv, d = 4, 2, 32
    lens = [5, 300, 257]
    T = sum(lens)
    q = torch.randn(T, hq, d, generator=g).to(torch.bfloat16)
    k = torch.randn(T, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(T, hkv, d, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, 5, 305, 562], dtype=torch.int32)
    dense = oattn.prefill(q, k, v, cu, cu, out_dtype=torch.float32)
    tables = [[3], [0, 4], [2, 1]]
    kp, vp = torch.zeros(5, BS, hkv, d, dtype=torch.bfloat16), torch.zeros(5, BS, hkv, d, dtype=torch.bfloat16)
    for s, (n, blks) in enumerate(zip(lens, tables)):
        for i, b in enumerate(blks):
            lo, hi = i * BS, min(n, (i + 1) * BS)
            kp[b, :hi - lo], vp[b, :hi - lo] = k[cu[s] + lo:cu[s] + hi], v[cu[s] + lo:cu[s] + hi]
    bt = torch.tensor([[3, -1], [0, 4], [2, 1]], dtype=torch.int32)
    paged = oattn.prefill(q, kp, vp, cu, cu, block_table=bt, out_dtype=torch.float32)
    assert torch.allclose(dense, paged, atol=1e-6)
    # prefix-cached: only the last 7 queries of sequence 1
    cq = torch.tensor([0, 0, 7, 7], dtype=torch.int32)
    part = oattn.prefill(q[298:305], kp, vp, cq, cu, block_table=bt, out_dtype=torch.float32)
    assert torch.allclose(part, dense[298:305], atol=1e-6)
    # decode = the last prefill row of each sequence
    last = torch.stack([q[4], q[304], q[561]])
    dec = oattn.decode(last, kp, vp, torch.tensor(lens, dtype=torch.int32), bt, out_dtype=torch.float32)
    assert torch.allclose(dec, dense[[4, 304, 561]], atol=1e-6)
    # window: row 304 with left=10 sees keys 289..299 of its sequence only
    win = oattn.decode(last, kp, vp, torch.tensor(lens, dtype=torch.int32), bt, window_left=10, out_dtype=torch.float32)
    ks, vs = k[5 + 289:305].float(), v[5 + 289:305].float()
    s = torch.einsum("hd,thd->ht", q[304].float().view(hkv, 2, d).reshape(hq, d), ks.repeat_interleave(2, 1)) * d ** -0.5
    ref = torch.einsum("ht,thd->hd", torch.softmax(s, -1), vs.repeat_interleave(2, 1))
    assert torch.allclose(win[1], ref, atol=1e-5)
    # padded rows give zeros
    z = oattn.decode(last, kp, vp, torch.tensor([0, 0, 0], dtype=torch.int32), bt)
    assert (z == 0).all()


def test_philox_known_answers():
    """Random123 known-answer vectors for Philox4x32-10."""
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        got = osamp.philox4x32(np.asarray([ctr], np.uint32), np.asarray([key], np.uint32))[0]
        assert tuple(int(x) for x in got) == want
    u = osamp.uniform_open(1, 2, 3, 1001)
    assert u.shape == (3, 1001) and (u > 0).all() and (u < 1).all()


def test_greedy_sampler_ties_take_lowest_index():
    logits = torch.tensor([[1.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0]], dtype=torch.bfloat16)
    assert osamp.greedy(logits).tolist() == [1, 0]
    assert osamp.greedy(logits, torch.tensor([0.5, 2.0])).tolist() == [1, 0]
    assert osamp.sample(logits, None, torch.tensor([1, 1], dtype=torch.int32), 3, 4).tolist()[0] in (1, 2)
