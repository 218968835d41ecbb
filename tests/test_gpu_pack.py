"""Device batch packing (CUDA) against the reference executor's golden outputs: bit-exact."""
from pathlib import Path

import numpy as np
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import cdiv, generator, randint
from oracle import packing as opack

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"
BS = 256


def prefill_meta(seq_len, cached, nblocks, blocks_flat, new_tokens):
    blk_off = np.concatenate([[0], np.cumsum(nblocks)]).astype(np.int32)
    return torch.from_numpy(np.concatenate([seq_len, cached, blk_off, blocks_flat, new_tokens]).astype(np.int32))


def run_prefill(cuda, seq_len, cached, nblocks, blocks_flat, tokens_flat, want_table):
    seq_len, cached, nblocks = (np.asarray(x, np.int32) for x in (seq_len, cached, nblocks))
    starts = np.concatenate([[0], np.cumsum(seq_len)])[:-1]
    new_tokens = np.concatenate([tokens_flat[s + c:s + n] for s, c, n in zip(starts, cached, seq_len)] + [np.zeros(0, np.int32)])
    T = int((seq_len - cached).sum())
    meta = prefill_meta(seq_len, cached, nblocks, np.asarray(blocks_flat, np.int32), new_tokens).to(cuda)
    status = ops.new_status(cuda)
    out = ops.pack_prefill(meta, len(seq_len), T, int(nblocks.sum()), int(max(nblocks.max(), 1)), BS, want_table, status)
    torch.cuda.synchronize()
    ops.check_status(status)
    return out


@pytest.mark.parametrize("name", ["plain", "edges", "prefix", "single"])
def test_prefill_matches_reference_golden(cuda, name):
    z = np.load(GOLD / "packing.npz")
    pre = f"{name}/prefill/"
    has_table = pre + "block_table" in z
    out = run_prefill(cuda, z[pre + "tok_len"], z[pre + "cached"], z[pre + "nblocks"], z[pre + "blocks_flat"],
                      z[pre + "tokens_flat"], has_table)
    for key in ("input_ids", "positions", "slot_mapping", "cu_seqlens_q", "cu_seqlens_k"):
        got, want = out[key].cpu().numpy(), z[pre + key]
        assert got.dtype == want.dtype and np.array_equal(got, want), key
    if has_table:
        assert np.array_equal(out["block_table"].cpu().numpy(), z[pre + "block_table"])


@pytest.mark.parametrize("name", ["plain", "edges", "prefix", "single"])
def test_decode_matches_reference_golden(cuda, name):
    z = np.load(GOLD / "packing.npz")
    pre = f"{name}/decode/"
    seq_len, nblocks = z[pre + "tok_len"], z[pre + "nblocks"]
    B, W = len(seq_len), int(nblocks.max())
    blk_off = np.concatenate([[0], np.cumsum(nblocks)]).astype(np.int32)
    meta = torch.from_numpy(np.concatenate([seq_len, blk_off, z[pre + "blocks_flat"], z[pre + "last_token"],
                                            np.full(B, -1)]).astype(np.int32)).to(cuda)
    padded, stride = B + 3, W + 5                     # static graph buffers are larger than the batch
    ids = torch.full((padded,), 7, dtype=torch.int64, device=cuda)
    pos = torch.full((padded,), 7, dtype=torch.int64, device=cuda)
    slot = torch.full((padded,), 7, dtype=torch.int32, device=cuda)
    lens = torch.full((padded,), 7, dtype=torch.int32, device=cuda)
    bt = torch.full((padded, stride), 7, dtype=torch.int32, device=cuda)
    status = ops.new_status(cuda)
    ops.pack_decode(meta, B, int(nblocks.sum()), W, BS, ids, pos, slot, lens, bt, padded_seqs=padded, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert np.array_equal(ids[:B].cpu().numpy(), z[pre + "input_ids"])
    assert np.array_equal(pos[:B].cpu().numpy(), z[pre + "positions"])
    assert np.array_equal(slot[:B].cpu().numpy(), z[pre + "slot_mapping"])
    assert np.array_equal(lens[:B].cpu().numpy(), z[pre + "cache_seqlens"])
    assert np.array_equal(bt[:B, :W].cpu().numpy(), z[pre + "block_table"])
    # padding rows: slot -1, length 0, table -1; columns beyond the width untouched
    assert (slot[B:] == -1).all() and (lens[B:] == 0).all() and (ids[B:] == 0).all() and (pos[B:] == 0).all()
    assert (bt[B:, :W] == -1).all() and (bt[:, W:] == 7).all()


def test_decode_tokens_from_previous_sampler_output(cuda):
    seq_len = np.asarray([10, 300, 257], np.int32)
    blocks = [[3], [5, 1], [0, 2]]
    blk_off = np.asarray([0, 1, 3, 5], np.int32)
    src = np.asarray([2, -1, 0], np.int32)
    host_tok = np.asarray([111, 222, 333], np.int32)
    meta = torch.from_numpy(np.concatenate([seq_len, blk_off, sum(blocks, []), host_tok, src]).astype(np.int32)).to(cuda)
    prev = torch.tensor([900, 901, 902, 903], dtype=torch.int64, device=cuda)
    B = 3
    ids = torch.zeros(B, dtype=torch.int64, device=cuda); pos = torch.zeros_like(ids)
    slot = torch.zeros(B, dtype=torch.int32, device=cuda); lens = torch.zeros_like(slot)
    bt = torch.zeros(B, 2, dtype=torch.int32, device=cuda)
    ops.pack_decode(meta, B, 5, 2, BS, ids, pos, slot, lens, bt, prev_sampled=prev)
    torch.cuda.synchronize()
    assert ids.tolist() == [902, 222, 900]
    want = opack.build_decode_input([[0] * n for n in seq_len], blocks, BS)
    assert np.array_equal(slot.cpu().numpy(), want["slot_mapping"])


def test_prefill_large_random_against_oracle(cuda):
    """Config-3-sized prefill batch (16 sequences, half with a 512-token cached prefix) plus a 600-sequence batch."""
    for seed, nseq, lo, hi in ((0, 16, 100, 2048), (1, 600, 1, 40)):
        g = generator(seed)
        suffix = randint(g, lo, hi, nseq)
        cached = [512 if (i % 2 == 0 and nseq == 16) else 0 for i in range(nseq)]
        lens = [c + s for c, s in zip(cached, suffix)]
        perm = torch.randperm(4000, generator=g).tolist()
        blocks, cur = [], 0
        for n in lens:
            nb = cdiv(n, BS)
            blocks.append(perm[cur:cur + nb]); cur += nb
        tokens = [torch.randint(0, 150000, (n,), generator=g).tolist() for n in lens]
        want = opack.build_prefill_input(tokens, blocks, cached, BS)
        flat = np.asarray([t for ts in tokens for t in ts], np.int32)
        out = run_prefill(cuda, lens, cached, [len(b) for b in blocks], [x for b in blocks for x in b], flat,
                          want["block_table"] is not None)
        for key in ("input_ids", "positions", "slot_mapping", "cu_seqlens_q", "cu_seqlens_k"):
            assert np.array_equal(out[key].cpu().numpy(), want[key]), key
        if want["block_table"] is not None:
            assert np.array_equal(out["block_table"].cpu().numpy(), want["block_table"])


def test_warmup_requests_without_blocks_get_slot_minus_one(cuda):
    out = run_prefill(cuda, [64] * 10, [0] * 10, [0] * 10, [], np.zeros(640, np.int32), False)
    assert (out["slot_mapping"] == -1).all() and out["cu_seqlens_q"].tolist() == list(range(0, 641, 64))


def test_executor_build_block_table_alone(cuda):
    """``Executor._build_block_table`` (executor.py:156-163) on its own: ``[B, max blocks]`` int32, rows right-padded
    with -1, packed on the device from the requests' block lists.  Driven through the executor's method on an object
    that carries only what the method reads."""
    from types import SimpleNamespace
    from mini_vllm_b200.executor.executor import Executor, _Staging
    blocks = [[5, 9, 2], [7], [], [1, 3, 8, 11, 4, 6, 0], [10, 12]]
    reqs = [SimpleNamespace(tokens=[0] * (len(b) * BS), blocks=b) for b in blocks]
    ex = object.__new__(Executor)
    ex.block_size, ex.status, ex._step, ex._stages = BS, ops.new_status(cuda), 0, [_Staging(cuda) for _ in range(Executor.RING)]
    table = Executor._build_block_table(ex, reqs)
    torch.cuda.synchronize()
    ops.check_status(ex.status)
    want = np.full((len(blocks), 7), -1, np.int32)
    for i, b in enumerate(blocks):
        want[i, :len(b)] = b
    assert table.dtype == torch.int32 and np.array_equal(table.cpu().numpy(), want)
    assert np.array_equal(want, opack.build_block_table(blocks))
