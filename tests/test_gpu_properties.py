"""Size-independent properties of the attention kernels at the sizes the benchmark runs them at, where
the fp32 oracle would take minutes: exact linearity in V, independence of the rows from the batch they
are launched in, agreement of the paged and the dense path."""
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import BLOCK_SIZE, cdiv, config5_requests, generator, randn_bf16, table_tensor

pytestmark = pytest.mark.gpu

HQ, HKV, D = 16, 8, 128


def cu(lens, dev):
    return torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)


def prefill_step_lengths(budget=16384):
    """The first prefill step of the default bench workload: prompts packed first come first served."""
    lens, tot = [], 0
    for r in config5_requests(seed=0, n=512):
        n = len(r.prompt)
        if tot + n > budget:
            break
        lens.append(n); tot += n
    return lens


def run_prefill(cuda, q, k, v, lens):
    status = ops.new_status(cuda)
    c = cu(lens, cuda)
    out = ops.prefill_attn(q, k, v, c, c, max(lens), D ** -0.5, -1, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    return out


def test_prefill_full_step_linearity_and_batch_independence(cuda):
    lens = prefill_step_lengths()
    assert sum(lens) > 12000 and len(lens) > 8
    g = generator(3)
    T = sum(lens)
    q, k, v = (randn_bf16(g, T, h, D).to(cuda) for h in (HQ, HKV, HKV))
    out = run_prefill(cuda, q, k, v, lens)
    assert torch.isfinite(out.float()).all()
    # doubling V doubles every output exactly (a power of two commutes with every rounding on the way)
    out2 = run_prefill(cuda, q, k, v * 2, lens)
    assert torch.equal(out2, out * 2)
    # a row's result does not depend on which other sequences share the launch, nor on their order:
    # the two halves of the batch launched separately, and the batch reversed
    half = len(lens) // 2
    t_half = sum(lens[:half])
    a = run_prefill(cuda, q[:t_half], k[:t_half], v[:t_half], lens[:half])
    b = run_prefill(cuda, q[t_half:], k[t_half:], v[t_half:], lens[half:])
    assert torch.equal(torch.cat([a, b]), out)
    offs = [0] + torch.tensor(lens).cumsum(0).tolist()
    order = list(reversed(range(len(lens))))
    idx = torch.cat([torch.arange(offs[i], offs[i + 1]) for i in order]).to(cuda)
    rev = run_prefill(cuda, q[idx], k[idx], v[idx], [lens[i] for i in order])
    assert torch.equal(rev, out[idx])
    # the first query of every sequence sees one key: its output is that key's value row
    first = torch.tensor(offs[:-1], device=cuda)
    group = HQ // HKV
    assert torch.equal(out[first], v[first].repeat_interleave(group, dim=1))


def test_prefill_paged_equals_dense_on_a_full_step(cuda):
    lens = prefill_step_lengths()
    g = generator(4)
    T = sum(lens)
    q, k, v = (randn_bf16(g, T, h, D).to(cuda) for h in (HQ, HKV, HKV))
    dense = run_prefill(cuda, q, k, v, lens)
    nblk = [cdiv(n, BLOCK_SIZE) for n in lens]
    pool_blocks = sum(nblk) + 3
    perm = torch.randperm(pool_blocks, generator=g).tolist()
    tables, nxt = [], 0
    for n in nblk:
        tables.append(perm[nxt:nxt + n]); nxt += n
    k_pool = torch.full((pool_blocks, BLOCK_SIZE, HKV, D), float("nan"), dtype=torch.bfloat16, device=cuda)
    v_pool = torch.full_like(k_pool, float("nan"))          # unwritten slots must never reach a result
    off = 0
    for n, blocks in zip(lens, tables):
        for i, blk in enumerate(blocks):
            m = min(BLOCK_SIZE, n - i * BLOCK_SIZE)
            k_pool[blk, :m] = k[off + i * BLOCK_SIZE: off + i * BLOCK_SIZE + m]
            v_pool[blk, :m] = v[off + i * BLOCK_SIZE: off + i * BLOCK_SIZE + m]
        off += n
    status = ops.new_status(cuda)
    c = cu(lens, cuda)
    paged = ops.prefill_attn(q, k_pool, v_pool, c, c, max(lens), D ** -0.5, -1,
                             block_table=table_tensor(tables).to(cuda), status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert torch.equal(paged, dense)


def test_decode_512_sequences_linearity(cuda):
    """The decode batch of the default bench workload right after its prefills: 512 sequences."""
    g = generator(5)
    lens = [len(r.prompt) + 1 for r in config5_requests(seed=0, n=512)]
    nblk = [cdiv(n, BLOCK_SIZE) for n in lens]
    pool_blocks = sum(nblk) + 1
    perm = torch.randperm(pool_blocks, generator=g).tolist()
    tables, nxt = [], 0
    for n in nblk:
        tables.append(perm[nxt:nxt + n]); nxt += n
    k_pool = randn_bf16(g, pool_blocks, BLOCK_SIZE, HKV, D).to(cuda)
    v_pool = randn_bf16(g, pool_blocks, BLOCK_SIZE, HKV, D).to(cuda)
    q = randn_bf16(g, len(lens), HQ, D).to(cuda)
    seqlens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    bt = table_tensor(tables).to(cuda)
    ws = ops.decode_workspace(len(lens), HQ, D, cuda)
    ops.decode_plan(seqlens, -1, HQ, HKV, D, ws, block_table=bt, block_size=BLOCK_SIZE)
    out = ops.decode_attn(q, k_pool, v_pool, seqlens, bt, D ** -0.5, -1, ws)
    out2 = ops.decode_attn(q, k_pool, v_pool * 2, seqlens, bt, D ** -0.5, -1, ws)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out2, out * 2)
    # every output is a convex combination of value rows: it stays inside their range
    assert out.float().abs().max().item() <= v_pool.float().abs().max().item()
    # the same batch in reverse order: the cut into work ranges differs, so agreement is to rounding
    rev = list(reversed(range(len(lens))))
    ridx = torch.tensor(rev, device=cuda)
    seq_r, bt_r = seqlens[ridx].contiguous(), bt[ridx].contiguous()
    ops.decode_plan(seq_r, -1, HQ, HKV, D, ws, block_table=bt_r, block_size=BLOCK_SIZE)
    out_r = ops.decode_attn(q[ridx].contiguous(), k_pool, v_pool, seq_r, bt_r, D ** -0.5, -1, ws)
    torch.cuda.synchronize()
    diff = (out_r.float() - out[ridx].float()).abs()
    assert diff.max().item() <= 2e-2 and diff.mean().item() <= 2e-3


def test_prefill_random_ragged_batches_are_deterministic_and_clean(cuda):
    """Many differently shaped launches back to back (what a serving loop does): a CTA works through dozens
    of items per launch in an order that depends on timing, so every launch is run twice and must give
    the same bits, finite values and a clean status word."""
    g = generator(21)
    status = ops.new_status(cuda)
    for it in range(60):
        n_long = int(torch.randint(0, 4, (1,), generator=g))
        n_short = int(torch.randint(1, 48, (1,), generator=g))
        lens = [int(x) for x in torch.randint(600, 3000, (n_long,), generator=g)] + \
               [int(x) for x in torch.randint(1, 300, (n_short,), generator=g)]
        order = torch.randperm(len(lens), generator=g).tolist()
        lens = [lens[i] for i in order]
        T = sum(lens)
        qkv = randn_bf16(g, T, (HQ + 2 * HKV) * D).to(cuda)
        q, k, v = (t.view(T, -1, D) for t in qkv.split([HQ * D, HKV * D, HKV * D], dim=-1))
        c = cu(lens, cuda)
        a = ops.prefill_attn(q, k, v, c, c, max(lens), D ** -0.5, -1, status=status)
        b = ops.prefill_attn(q, k, v, c, c, max(lens), D ** -0.5, -1, status=status)
        assert torch.equal(a, b), f"launch {it}: two runs differ"
        assert torch.isfinite(a.float()).all(), f"launch {it}: non-finite output"
    torch.cuda.synchronize()
    ops.check_status(status)
