"""Secondary cross-check of the attention kernels against flash_attn, on the GPU.

The reference names ``flash_attn`` as the implementation its attention calls are interchangeable with
(``minivllm/models/layers/attention.py:6``: the commented-out import; README).  Where the installed flash_attn
runs on this GPU, the same two entry points the reference would call - ``flash_attn_varlen_func`` and
``flash_attn_with_kvcache`` with a block table - are given the inputs of the CUDA kernels under test and both
bf16 results must agree within the attention tolerance.  The primary check stays the fp32 oracle; this one
pins the kernels to an independent implementation of the same calls.  Skipped where flash_attn cannot be
imported or has no kernel for the device.
"""
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import BLOCK_SIZE, cdiv, config1, config3, generator, randn_bf16
from tests.helpers import assert_close_attn, fill_paged, sequential_tables, table_tensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fa(cuda):
    try:
        import flash_attn
        q = torch.zeros(4, 2, 64, dtype=torch.bfloat16, device=cuda)
        cu = torch.tensor([0, 4], dtype=torch.int32, device=cuda)
        flash_attn.flash_attn_varlen_func(q, q, q, cu, cu, 4, 4, causal=True)
        torch.cuda.synchronize()
    except Exception as e:                              # import error, or "no kernel image" for this device
        pytest.skip(f"flash_attn does not run here: {type(e).__name__}: {str(e)[:120]}")
    return flash_attn


def cu(lens, dev):
    return torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)


@pytest.mark.parametrize("hq,hkv,d,window", [(16, 8, 128, -1), (4, 1, 256, -1), (4, 1, 256, 64), (16, 8, 128, 300)])
def test_prefill_dense_agrees_with_flash_attn(cuda, fa, hq, hkv, d, window):
    case, g = config1()
    lens = case.prefill_lens + [1, 129, 1500]
    T = sum(lens)
    q, k, v = (randn_bf16(g, T, h, d).to(cuda) for h in (hq, hkv, hkv))
    c = cu(lens, cuda)
    ours = ops.prefill_attn(q, k, v, c, c, max(lens), d ** -0.5, window)
    theirs = fa.flash_attn_varlen_func(q, k, v, c, c, max(lens), max(lens), softmax_scale=d ** -0.5, causal=True,
                                       window_size=(window, 0) if window >= 0 else (-1, -1))
    torch.cuda.synchronize()
    assert_close_attn(ours, theirs, f"prefill vs flash_attn_varlen_func hq={hq} d={d} window={window}")


def test_prefill_with_cached_prefix_agrees_with_flash_attn(cuda, fa):
    """Config 3's prefill part: q_len < k_len for half the sequences, keys gathered through the block table."""
    case, g = config3()
    q_lens = [n - c for n, c in zip(case.prefill_lens, case.prefill_cached)]
    k_pool, v_pool = fill_paged(g, case.prefill_lens, case.prefill_blocks, case.pool_blocks, 8, 128)
    k_pool, v_pool = torch.nan_to_num(k_pool).to(cuda), torch.nan_to_num(v_pool).to(cuda)
    q = randn_bf16(g, sum(q_lens), 16, 128).to(cuda)
    cq, ck, bt = cu(q_lens, cuda), cu(case.prefill_lens, cuda), table_tensor(case.prefill_blocks).to(cuda)
    ours = ops.prefill_attn(q, k_pool, v_pool, cq, ck, max(q_lens), 128 ** -0.5, -1, block_table=bt)
    theirs = fa.flash_attn_varlen_func(q, k_pool, v_pool, cq, ck, max(q_lens), max(case.prefill_lens),
                                       softmax_scale=128 ** -0.5, causal=True, block_table=bt)
    torch.cuda.synchronize()
    assert_close_attn(ours, theirs, "paged prefill vs flash_attn_varlen_func with a block table")


@pytest.mark.parametrize("hq,hkv,d,window", [(16, 8, 128, -1), (4, 1, 256, -1), (4, 1, 256, 512)])
def test_decode_agrees_with_flash_attn(cuda, fa, hq, hkv, d, window):
    g = generator(50 + d + window)
    lens = [int(x) for x in torch.randint(1, 3000, (37,), generator=g)] + [1, 256, 257, 4096]
    num_blocks = sum(cdiv(n, BLOCK_SIZE) for n in lens) + 2
    tables = sequential_tables(g, lens, num_blocks)
    k_pool, v_pool = fill_paged(g, lens, tables, num_blocks, hkv, d)
    k_pool, v_pool = torch.nan_to_num(k_pool).to(cuda), torch.nan_to_num(v_pool).to(cuda)
    q = randn_bf16(g, len(lens), hq, d).to(cuda)
    seqlens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    bt = table_tensor(tables).to(cuda)
    ws = ops.decode_workspace(len(lens), hq, d, cuda)
    ops.decode_plan(seqlens, window, hq, hkv, d, ws, block_table=bt, block_size=BLOCK_SIZE)
    ours = ops.decode_attn(q, k_pool, v_pool, seqlens, bt, d ** -0.5, window, ws)
    theirs = fa.flash_attn_with_kvcache(q.unsqueeze(1), k_pool, v_pool, cache_seqlens=seqlens, block_table=bt,
                                        softmax_scale=d ** -0.5, causal=True,
                                        window_size=(window, 0) if window >= 0 else (-1, -1))[:, 0]
    torch.cuda.synchronize()
    assert_close_attn(ours, theirs, f"decode vs flash_attn_with_kvcache hq={hq} d={d} window={window}")
