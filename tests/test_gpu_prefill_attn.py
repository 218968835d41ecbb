"""Varlen causal prefill attention (tcgen05, through the C ABI) against the fp32 oracle."""
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import BLOCK_SIZE, cdiv, config1, config3, generator, randn_bf16
from oracle import attention as oattn
from tests.helpers import assert_close_attn, fill_paged, sequential_tables, table_tensor

pytestmark = pytest.mark.gpu


def cu(lens):
    return torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)


def with_work_list(cuda, out, q_lens, k_lens, hq, hkv, d, call):
    """The same launch with its work given as a list (every case of this file runs both ways): bit-identical to
    the plain grid, also when the list comes in another order."""
    import numpy as np
    items = ops.build_prefill_items(q_lens, k_lens, ops.prefill_item_rows(hq, hkv, d))
    assert sorted(map(tuple, items.tolist())) == [(s, b) for s, n in enumerate(q_lens)
                                                  for b in range(cdiv(n, ops.prefill_item_rows(hq, hkv, d)))]
    for order in (items, items[::-1].copy()):
        status = ops.new_status(cuda)
        listed = call(torch.from_numpy(order).to(cuda), status)
        torch.cuda.synchronize()
        ops.check_status(status)
        assert torch.equal(listed, out), "the work-list launch differs from the grid launch"


def run_dense(cuda, lens, hq, hkv, d, window_left=-1, seed=0, packed_qkv=False):
    g = generator(seed)
    T = sum(lens)
    if packed_qkv:                     # q/k/v are column slices of one GEMM output, as in the Qwen3 layer
        qkv = randn_bf16(g, T, (hq + 2 * hkv) * d)
        q, k, v = (t.view(T, -1, d) for t in qkv.split([hq * d, hkv * d, hkv * d], dim=-1))
        qkv_d = qkv.to(cuda)
        qd, kd, vd = (t.view(T, -1, d) for t in qkv_d.split([hq * d, hkv * d, hkv * d], dim=-1))
    else:
        q, k, v = randn_bf16(g, T, hq, d), randn_bf16(g, T, hkv, d), randn_bf16(g, T, hkv, d)
        qd, kd, vd = q.to(cuda), k.to(cuda), v.to(cuda)
    cq = cu(lens)
    want = oattn.prefill(q, k, v, cq, cq, window_left=window_left)
    status = ops.new_status(cuda)
    out = ops.prefill_attn(qd, kd, vd, cq.to(cuda), cq.to(cuda), max(lens), d ** -0.5, window_left, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert_close_attn(out, want, f"prefill dense lens={lens[:4]}.. hq={hq} hkv={hkv} d={d} w={window_left}")
    with_work_list(cuda, out, lens, lens, hq, hkv, d,
                   lambda items, st: ops.prefill_attn(qd, kd, vd, cq.to(cuda), cq.to(cuda), max(lens), d ** -0.5,
                                                      window_left, status=st, items=items))


def run_paged(cuda, q_lens, k_lens, hq, hkv, d, window_left=-1, seed=0, tables=None, num_blocks=None, g=None):
    g = g or generator(seed)
    num_blocks = num_blocks or sum(cdiv(n, BLOCK_SIZE) for n in k_lens) + 2
    tables = tables or sequential_tables(g, k_lens, num_blocks)
    k_pool, v_pool = fill_paged(g, k_lens, tables, num_blocks, hkv, d)
    q = randn_bf16(g, sum(q_lens), hq, d)
    cq, ck, bt = cu(q_lens), cu(k_lens), table_tensor(tables)
    want = oattn.prefill(q, k_pool, v_pool, cq, ck, block_table=bt, window_left=window_left)
    status = ops.new_status(cuda)
    qd, kd, vd = q.to(cuda), k_pool.to(cuda), v_pool.to(cuda)
    out = ops.prefill_attn(qd, kd, vd, cq.to(cuda), ck.to(cuda), max(q_lens),
                           d ** -0.5, window_left, block_table=bt.to(cuda), status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert_close_attn(out, want, f"prefill paged q={q_lens[:4]}.. k={k_lens[:4]}.. d={d} w={window_left}")
    with_work_list(cuda, out, q_lens, k_lens, hq, hkv, d,
                   lambda items, st: ops.prefill_attn(qd, kd, vd, cq.to(cuda), ck.to(cuda), max(q_lens), d ** -0.5,
                                                      window_left, block_table=bt.to(cuda), status=st, items=items))


def test_single_short_sequence(cuda):
    run_dense(cuda, [37], 16, 8, 128)


def test_tile_boundary_lengths(cuda):
    run_dense(cuda, [1, 127, 128, 129, 255, 256, 257, 300], 16, 8, 128, seed=1)


def test_config1_prefill_packed_qkv(cuda):
    case, _ = config1()
    run_dense(cuda, case.prefill_lens, 16, 8, 128, seed=2, packed_qkv=True)


def test_long_sequence(cuda):
    run_dense(cuda, [2048, 700], 16, 8, 128, seed=3)


@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 2), (8, 1), (32, 8)])
def test_gqa_ratios(cuda, hq, hkv):
    run_dense(cuda, [200, 513], hq, hkv, 128, seed=hq + hkv)


def test_head_dim_256(cuda):
    run_dense(cuda, [64, 300, 129], 4, 1, 256, seed=4)


@pytest.mark.parametrize("window", [0, 64, 512])
def test_sliding_window(cuda, window):
    run_dense(cuda, [100, 700, 1300], 4, 1, 256, window_left=window, seed=5)
    run_dense(cuda, [100, 700], 16, 8, 128, window_left=window, seed=6)


def test_paged_full_prefill_matches_dense_semantics(cuda):
    run_paged(cuda, [244, 460, 485], [244, 460, 485], 16, 8, 128, seed=7)


def test_paged_prefix_cached_suffix_queries(cuda):
    """q_len < k_len: queries cover only the suffix, bottom-right aligned causal mask."""
    run_paged(cuda, [100, 1, 300, 257], [612, 513, 812, 257], 16, 8, 128, seed=8)


def test_paged_shared_prefix_blocks(cuda):
    """Two sequences share their first two blocks (same-step prefix sharing)."""
    g = generator(9)
    tables = [[5, 6, 1], [5, 6, 2, 3], [7]]
    k_lens, q_lens = [700, 1000, 90], [188, 488, 90]
    # build pools so that the shared blocks hold the same keys for both sequences
    k_pool, v_pool = fill_paged(g, [1000, 700 - 512, 90], [[5, 6, 2, 3], [1], [7]], 8, 8, 128)
    q = randn_bf16(g, sum(q_lens), 16, 128)
    cq, ck, bt = cu(q_lens), cu(k_lens), table_tensor(tables)
    want = oattn.prefill(q, k_pool, v_pool, cq, ck, block_table=bt)
    out = ops.prefill_attn(q.to(cuda), k_pool.to(cuda), v_pool.to(cuda), cq.to(cuda), ck.to(cuda), max(q_lens),
                           128 ** -0.5, -1, block_table=bt.to(cuda))
    torch.cuda.synchronize()
    assert_close_attn(out, want, "shared prefix")


def test_config3_prefill_part(cuda):
    case, g = config3()
    q_lens = [n - c for n, c in zip(case.prefill_lens, case.prefill_cached)]
    run_paged(cuda, q_lens, case.prefill_lens, 16, 8, 128, tables=case.prefill_blocks,
              num_blocks=case.pool_blocks, g=g)


def test_many_short_sequences_between_long_ones(cuda):
    """A prefill step as the scheduler packs it: a few long prompts among dozens of one-tile ones, each
    ending in a partial KV tile.  One CTA then works through many items back to back, and the producer
    fixes up the partial V tile of the next items while the current one is still being multiplied; run
    a few times because the interleaving is timing dependent."""
    g = generator(11)
    lens = [2440, 37, 54, 101, 2089, 33, 77, 130, 65, 1500] + [int(x) for x in torch.randint(32, 200, (40,), generator=g)]
    for rep in range(3):
        run_dense(cuda, lens, 16, 8, 128, seed=20 + rep, packed_qkv=True)
    k_lens = lens[:24]
    run_paged(cuda, k_lens, k_lens, 16, 8, 128, seed=30)


@pytest.mark.parametrize("boost", [6.0, 30.0])
def test_logits_that_jump_between_key_tiles(cuda, boost):
    """Keys whose logits are far larger in later tiles than in earlier ones (and the other way round): the running
    softmax reference has to move by much more than its lazy threshold from one key tile to the next, in the middle
    of a sequence, and the result must still be the oracle's."""
    g = generator(71)
    lens = [900, 400, 1300]
    T = sum(lens)
    q, k, v = randn_bf16(g, T, 16, 128), randn_bf16(g, T, 8, 128), randn_bf16(g, T, 8, 128)
    k = k.float()
    k[300:520] *= boost            # a loud stretch inside the first sequence (tiles 2-4), quiet again afterwards
    k[900 + 256:900 + 400] *= boost
    k[1300 + 1100:] *= boost       # the last tiles of the third sequence
    k = k.to(torch.bfloat16)
    cq = cu(lens)
    want = oattn.prefill(q, k, v, cq, cq)
    status = ops.new_status(cuda)
    out = ops.prefill_attn(q.to(cuda), k.to(cuda), v.to(cuda), cq.to(cuda), cq.to(cuda), max(lens), 128 ** -0.5, -1,
                           status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert_close_attn(out, want, f"logit jumps x{boost}")


def test_work_list_entries_outside_the_batch_are_skipped(cuda):
    """A list with entries that name no query block of the batch (a sequence or a block past the end) plus every real
    block: the real ones are computed, the others skipped, nothing is reported."""
    import numpy as np
    g = generator(5)
    lens = [300, 40, 700]
    q, k, v = randn_bf16(g, sum(lens), 16, 128), randn_bf16(g, sum(lens), 8, 128), randn_bf16(g, sum(lens), 8, 128)
    cq = cu(lens).to(cuda)
    qd, kd, vd = q.to(cuda), k.to(cuda), v.to(cuda)
    ref = ops.prefill_attn(qd, kd, vd, cq, cq, max(lens), 128 ** -0.5)
    items = ops.build_prefill_items(lens, lens, ops.prefill_item_rows(16, 8, 128))
    noisy = np.concatenate([np.array([[7, 0], [1, 5], [-1, 0], [0, -2]], np.int32), items]).astype(np.int32)
    status = ops.new_status(cuda)
    out = ops.prefill_attn(qd, kd, vd, cq, cq, max(lens), 128 ** -0.5, status=status, items=torch.from_numpy(noisy).to(cuda))
    torch.cuda.synchronize()
    ops.check_status(status)
    assert torch.equal(out, ref)
