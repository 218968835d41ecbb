"""Paged decode attention (CUDA, through the C ABI) against the fp32 gather-and-SDPA oracle."""
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import BLOCK_SIZE, cdiv, config1, config3, config4, generator, randn_bf16
from oracle import attention as oattn
from tests.helpers import assert_close_attn, fill_paged, sequential_tables, table_tensor

pytestmark = pytest.mark.gpu


def run_case(cuda, lens, hq, hkv, d, window_left=-1, seed=0, table_width=None, pad_rows=0, num_blocks=None,
             tables=None, g=None):
    g = g or generator(seed)
    num_blocks = num_blocks or sum(max(1, cdiv(n, BLOCK_SIZE)) for n in lens) + 3
    tables = tables or sequential_tables(g, lens, num_blocks)
    k_pool, v_pool = fill_paged(g, lens, tables, num_blocks, hkv, d)
    B = len(lens) + pad_rows
    q = randn_bf16(g, B, hq, d)
    seqlens = torch.tensor(list(lens) + [0] * pad_rows, dtype=torch.int32)
    bt = table_tensor(tables + [[]] * pad_rows if pad_rows else tables, width=table_width)
    want = oattn.decode(q, k_pool, v_pool, seqlens, bt, window_left=window_left)

    status = ops.new_status(cuda)
    ws = ops.decode_workspace(B, hq, d, cuda)
    seqlens_d, bt_d = seqlens.to(cuda), bt.to(cuda)
    ops.decode_plan(seqlens_d, window_left, hq, hkv, d, ws, block_table=bt_d, block_size=256)
    out = torch.full((B, hq, d), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.decode_attn(q.to(cuda), k_pool.to(cuda), v_pool.to(cuda), seqlens_d, bt_d, d ** -0.5, window_left, ws,
                    out=out, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert_close_attn(out, want, f"decode hq={hq} hkv={hkv} d={d} window={window_left}")
    if pad_rows:
        assert (out[len(lens):] == 0).all()
    return out


def test_config1_shapes(cuda):
    case, g = config1()
    run_case(cuda, [n + 1 for n in case.prefill_lens], 16, 8, 128, tables=case.prefill_blocks, num_blocks=64, g=g)


def test_block_boundary_lengths(cuda):
    run_case(cuda, [1, 2, 15, 16, 17, 31, 32, 33, 255, 256, 257, 511, 512, 513, 1000], 16, 8, 128)


def test_padding_rows_and_wide_table(cuda):
    run_case(cuda, [300, 7, 1024], 16, 8, 128, table_width=40, pad_rows=5)


def test_one_long_many_short(cuda):
    run_case(cuda, [9000] + [3] * 20 + [700], 16, 8, 128)


@pytest.mark.parametrize("hq,hkv,d", [(4, 1, 256), (8, 2, 128), (4, 4, 128), (32, 8, 128), (8, 1, 128),
                                       (16, 16, 128), (8, 2, 256), (16, 4, 256), (8, 8, 256)])
def test_head_shapes(cuda, hq, hkv, d):
    run_case(cuda, [5, 129, 640, 2049, 77], hq, hkv, d, seed=hq * 100 + hkv)


@pytest.mark.parametrize("window", [0, 1, 15, 16, 511, 512, 4096])
def test_sliding_window_gemma_shapes(cuda, window):
    run_case(cuda, [1, 100, 512, 513, 514, 1500, 3000], 4, 1, 256, window_left=window, seed=window)


def test_sliding_window_qwen_shapes(cuda):
    run_case(cuda, [40, 700, 1300], 16, 8, 128, window_left=200)


def test_config3_decode_part(cuda):
    case, g = config3()
    run_case(cuda, case.decode_ctx, 16, 8, 128, tables=case.decode_blocks, num_blocks=case.pool_blocks, g=g)


def test_config4_global_and_window(cuda):
    case, g = config4()
    run_case(cuda, case.decode_ctx, 4, 1, 256, tables=case.decode_blocks, num_blocks=case.pool_blocks, g=g)
    run_case(cuda, case.decode_ctx, 4, 1, 256, window_left=512, tables=case.decode_blocks,
             num_blocks=case.pool_blocks, g=generator(1))


def test_graph_capture_and_replay(cuda):
    """The plan + attention launch sequence is capturable; a replay with new lengths gives new results."""
    g = generator(7)
    hq, hkv, d, B = 16, 8, 128, 8
    lens_a, lens_b = [100, 300, 50, 0, 0, 0, 0, 0], [101, 301, 51, 800, 0, 0, 0, 0]
    num_blocks = 24
    tables = [[0, 1], [2, 3], [4], [5, 6, 7, 8], [], [], [], []]
    k_pool, v_pool = fill_paged(g, [512, 512, 256, 1024], tables[:4], num_blocks, hkv, d)
    q = randn_bf16(g, B, hq, d)
    q_d, k_d, v_d = q.to(cuda), k_pool.to(cuda), v_pool.to(cuda)
    seqlens = torch.zeros(B, dtype=torch.int32, device=cuda)
    bt = torch.full((B, num_blocks), -1, dtype=torch.int32, device=cuda)
    bt[:, :4] = table_tensor(tables, width=4).to(cuda)
    ws = ops.decode_workspace(B, hq, d, cuda)
    out = torch.zeros(B, hq, d, dtype=torch.bfloat16, device=cuda)

    def step():
        ops.decode_plan(seqlens, -1, hq, hkv, d, ws, block_table=bt, block_size=256)
        ops.decode_attn(q_d, k_d, v_d, seqlens, bt, d ** -0.5, -1, ws, out=out)

    seqlens.copy_(torch.tensor(lens_a, dtype=torch.int32))
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for lens in (lens_a, lens_b):
        seqlens.copy_(torch.tensor(lens, dtype=torch.int32))
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        want = oattn.decode(q, k_pool, v_pool, torch.tensor(lens, dtype=torch.int32), bt.cpu())
        assert_close_attn(out, want, "graph replay")


def test_bad_block_id_is_reported_not_fatal(cuda):
    g = generator(3)
    hq, hkv, d = 16, 8, 128
    k_pool, v_pool = fill_paged(g, [300], [[1, 2]], 4, hkv, d)
    q = randn_bf16(g, 1, hq, d).to(cuda)
    seqlens = torch.tensor([300], dtype=torch.int32, device=cuda)
    bt = torch.tensor([[1, 99]], dtype=torch.int32, device=cuda)      # 99 is outside the 4-block pool
    status = ops.new_status(cuda)
    ws = ops.decode_workspace(1, hq, d, cuda)
    ops.decode_plan(seqlens, -1, hq, hkv, d, ws, block_table=bt, block_size=256)
    ops.decode_attn(q, k_pool.to(cuda), v_pool.to(cuda), seqlens, bt, d ** -0.5, -1, ws, status=status)
    torch.cuda.synchronize()
    assert status[0].item() == 2


def plan_header(ws: torch.Tensor) -> dict:
    names = ["total_tiles", "per_cta", "num_ctas", "cta_tokens", "num_seqs", "window_left", "aligned"]
    return dict(zip(names, ws[:28].view(torch.int32).tolist()))


def planned(cuda, lens, hq, hkv, d, window_left):
    ws = ops.decode_workspace(len(lens), hq, d, cuda)
    ops.decode_plan(torch.tensor(lens, dtype=torch.int32, device=cuda), window_left, hq, hkv, d, ws)
    torch.cuda.synchronize()
    return plan_header(ws)


def test_plan_keeps_short_sequences_whole(cuda):
    """Many short contexts: every CTA boundary sits on a sequence boundary (nothing to merge).  A few long
    contexts: the even cut, with sequences split across CTAs.  Both give the oracle's result."""
    g = generator(41)
    short = [int(x) for x in torch.randint(290, 311, (140,), generator=g)]     # 19-20 tiles each, 19 per CTA if cut evenly
    hdr = planned(cuda, short, 16, 8, 128, -1)
    assert hdr["aligned"] == 1 and hdr["num_seqs"] == 140 and hdr["cta_tokens"] == 16
    run_case(cuda, short, 16, 8, 128, seed=42)
    windowed = [int(x) for x in torch.randint(512, 4096, (128,), generator=g)]
    assert planned(cuda, windowed, 4, 1, 256, 512)["aligned"] == 1        # a sliding-window layer of config 4
    assert planned(cuda, windowed, 4, 1, 256, -1)["aligned"] == 0         # its global layer
    run_case(cuda, windowed, 4, 1, 256, window_left=512, seed=43)
    assert planned(cuda, [9000, 40, 2000], 16, 8, 128, -1)["aligned"] == 0
    assert planned(cuda, [0, 0, 0], 16, 8, 128, -1)["total_tiles"] == 0
    # sequences of zero length between the others do not upset the boundaries
    run_case(cuda, [300, 0, 0, 280, 310, 0, 295] * 12, 16, 8, 128, seed=44)
