"""``mvb_decode_attn_static``: decode attention for callers that cannot allocate a workspace.

Some embedders of the library have every byte of device memory assigned before serving starts, or sit
behind a binding that can only forward buffers it was handed; they cannot create the scratch buffer
the regular entry point wants.  This variant keeps its scratch in an array inside the library.  The
test calls it through the C ABI, twice in a row with different batches (the second call must not be
disturbed by what the first left in the shared array), and compares with the regular entry point.
It lives in a file that sorts last so a run that stops at the first failure has already covered
everything else; it passes on its own in a fresh process as well.
"""
import pytest
import torch

from mini_vllm_b200 import _cabi, ops
from mini_vllm_b200.workloads import generator, randn_bf16
from oracle import attention as oattn
from tests.helpers import assert_close_attn, fill_paged, sequential_tables, table_tensor

pytestmark = pytest.mark.gpu


def both_ways(cuda, lens, hq, hkv, d, window_left, seed, check_oracle=False):
    g = generator(seed)
    num_blocks = sum(max(1, -(-n // 256)) for n in lens) + 2
    tables = sequential_tables(g, lens, num_blocks)
    k_pool, v_pool = fill_paged(g, lens, tables, num_blocks, hkv, d)
    q = randn_bf16(g, len(lens), hq, d).to(cuda)
    seqlens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    bt = table_tensor(tables).to(cuda)
    k_pool, v_pool = k_pool.to(cuda), v_pool.to(cuda)

    ws = ops.decode_workspace(len(lens), hq, d, cuda)
    ops.decode_plan(seqlens, window_left, hq, hkv, d, ws)
    want = ops.decode_attn(q, k_pool, v_pool, seqlens, bt, d ** -0.5, window_left, ws)

    out = torch.full_like(want, float("nan"))
    status = ops.new_status(cuda)
    ops.decode_attn_static(q, k_pool, v_pool, seqlens, bt, d ** -0.5, window_left, out, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert_close_attn(out, want, "static-scratch decode vs workspace decode")
    if check_oracle:
        want32 = oattn.decode(q.cpu(), k_pool.cpu(), v_pool.cpu(), seqlens.cpu(), bt.cpu(), window_left=window_left,
                              out_dtype=torch.float32)
        assert_close_attn(out, want32, "static-scratch decode vs the fp32 oracle")


def test_two_calls_in_a_row_match_the_workspace_entry_point(cuda):
    both_ways(cuda, [300, 5, 1024, 2049, 77, 0, 640], 16, 8, 128, -1, seed=31)
    both_ways(cuda, [4000, 17], 16, 8, 128, -1, seed=32)          # fewer, longer rows: other plan, more partials
    both_ways(cuda, [100, 700, 1500], 4, 1, 256, 512, seed=33)    # another head shape and a window
    both_ways(cuda, [513, 64, 1300, 9], 16, 8, 128, -1, seed=34, check_oracle=True)


def test_bad_arguments_are_refused_before_anything_is_enqueued(cuda):
    """A call that is going to be rejected must not have put its plan kernel on the stream first: every
    operand is looked at before the first launch, so the status says so and the output stays untouched."""
    hq, hkv, d, rows = 16, 8, 128, 3
    q = torch.zeros(rows, hq, d, dtype=torch.bfloat16, device=cuda)
    pool = torch.zeros(2, 256, hkv, d, dtype=torch.bfloat16, device=cuda)
    seqlens = torch.full((rows,), 10, dtype=torch.int32, device=cuda)
    bt = torch.zeros(rows, 1, dtype=torch.int32, device=cuda)
    out = torch.full_like(q, 7.0)
    lib, stream = _cabi.load(), torch.cuda.current_stream().cuda_stream
    args = lambda qp, kp, op: (qp, q.stride(0), kp, pool.data_ptr(), 2, 256, seqlens.data_ptr(), bt.data_ptr(),
                               bt.stride(0), 1, rows, hq, hkv, d, 1.0, -1, op, out.stride(0), None, stream)
    assert lib.mvb_decode_attn_static(*args(None, pool.data_ptr(), out.data_ptr())) == -1          # NULL q
    assert lib.mvb_decode_attn_static(*args(q.data_ptr(), None, out.data_ptr())) == -1             # NULL K pool
    assert lib.mvb_decode_attn_static(*args(q.data_ptr(), pool.data_ptr(), out.data_ptr() + 2)) == -5   # misaligned out
    torch.cuda.synchronize()
    assert (out == 7.0).all()


def test_request_beyond_the_built_in_scratch_is_refused(cuda):
    hq, hkv, d, rows = 64, 8, 128, 4                              # partials of 64 heads x 128 exceed the 8 MiB array
    q = torch.zeros(rows, hq, d, dtype=torch.bfloat16, device=cuda)
    pool = torch.zeros(1, 256, hkv, d, dtype=torch.bfloat16, device=cuda)
    seqlens = torch.zeros(rows, dtype=torch.int32, device=cuda)
    bt = torch.zeros(rows, 1, dtype=torch.int32, device=cuda)
    with pytest.raises(_cabi.KernelError, match="built-in"):
        ops.decode_attn_static(q, pool, pool, seqlens, bt, 1.0, -1, torch.empty_like(q))
