"""Fused lm_head + greedy argmax (tcgen05 GEMM with an argmax epilogue) against lm_head followed by the sampler."""
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import generator, randn_bf16

pytestmark = pytest.mark.gpu


def fused(cuda, x, w, **kw):
    scratch = ops.lm_head_argmax_scratch(x.shape[0], cuda)
    status = ops.new_status(cuda)
    out = ops.lm_head_argmax(x, w, scratch, status=status, **kw)
    torch.cuda.synchronize()
    ops.check_status(status)
    assert int(scratch.sum()) == 0, "the scratch must be left zeroed for the next call"
    return out, scratch


@pytest.mark.parametrize("rows,hidden,vocab", [(1, 64, 8), (5, 128, 1003), (64, 1024, 151936), (130, 1024, 4096),
                                               (512, 1024, 151936), (300, 1152, 262144)])
def test_exact_arithmetic_matches_argmax_of_the_logits(cuda, rows, hidden, vocab):
    """Small integers: every product and partial sum is exact in fp32 whatever the order, so the fused kernel and
    lm_head + sampler see the same logits bit for bit - and many exact ties, where the lowest column must win."""
    g = generator(rows + vocab)
    x = torch.randint(-2, 3, (rows, hidden), generator=g).to(torch.bfloat16).to(cuda)
    w = torch.randint(-2, 3, (vocab, hidden), generator=g).to(torch.bfloat16).to(cuda)
    logits = torch.nn.functional.linear(x, w)                  # exact integer sums, rounded to bf16 once
    want = ops.sample(logits)                                  # the unfused path: bf16 logits, first argmax
    got, _ = fused(cuda, x, w)
    assert torch.equal(got, want)
    assert torch.equal(got.cpu(), logits.float().cpu().argmax(-1))


@pytest.mark.parametrize("rows", [3, 64, 512])
def test_random_weights_agree_with_the_unfused_path_up_to_rounding_ties(cuda, rows):
    """N(0, 0.02) weights and unit-RMS activations, the model's own statistics.  The accumulation order differs from
    cuBLAS, so a logit may land on the neighbouring bf16 value: the chosen column's unfused logit must be within one
    bf16 step of the unfused maximum, and equal the unfused argmax wherever the unfused top two are further apart."""
    g = generator(900 + rows)
    hidden, vocab = 1024, 151936
    x = randn_bf16(g, rows, hidden).to(cuda)
    w = (torch.randn(vocab, hidden, generator=g) * 0.02).to(torch.bfloat16).to(cuda)
    logits = torch.nn.functional.linear(x, w).float()
    top2 = logits.topk(2, dim=-1)
    got, scratch = fused(cuda, x, w)
    chosen = logits[torch.arange(rows, device=cuda), got]
    ulp = torch.exp2(torch.floor(torch.log2(top2.values[:, 0].abs())) - 7)
    assert ((top2.values[:, 0] - chosen) <= ulp + 1e-9).all()
    clear = (top2.values[:, 0] - top2.values[:, 1]) > ulp
    assert clear.float().mean().item() > 0.8
    assert torch.equal(got[clear], top2.indices[clear, 0])
    # a second call on the same scratch, with the ids scattered into a table as the engine does
    table = torch.full((rows + 7,), -1, dtype=torch.int64, device=cuda)
    index = torch.randperm(rows + 7, generator=g)[:rows].to(torch.int32).to(cuda)
    again = ops.lm_head_argmax(x, w, scratch, scatter_table=table, scatter_index=index)
    torch.cuda.synchronize()
    assert torch.equal(again, got) and torch.equal(table[index.long()], got)


def test_strided_rows_and_argument_checks(cuda):
    g = generator(5)
    big = randn_bf16(g, 40, 2 * 256).to(cuda)
    x = big[:, :256]                                           # row stride twice the width
    w = (torch.randn(3000, 256, generator=g) * 0.05).to(torch.bfloat16).to(cuda)
    got, scratch = fused(cuda, x, w)
    logits = torch.nn.functional.linear(x.contiguous(), w).float()
    chosen = logits[torch.arange(40, device=cuda), got]
    assert ((logits.max(-1).values - chosen) <= 2 ** -5).all()
    from mini_vllm_b200 import _cabi
    with pytest.raises(_cabi.KernelError, match="unsupported shape"):
        ops.lm_head_argmax(big[:, :100].contiguous(), w[:, :100].contiguous(), scratch)     # hidden not a multiple of 64
    with pytest.raises(_cabi.KernelError, match="invalid argument"):
        ops.lm_head_argmax(x, w, scratch[:8])                                               # scratch too small
