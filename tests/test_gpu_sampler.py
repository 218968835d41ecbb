"""Sampler kernel (CUDA) against torch.argmax (greedy, bit-exact) and the Philox/Gumbel oracle."""
import pytest
import torch

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import generator, randn_bf16
from oracle import sampler as osamp

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,V", [(1, 151936), (64, 151936), (7, 262144), (5, 1000), (3, 1003)])
def test_greedy_is_first_argmax(cuda, B, V):
    g = generator(B + V)
    logits = randn_bf16(g, B, V) * 4
    logits[0, 17] = logits[0].max()          # force ties: the lowest index must win
    logits[0, 5] = logits[0].max()
    out = ops.sample(logits.to(cuda))
    assert out.dtype == torch.int64
    assert torch.equal(out.cpu(), osamp.greedy(logits))


@pytest.mark.parametrize("B", [1, 3, 40, 200, 400])
def test_greedy_special_values_and_batch_sizes(cuda, B):
    """The row is split over 1, 2, 4 or 8 CTAs depending on the batch; ties across words of one load,
    across threads and across slices, signed zeros, -inf rows and NaNs follow torch.argmax."""
    V = 151936
    g = generator(100 + B)
    logits = randn_bf16(g, B, V)
    top = logits.max().item() + 1.0
    logits[0, V - 1] = top; logits[0, V // 2 + 3] = top; logits[0, 4097] = top      # same value in three slices
    if B > 1:
        logits[1] = float("-inf")                                                  # nothing is larger than the start value
    if B > 2:
        logits[2] = -1.0
        logits[2, 9] = -0.0; logits[2, 8] = 0.0; logits[2, 123456] = 0.0             # +0 == -0: the lowest index wins
    if B > 3:
        logits[3, 77777] = float("nan"); logits[3, 99] = top                       # NaN counts as the largest
        logits[4, 5] = float("-inf"); logits[4, 6] = float("inf"); logits[4, 70000] = float("inf")
    want = osamp.greedy(logits)
    if B > 3:
        assert want[3] == 77777
    out = ops.sample(logits.to(cuda)).cpu()
    assert torch.equal(out, want)


def test_greedy_unaligned_rows(cuda):
    """Rows that do not start on 16 bytes take the scalar path."""
    g = generator(6)
    full = randn_bf16(g, 9, 5000 + 3)
    out = ops.sample(full.to(cuda)[:, 3:])
    assert torch.equal(out.cpu(), osamp.greedy(full[:, 3:]))


def test_greedy_with_temperature_and_row_stride(cuda):
    g = generator(5)
    full = randn_bf16(g, 6, 4096 + 8)
    logits = full[:, 8:]                      # rows start 16 bytes in, stride != vocab
    temps = torch.tensor([0.5, 1.0, 2.0, 0.1, 3.3, 0.7])
    out = ops.sample(full.to(cuda)[:, 8:], temperatures=temps.to(cuda))
    assert torch.equal(out.cpu(), osamp.greedy(logits, temps))


@pytest.mark.parametrize("V", [1000, 1003, 151936])     # 1003: odd width, most rows not 16-byte aligned
def test_topk_gumbel_matches_oracle(cuda, V):
    g = generator(9)
    B = 12
    logits = randn_bf16(g, B, V) * 3
    temps = torch.tensor([0.7, 1.0, 1.3] * 4)
    top_k = torch.tensor([1, 2, 5, 50, 0, 1000, 3, 8, 1, 40, V, 7], dtype=torch.int32)
    seed, offset = 1234567890123, 42
    out = ops.sample(logits.to(cuda), temps.to(cuda), top_k.to(cuda), seed, offset).cpu()
    scores = osamp.gumbel_scores(logits, temps, top_k, seed, offset)
    best = scores.max(dim=-1).values
    picked = scores[torch.arange(B), out]
    # device logf may differ from the host's in the last ulp: the pick must be (one of) the best
    assert torch.isfinite(picked).all(), "picked a token outside the top-k set"
    assert (best - picked).abs().max().item() <= 1e-4
    assert (out == scores.argmax(-1)).float().mean().item() >= 0.9
    # top_k = 1 rows are greedy whatever the noise
    greedy = osamp.greedy(logits)
    assert out[0] == greedy[0] and out[8] == greedy[8]
    # a different offset gives a different stream somewhere
    out2 = ops.sample(logits.to(cuda), temps.to(cuda), top_k.to(cuda), seed, offset + 1).cpu()
    assert not torch.equal(out, out2)


def test_topk_frequencies_follow_softmax(cuda):
    """Gumbel-max draws follow softmax(logits / T) restricted to the top-k set."""
    V, k, n = 64, 4, 4000
    g = generator(21)
    row = randn_bf16(g, 1, V)
    logits = row.expand(n, V).contiguous()
    temps = torch.full((n,), 0.8)
    out = ops.sample(logits.to(cuda), temps.to(cuda), torch.full((n,), k, dtype=torch.int32).to(cuda), 77, 0).cpu()
    top = torch.topk(row[0].float(), k)
    probs = torch.softmax(top.values / 0.8, -1)
    counts = torch.stack([(out == i).sum() for i in top.indices]).float() / n
    assert counts.sum().item() == pytest.approx(1.0)
    assert (counts - probs).abs().max().item() < 0.04


def test_top_p_nucleus_matches_oracle(cuda):
    g = generator(33)
    B, V = 16, 32000
    logits = randn_bf16(g, B, V) * 4
    temps = torch.tensor([0.6, 1.0, 1.4, 0.9] * 4)
    top_k = torch.tensor([0, 0, 50, 0, 1000, 0, 0, 5] * 2, dtype=torch.int32)
    top_p = torch.tensor([0.5, 0.9, 0.8, 1.0, 0.3, 0.05, 0.99, 0.7] * 2)
    seed, offset = 99, 7
    out = ops.sample(logits.to(cuda), temps.to(cuda), top_k.to(cuda), seed, offset, top_p=top_p.to(cuda)).cpu()
    scores = osamp.gumbel_scores(logits, temps, top_k, seed, offset, top_p=top_p)
    picked = scores[torch.arange(B), out]
    best = scores.max(dim=-1).values
    # the nucleus boundary is decided by float sums in a different order than the oracle's float64:
    # a row may differ by the boundary token, so most rows must agree exactly and every pick must be kept
    ok = torch.isfinite(picked) & ((best - picked).abs() <= 1e-4)
    assert ok.float().mean().item() >= 0.85, (picked, best)
    # tiny nucleus (top_p 0.05 on a peaked row) is the argmax more often than not; top_p=1 row equals plain top-k
    plain = ops.sample(logits.to(cuda), temps.to(cuda), top_k.to(cuda), seed, offset).cpu()
    assert out[3] == plain[3] and out[11] == plain[11]


def test_top_p_without_top_k_tensor(cuda):
    g = generator(34)
    logits = randn_bf16(g, 4, 5000) * 5
    top_p = torch.tensor([1e-6, 1e-6, 1e-6, 1e-6])              # nucleus = the single most likely token
    out = ops.sample(logits.to(cuda), None, None, 5, 0, top_p=top_p.to(cuda)).cpu()
    assert torch.equal(out, osamp.greedy(logits))


def check_against_oracle(cuda, logits, temps, top_k, top_p, seed, offset, min_exact=0.9):
    B = logits.shape[0]
    out = ops.sample(logits.to(cuda), None if temps is None else temps.to(cuda), None if top_k is None else top_k.to(cuda),
                     seed, offset, top_p=None if top_p is None else top_p.to(cuda)).cpu()
    scores = osamp.gumbel_scores(logits, temps, top_k, seed, offset, top_p=top_p)
    picked = scores[torch.arange(B), out]
    best = scores.max(dim=-1).values
    ok = torch.isfinite(picked) & ((best - picked).abs() <= 1e-4)
    assert ok.float().mean().item() >= min_exact, (out, scores.argmax(-1))
    return out, scores


@pytest.mark.parametrize("B", [1, 3, 40, 200, 400])
def test_topk_rows_split_over_clusters_of_every_size(cuda, B):
    """A row is split over 8, 4, 2 or 1 CTAs depending on the batch; the candidates of all slices meet in the first
    CTA.  Winners in the first, a middle and the last slice, and rows whose k-th value ties with many others."""
    V = 151936
    g = generator(300 + B)
    logits = randn_bf16(g, B, V) * 2
    top_k = torch.full((B,), 50, dtype=torch.int32)
    top = logits.max().item()
    logits[0, 3] = top + 1.0; logits[0, V // 2 + 11] = top + 1.0; logits[0, V - 1] = top + 1.0   # one value in three slices
    top_k[0] = 2                                               # the k-th value is tied: all three stay in
    if B > 2:
        logits[1, :] = -3.0
        logits[1, 100:180] = 1.5                               # 80 equal candidates for k = 50: every one of them is kept
        logits[2, V - 7:] = top + 2.0
        top_k[2] = 7
    temps = torch.full((B,), 0.9)
    out, scores = check_against_oracle(cuda, logits, temps, top_k, None, 4242, 3, min_exact=0.95)
    assert out[0] in (3, V // 2 + 11, V - 1)
    if B > 2:
        assert 100 <= out[1] < 180 and out[2] >= V - 7


def test_topk_rows_that_leave_the_window(cuda):
    """Rows the short-list way cannot handle fall back to radix selection over the whole row: a maximum so far
    above the rest that fewer than k entries lie within one binade of it, k larger than the list can hold, a NaN
    in the row, a row of one repeated value, top-k off (k = 0) with and without a nucleus."""
    V = 151936
    g = generator(77)
    logits = randn_bf16(g, 8, V)
    logits[0, 1234] = 60.0                                     # nothing else within one binade
    logits[2, 999] = float("nan")
    logits[3, :] = 0.25
    top_k = torch.tensor([40, 6000, 30, 10, 0, 0, 50, 50], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.6, 1.0, 0.3, 1e-6])
    temps = torch.tensor([1.0, 0.8, 1.0, 1.0, 0.7, 1.2, 1.0, 1.0])
    out = ops.sample(logits.to(cuda), temps.to(cuda), top_k.to(cuda), 5, 9, top_p=top_p.to(cuda)).cpu()
    keep = [0, 1, 3, 4, 5, 6, 7]                               # (the oracle's topk has no defined order for a NaN row)
    full = osamp.gumbel_scores(torch.nan_to_num(logits, nan=0.0), temps, top_k, 5, 9, top_p=top_p)
    for r in keep:
        assert torch.isfinite(full[r, out[r]]), f"row {r}: token {out[r]} is outside the kept set"
        assert (full[r].max() - full[r, out[r]]).abs().item() <= 1e-4, f"row {r}"
    assert out[7] == logits[7].float().argmax()                # a nucleus of one token
    assert 0 <= out[2] < V
