"""The device status word: a bounded wait that runs out is reported, not hung on."""
import pytest
import torch

from mini_vllm_b200 import _cabi, ops

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_timeout_and_the_stream_carries_on(cuda):
    """Every mbarrier wait in the attention kernels has an iteration limit.  Here the same wait is run on a
    barrier nothing arrives at, with a small limit: the kernel must come back on its own, the status word
    must say "wait timeout" with the limit as detail, and later work on the stream must be unaffected."""
    status = ops.new_status(cuda)
    ops.selftest_wait_timeout(status, limit=1024)
    after = torch.arange(8, device=cuda) * 2                 # queued behind the self-test on the same stream
    torch.cuda.synchronize()
    assert status.tolist() == [4, 1024, 0, 0]
    assert after.tolist() == list(range(0, 16, 2))
    with pytest.raises(_cabi.KernelError, match="bounded device wait ran out"):
        ops.check_status(status)
    # first error wins: a second timeout does not overwrite the record
    ops.selftest_wait_timeout(status, limit=16)
    torch.cuda.synchronize()
    assert status.tolist() == [4, 1024, 0, 0]
    # a real kernel launched afterwards still works and leaves a fresh status word clean
    clean = ops.new_status(cuda)
    logits = torch.randn(4, 1000, device=cuda).to(torch.bfloat16)
    assert torch.equal(ops.sample(logits), logits.float().argmax(-1))
    torch.cuda.synchronize()
    ops.check_status(clean)
