"""Decoder glue kernels (activation*up, residual add + RMSNorm) against the unfused PyTorch sequence."""
import pytest
import torch
import torch.nn.functional as F

from mini_vllm_b200 import ops
from mini_vllm_b200.workloads import generator, randn_bf16

pytestmark = pytest.mark.gpu


def close(got, want, what):
    got, want = got.float().cpu(), want.float().cpu()
    rel = ((got - want).abs() / want.abs().clamp_min(1.0)).max().item()
    same = (got == want).float().mean().item()
    assert rel <= 2 ** -6 and same >= 0.98, f"{what}: max rel {rel:.4g}, {same:.4f} bit-equal"


@pytest.mark.parametrize("rows,inter,gelu", [(64, 3072, False), (5, 6912, True), (1000, 512, False)])
def test_act_mul(cuda, rows, inter, gelu):
    g = generator(rows + inter)
    full = randn_bf16(g, rows, 2 * inter + 8) * 2
    gate_up = full[:, :2 * inter]                     # row stride larger than the width
    gate, up = gate_up.split([inter, inter], dim=-1)
    want = (F.gelu(gate, approximate="tanh") if gelu else F.silu(gate)) * up
    got = ops.act_mul(full.to(cuda)[:, :2 * inter], inter, gelu)
    close(got, want, "act_mul")


def rms(v, w, eps, unit_offset):
    if not unit_offset:
        return F.rms_norm(v, (v.shape[-1],), w, eps)
    vf = v.float()
    vf = vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + eps)
    return (vf * (1.0 + w.float())).type_as(v)


@pytest.mark.parametrize("rows,hidden,unit_offset,branch_norm", [(64, 1024, False, False), (7, 1152, True, True),
                                                                 (300, 4096, False, False), (3, 256, True, True)])
def test_add_rmsnorm(cuda, rows, hidden, unit_offset, branch_norm):
    g = generator(hidden + rows)
    x, y = randn_bf16(g, rows, hidden) * 3, randn_bf16(g, rows, hidden)
    w = randn_bf16(g, hidden) * 0.3 + (0 if unit_offset else 1)
    yw = randn_bf16(g, hidden) * 0.3 if branch_norm else None
    y2 = rms(y, yw, 1e-6, unit_offset) if branch_norm else y
    x_want = x + y2
    out_want = rms(x_want, w, 1e-6, unit_offset)
    xd = x.to(cuda)
    out = ops.add_rmsnorm(xd, y.to(cuda), w.to(cuda), 1e-6, unit_offset, y_weight=None if yw is None else yw.to(cuda))
    torch.cuda.synchronize()
    close(xd, x_want, "residual")
    close(out, out_want, "norm")


@pytest.mark.parametrize("hidden,unit_offset,branch_norm", [(1024, False, False), (1152, True, True)])
def test_add_rmsnorm_last_tokens_is_the_gathered_full_result(cuda, hidden, unit_offset, branch_norm):
    """The last-token variant equals running the full kernel over every row and indexing cu_seqlens_q[1:] - 1
    afterwards (what the reference does, qwen3.py:215-217), bit for bit, and leaves the residual stream alone."""
    g = generator(hidden)
    lens = [5, 1, 300, 64, 17]
    T = sum(lens)
    x, y = (randn_bf16(g, T, hidden) * 3).to(cuda), randn_bf16(g, T, hidden).to(cuda)
    w = (randn_bf16(g, hidden) * 0.3 + (0 if unit_offset else 1)).to(cuda)
    yw = (randn_bf16(g, hidden) * 0.3).to(cuda) if branch_norm else None
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=cuda)
    x_before = x.clone()
    got = ops.add_rmsnorm_last_tokens(x, y, w, 1e-6, unit_offset, cu, y_weight=yw)
    assert torch.equal(x, x_before)
    full = ops.add_rmsnorm(x.clone(), y, w, 1e-6, unit_offset, y_weight=yw)
    want = full[(cu[1:] - 1).long()]
    assert got.shape == (len(lens), hidden)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
