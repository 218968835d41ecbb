"""The shared library loads on a machine without a GPU and exports every function the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

from mini_vllm_b200 import _cabi

HEADER = Path(__file__).resolve().parent.parent / "include" / "mini_vllm_b200.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mvb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("mvb_pack_prefill", "mvb_pack_decode", "mvb_rope_kv_write", "mvb_decode_plan", "mvb_decode_attn",
                 "mvb_decode_attn_static", "mvb_prefill_attn", "mvb_sample", "mvb_decode_workspace_bytes"):
        assert must in names


def test_library_exports_every_declared_symbol_and_binding_covers_them():
    lib = _cabi.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _cabi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == set(declared_functions())


def test_host_only_calls_work_without_a_gpu():
    lib = _cabi.load()
    assert lib.mvb_abi_version() >= 6
    assert lib.mvb_status_string(0) == b"ok"
    assert b"scratch" in lib.mvb_status_string(-7)
    assert lib.mvb_decode_workspace_bytes(512, 16, 128) > 2 * 160 * 16 * 128 * 4
    assert lib.mvb_decode_workspace_bytes(0, 16, 128) == 0
    # argument errors are caught on the host before anything is launched
    assert lib.mvb_rope_kv_write(None, 0, None, 0, None, 0, None, None, 0, None, None, None, 0, 4, 2, 2, 100, 0,
                                 None, None) == -2          # head_dim not a multiple of 16
    assert lib.mvb_sample(None, 0, 1, 10, None, None, None, 0, 0, None, None, None, None, None) == -1
    assert lib.mvb_decode_plan(None, 1, -1, 16, 8, 128, None, 0, None) == -1
    assert lib.mvb_selftest_wait_timeout(None, 16, None) == -1
    # query-block size of the prefill kernel's work items: a property of the head layout
    assert lib.mvb_prefill_item_rows(16, 8, 128) == 128 and lib.mvb_prefill_item_rows(8, 8, 128) == 256
    assert lib.mvb_prefill_item_rows(4, 1, 256) == 128 and lib.mvb_prefill_item_rows(16, 8, 96) == -2
    assert lib.mvb_prefill_attn_items(None, 0, None, 0, None, 0, 1, None, None, None, 0, 0, 1, 1, 1, 16, 8, 128, 1.0, -1,
                                      None, 0, None, 0, None, None) == -1          # no list
    # the scratch-free decode entry looks at every operand before its first launch
    assert lib.mvb_decode_attn_static(None, 0, None, None, 1, 256, None, None, 1, 1, 1, 16, 8, 128, 1.0, -1, None, 0,
                                      None, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_cabi.KernelError, match="no CPU or PyTorch fallback"):
        _cabi.load()


def test_ops_reject_cpu_tensors():
    import torch
    from mini_vllm_b200 import ops
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.sample(torch.zeros(2, 16, dtype=torch.bfloat16))


def test_prefill_work_list_builder():
    """Every query block of every sequence once, the blocks that see the most keys first (host arithmetic only)."""
    import numpy as np
    from mini_vllm_b200 import ops
    q_lens, k_lens = [300, 128, 1, 0, 129], [812, 128, 5000, 40, 129]
    items = ops.build_prefill_items(q_lens, k_lens, 128)
    assert items.dtype == np.int32 and items.shape == (7, 2)
    assert sorted(map(tuple, items.tolist())) == [(0, 0), (0, 1), (0, 2), (1, 0), (2, 0), (4, 0), (4, 1)]
    visible = [k_lens[s] - q_lens[s] + min((b + 1) * 128, q_lens[s]) for s, b in items.tolist()]
    assert visible == sorted(visible, reverse=True) and visible[0] == 5000
    assert ops.build_prefill_items([], [], 128).shape == (0, 2)
    assert ops.build_prefill_items([300], [300], 256).tolist() == [[0, 1], [0, 0]]
