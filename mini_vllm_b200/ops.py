"""Tensor-level wrappers over the C ABI: pointers, strides and the current CUDA stream.

Each function validates shapes/dtypes, passes raw device pointers to the library and
raises on a non-zero status.  Nothing here computes on the host.
"""
from __future__ import annotations

import torch

from . import _cabi

_DEV_ERRORS = {1: "slot outside the KV pool", 2: "block id outside the KV pool",
               3: "position outside the cos/sin table", 4: "a bounded device wait ran out",
               5: "sequence length does not fit its block list"}


class LaunchCounter:
    """Counts kernels of this library enqueued through the wrappers below (graph replays add theirs)."""
    total = 0

    @classmethod
    def add(cls, n: int) -> None:
        cls.total += n


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (the kernels have no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")


def _heads_contiguous(t: torch.Tensor, name: str) -> None:
    if t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
        raise ValueError(f"{name} must be [tokens, heads, head_dim] with contiguous heads")


def new_status(device) -> torch.Tensor:
    """A zeroed device int32[4] for kernels to record device-detected errors in."""
    return torch.zeros(4, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    """Synchronising read of a status word; raises if a kernel recorded an error."""
    code, detail, block, thread = status.tolist()
    if code:
        raise _cabi.KernelError(f"device error {code} ({_DEV_ERRORS.get(code, '?')}), detail {detail}, "
                                f"block {block}, thread {thread}")


def selftest_wait_timeout(status: torch.Tensor, limit: int = 1024) -> None:
    """Run the kernels' bounded mbarrier wait on a barrier nobody arrives at; ``status`` then reads
    ``[4, limit, 0, 0]`` (a wait timeout), and the stream carries on."""
    _need(status, torch.int32, "status")
    _cabi.check(_cabi.load().mvb_selftest_wait_timeout(_ptr(status), int(limit), _stream()), "mvb_selftest_wait_timeout")
    LaunchCounter.add(1)


def pack_prefill(meta: torch.Tensor, num_seqs: int, num_tokens: int, num_blocks_total: int, table_width: int,
                 block_size: int, want_table: bool, status: torch.Tensor | None = None) -> dict:
    """meta: device int32 = [seq_len(B) | cached_len(B) | blk_off(B+1) | blocks_flat | new_tokens(T)]."""
    _need(meta, torch.int32, "meta")
    dev = meta.device
    B, T = num_seqs, num_tokens
    base, es = meta.data_ptr(), 4
    o_seq, o_cached, o_off = 0, B, 2 * B
    o_blocks = o_off + B + 1
    o_tok = o_blocks + num_blocks_total
    assert meta.numel() >= o_tok + T
    out = {
        "input_ids": torch.empty(T, dtype=torch.int64, device=dev),
        "positions": torch.empty(T, dtype=torch.int64, device=dev),
        "slot_mapping": torch.empty(T, dtype=torch.int32, device=dev),
        "cu_seqlens_q": torch.empty(B + 1, dtype=torch.int32, device=dev),
        "cu_seqlens_k": torch.empty(B + 1, dtype=torch.int32, device=dev),
        "block_table": torch.empty(B, table_width, dtype=torch.int32, device=dev) if want_table else None,
    }
    rc = _cabi.load().mvb_pack_prefill(
        base + es * o_seq, base + es * o_cached, base + es * o_off, base + es * o_blocks, base + es * o_tok,
        B, T, table_width, block_size, _ptr(out["input_ids"]), _ptr(out["positions"]), _ptr(out["slot_mapping"]),
        _ptr(out["cu_seqlens_q"]), _ptr(out["cu_seqlens_k"]), _ptr(out["block_table"]), _ptr(status), _stream())
    _cabi.check(rc, "mvb_pack_prefill")
    LaunchCounter.add(1)
    return out


def pack_decode(meta: torch.Tensor, num_seqs: int, num_blocks_total: int, table_width: int, block_size: int,
                input_ids: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor,
                cache_seqlens: torch.Tensor, block_table: torch.Tensor, padded_seqs: int | None = None,
                prev_sampled: torch.Tensor | None = None, status: torch.Tensor | None = None) -> None:
    """meta: device int32 = [seq_len(B) | blk_off(B+1) | blocks_flat | host_tokens(B) | src_index(B)].

    Outputs are written into the given (possibly static, graph-owned) buffers; rows
    ``num_seqs..padded_seqs-1`` become padding rows.
    """
    _need(meta, torch.int32, "meta")
    B = num_seqs
    padded = B if padded_seqs is None else padded_seqs
    base, es = meta.data_ptr(), 4
    o_off = B
    o_blocks = o_off + B + 1
    o_tok = o_blocks + num_blocks_total
    o_src = o_tok + B
    assert meta.numel() >= o_src + B
    assert block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[1] >= table_width
    for t, n in ((input_ids, "input_ids"), (positions, "positions")):
        _need(t, torch.int64, n)
        assert t.numel() >= padded and t.is_contiguous()
    for t, n in ((slot_mapping, "slot_mapping"), (cache_seqlens, "cache_seqlens"), (block_table, "block_table")):
        _need(t, torch.int32, n)
    assert block_table.shape[0] >= padded
    rc = _cabi.load().mvb_pack_decode(
        base, base + es * o_off, base + es * o_blocks, base + es * o_tok, _ptr(prev_sampled),
        base + es * o_src if prev_sampled is not None else None, B, padded, table_width, block_table.stride(0),
        block_size, _ptr(input_ids), _ptr(positions), _ptr(slot_mapping), _ptr(cache_seqlens), _ptr(block_table),
        _ptr(status), _stream())
    _cabi.check(rc, "mvb_pack_decode")
    LaunchCounter.add(1)


def rope_kv_write(q: torch.Tensor | None, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor | None,
                  cos_sin: torch.Tensor | None, slot_mapping: torch.Tensor | None,
                  k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, k_in_place: bool = True,
                  status: torch.Tensor | None = None) -> None:
    """Rotate q (in place) and k, write k/v to their cache slots.  cos_sin=None: no rotation."""
    _need(k, torch.bfloat16, "k"); _need(v, torch.bfloat16, "v")
    _heads_contiguous(k, "k"); _heads_contiguous(v, "v")
    T, hkv, d = k.shape
    hq = 0
    if q is not None:
        _need(q, torch.bfloat16, "q"); _heads_contiguous(q, "q")
        assert q.shape[0] == T and q.shape[2] == d
        hq = q.shape[1]
    max_pos = 0
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos_sin"); _need(positions, torch.int64, "positions")
        assert cos_sin.is_contiguous() and cos_sin.shape[1] == d and positions.numel() == T
        max_pos = cos_sin.shape[0]
    num_slots = 0
    if slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
        assert slot_mapping.numel() == T
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[-2:] == (hkv, d)
        num_slots = k_cache.shape[0] * k_cache.shape[1]
    rc = _cabi.load().mvb_rope_kv_write(
        _ptr(q), q.stride(0) if q is not None else 0, _ptr(k), k.stride(0), _ptr(v), v.stride(0),
        _ptr(positions) if cos_sin is not None else None, _ptr(cos_sin), max_pos, _ptr(slot_mapping),
        _ptr(k_cache) if slot_mapping is not None else None, _ptr(v_cache) if slot_mapping is not None else None,
        num_slots, T, hq, hkv, d, 1 if k_in_place else 0, _ptr(status), _stream())
    _cabi.check(rc, "mvb_rope_kv_write")
    LaunchCounter.add(1)


def qk_norm_rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_weight: torch.Tensor,
                          k_weight: torch.Tensor, eps: float, unit_offset: bool, positions: torch.Tensor,
                          cos_sin: torch.Tensor, slot_mapping: torch.Tensor | None, k_cache: torch.Tensor | None,
                          v_cache: torch.Tensor | None, k_in_place: bool = True,
                          status: torch.Tensor | None = None) -> None:
    """Per-head RMSNorm of q and k, RoPE and the cache write in one kernel; q (and k) updated in place."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _need(t, torch.bfloat16, n); _heads_contiguous(t, n)
    _need(q_weight, torch.bfloat16, "q_weight"); _need(k_weight, torch.bfloat16, "k_weight")
    _need(cos_sin, torch.float32, "cos_sin"); _need(positions, torch.int64, "positions")
    T, hkv, d = k.shape
    hq = q.shape[1]
    assert q.shape[0] == T and q.shape[2] == d and cos_sin.is_contiguous() and cos_sin.shape[1] == d
    assert q_weight.numel() == d and k_weight.numel() == d and q_weight.is_contiguous() and k_weight.is_contiguous()
    num_slots = 0
    if slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
        assert slot_mapping.numel() == T and k_cache.is_contiguous() and v_cache.is_contiguous()
        num_slots = k_cache.shape[0] * k_cache.shape[1]
    rc = _cabi.load().mvb_qk_norm_rope_kv_write(
        _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps),
        1 if unit_offset else 0, _ptr(positions), _ptr(cos_sin), cos_sin.shape[0], _ptr(slot_mapping),
        _ptr(k_cache) if slot_mapping is not None else None, _ptr(v_cache) if slot_mapping is not None else None,
        num_slots, T, hq, hkv, d, 1 if k_in_place else 0, _ptr(status), _stream())
    _cabi.check(rc, "mvb_qk_norm_rope_kv_write")
    LaunchCounter.add(1)


def decode_workspace(max_seqs: int, num_q_heads: int, head_dim: int, device) -> torch.Tensor:
    n = _cabi.load().mvb_decode_workspace_bytes(max_seqs, num_q_heads, head_dim)
    if n == 0:
        raise ValueError("bad decode workspace shape")
    return torch.empty(n, dtype=torch.uint8, device=device)


def decode_plan(cache_seqlens: torch.Tensor, window_left: int, num_q_heads: int, num_kv_heads: int,
                head_dim: int, workspace: torch.Tensor, block_table: torch.Tensor | None = None,
                block_size: int = 0) -> None:
    """Plan the split of one decode step.  With ``block_table`` (the one the attention calls will get)
    the plan also records each CTA's first block id, sparing every layer a dependent load."""
    _need(cache_seqlens, torch.int32, "cache_seqlens")
    if block_table is not None:
        _need(block_table, torch.int32, "block_table")
        assert block_table.stride(1) == 1 and block_table.shape[0] >= cache_seqlens.numel() and block_size > 0
        rc = _cabi.load().mvb_decode_plan_with_table(
            _ptr(cache_seqlens), _ptr(block_table), block_table.stride(0), block_size, cache_seqlens.numel(),
            window_left, num_q_heads, num_kv_heads, head_dim, _ptr(workspace), workspace.numel(), _stream())
    else:
        rc = _cabi.load().mvb_decode_plan(_ptr(cache_seqlens), cache_seqlens.numel(), window_left, num_q_heads,
                                          num_kv_heads, head_dim, _ptr(workspace), workspace.numel(), _stream())
    _cabi.check(rc, "mvb_decode_plan")
    LaunchCounter.add(1)


def decode_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cache_seqlens: torch.Tensor,
                block_table: torch.Tensor, scale: float, window_left: int, workspace: torch.Tensor,
                out: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """q [B,Hq,D]; the plan for (cache_seqlens, window_left) must already be in ``workspace``."""
    _need(q, torch.bfloat16, "q"); _heads_contiguous(q, "q")
    _need(cache_seqlens, torch.int32, "cache_seqlens"); _need(block_table, torch.int32, "block_table")
    B, hq, d = q.shape
    nblk, bs, hkv, d2 = k_cache.shape
    assert d2 == d and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
    assert block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= B
    assert cache_seqlens.numel() >= B
    if out is None:
        out = torch.empty(B, hq, d, dtype=torch.bfloat16, device=q.device)
    rc = _cabi.load().mvb_decode_attn(
        _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), nblk, bs, _ptr(cache_seqlens), _ptr(block_table),
        block_table.stride(0), block_table.shape[1], B, hq, hkv, d, float(scale), window_left, _ptr(out),
        out.stride(0), _ptr(workspace), workspace.numel(), _ptr(status), _stream())
    _cabi.check(rc, "mvb_decode_attn")
    LaunchCounter.add(1)
    return out


def decode_attn_static(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cache_seqlens: torch.Tensor,
                       block_table: torch.Tensor, scale: float, window_left: int, out: torch.Tensor,
                       status: torch.Tensor | None = None) -> torch.Tensor:
    """Decode attention that brings its own scratch (``mvb_decode_attn_static``).

    For callers that have no way to allocate a workspace next to this call: the plan and the partial
    results live in an 8 MiB array inside the library, so the only buffers involved are the ones passed
    here, ``out`` included.  Calls on one device share that array and must not overlap on the GPU;
    the first call on a device should happen outside stream capture.  Raises ``KernelError`` when the
    request is too large for the built-in array.
    """
    _need(q, torch.bfloat16, "q"); _heads_contiguous(q, "q")
    _need(cache_seqlens, torch.int32, "cache_seqlens"); _need(block_table, torch.int32, "block_table")
    _need(out, torch.bfloat16, "out")
    B, hq, d = q.shape
    nblk, bs, hkv, _ = k_cache.shape
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.stride(1) == 1
    rc = _cabi.load().mvb_decode_attn_static(
        _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), nblk, bs, _ptr(cache_seqlens), _ptr(block_table),
        block_table.stride(0), block_table.shape[1], B, hq, hkv, d, float(scale), window_left, _ptr(out),
        out.stride(0), _ptr(status), _stream())
    _cabi.check(rc, "mvb_decode_attn_static")
    LaunchCounter.add(2)
    return out


def prefill_item_rows(num_q_heads: int, num_kv_heads: int, head_dim: int) -> int:
    """Rows of q that one work item of the prefill kernel covers (128 or 256; a property of the head layout)."""
    rows = _cabi.load().mvb_prefill_item_rows(num_q_heads, num_kv_heads, head_dim)
    _cabi.check(min(rows, 0), "mvb_prefill_item_rows")
    return rows


def build_prefill_items(q_lens, k_lens, item_rows: int):
    """The work list of a prefill launch: int32 [n, 2] of (sequence, query block), every query block of every
    sequence once, the blocks that see the most keys first (the order in which the GPU takes them).  Pure host
    arithmetic on the per-sequence lengths the packing step already has; numpy in, numpy out."""
    import numpy as np
    q_lens = np.asarray(q_lens, np.int64)
    k_lens = np.asarray(k_lens, np.int64)
    n_qb = (q_lens + item_rows - 1) // item_rows
    seq = np.repeat(np.arange(q_lens.size, dtype=np.int64), n_qb)
    first = np.cumsum(n_qb) - n_qb
    qb = np.arange(int(n_qb.sum()), dtype=np.int64) - np.repeat(first, n_qb)
    # keys visible to the block's last row: its position + 1
    visible = k_lens[seq] - q_lens[seq] + np.minimum((qb + 1) * item_rows, q_lens[seq])
    order = np.argsort(-visible, kind="stable")
    return np.stack([seq[order], qb[order]], axis=1).astype(np.int32)


def prefill_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                 cu_seqlens_k: torch.Tensor, max_seqlen_q: int, scale: float, window_left: int = -1,
                 block_table: torch.Tensor | None = None, out: torch.Tensor | None = None,
                 status: torch.Tensor | None = None, items: torch.Tensor | None = None) -> torch.Tensor:
    """q [Tq,Hq,D]; k/v dense [Tk,Hkv,D] (block_table None) or the paged pool [blocks,bs,Hkv,D].

    ``items`` (int32 [n, 2] on the device, from ``build_prefill_items``) gives the launch its work as a list of
    (sequence, query block) pairs instead of a grid over the longest sequence's block count: same result, no
    empty block indices, the longest blocks first."""
    _need(q, torch.bfloat16, "q"); _heads_contiguous(q, "q")
    _need(cu_seqlens_q, torch.int32, "cu_seqlens_q"); _need(cu_seqlens_k, torch.int32, "cu_seqlens_k")
    Tq, hq, d = q.shape
    if block_table is None:
        _heads_contiguous(k, "k"); _heads_contiguous(v, "v")
        kv_rows, hkv, k_stride, v_stride, bs, tstride = k.shape[0], k.shape[1], k.stride(0), v.stride(0), 0, 0
    else:
        _need(block_table, torch.int32, "block_table")
        assert k.dim() == 4 and k.is_contiguous() and v.is_contiguous()
        nblk, bs, hkv, _ = k.shape
        kv_rows, k_stride, v_stride, tstride = nblk * bs, hkv * d, hkv * d, block_table.stride(0)
    if out is None:
        out = torch.empty(Tq, hq, d, dtype=torch.bfloat16, device=q.device)
    if items is not None and 0 < items.shape[0] <= 65535:
        _need(items, torch.int32, "items")
        assert items.dim() == 2 and items.shape[1] == 2 and items.is_contiguous()
        rc = _cabi.load().mvb_prefill_attn_items(
            _ptr(q), q.stride(0), _ptr(k), k_stride, _ptr(v), v_stride, kv_rows, _ptr(cu_seqlens_q), _ptr(cu_seqlens_k),
            _ptr(block_table), tstride, bs, cu_seqlens_q.numel() - 1, Tq, int(max_seqlen_q), hq, hkv, d, float(scale),
            window_left, _ptr(out), out.stride(0), _ptr(items), items.shape[0], _ptr(status), _stream())
        _cabi.check(rc, "mvb_prefill_attn_items")
        LaunchCounter.add(1)
        return out
    rc = _cabi.load().mvb_prefill_attn(
        _ptr(q), q.stride(0), _ptr(k), k_stride, _ptr(v), v_stride, kv_rows, _ptr(cu_seqlens_q), _ptr(cu_seqlens_k),
        _ptr(block_table), tstride, bs, cu_seqlens_q.numel() - 1, Tq, int(max_seqlen_q), hq, hkv, d, float(scale),
        window_left, _ptr(out), out.stride(0), _ptr(status), _stream())
    _cabi.check(rc, "mvb_prefill_attn")
    LaunchCounter.add(1)
    return out


def sample(logits: torch.Tensor, temperatures: torch.Tensor | None = None, top_k: torch.Tensor | None = None,
           seed: int = 0, offset: int = 0, out: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
           scatter_table: torch.Tensor | None = None, scatter_index: torch.Tensor | None = None) -> torch.Tensor:
    """logits bf16 [B,V] -> int64 [B].  top_k and top_p None: greedy; else temperature/top-k/top-p/Gumbel-max.

    With ``scatter_table`` (int64) and ``scatter_index`` (int32 [B]) the tokens are also written to
    ``scatter_table[scatter_index]`` on the device."""
    _need(logits, torch.bfloat16, "logits")
    assert logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    if temperatures is not None:
        _need(temperatures, torch.float32, "temperatures")
    if top_k is not None:
        _need(top_k, torch.int32, "top_k")
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    if scatter_table is not None:
        _need(scatter_table, torch.int64, "scatter_table"); _need(scatter_index, torch.int32, "scatter_index")
        assert scatter_index.numel() >= B
    if top_p is not None:
        _need(top_p, torch.float32, "top_p")
    rc = _cabi.load().mvb_sample(_ptr(logits), logits.stride(0), B, V, _ptr(temperatures), _ptr(top_k), _ptr(top_p),
                                 seed & (2**64 - 1), offset & (2**64 - 1), _ptr(out), _ptr(scatter_table),
                                 _ptr(scatter_index), None, _stream())
    _cabi.check(rc, "mvb_sample")
    LaunchCounter.add(1)
    return out


def act_mul(gate_up: torch.Tensor, intermediate: int, gelu_tanh: bool, out: torch.Tensor | None = None) -> torch.Tensor:
    """``act(gate) * up`` on a packed ``[rows, 2 * intermediate]`` projection (SiLU, or tanh-GELU)."""
    _need(gate_up, torch.bfloat16, "gate_up")
    assert gate_up.dim() == 2 and gate_up.stride(1) == 1 and gate_up.shape[1] == 2 * intermediate
    rows = gate_up.shape[0]
    if out is None:
        out = torch.empty(rows, intermediate, dtype=torch.bfloat16, device=gate_up.device)
    rc = _cabi.load().mvb_act_mul(_ptr(gate_up), gate_up.stride(0), _ptr(out), out.stride(0), rows, intermediate,
                                  1 if gelu_tanh else 0, _stream())
    _cabi.check(rc, "mvb_act_mul")
    LaunchCounter.add(1)
    return out


def add_rmsnorm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, unit_offset: bool,
                y_weight: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x += y`` (or ``x += rmsnorm(y, y_weight)``) in place, returns ``rmsnorm(x, weight)``."""
    _need(x, torch.bfloat16, "x"); _need(y, torch.bfloat16, "y"); _need(weight, torch.bfloat16, "weight")
    assert x.dim() == 2 and x.is_contiguous() and y.shape == x.shape and y.stride(1) == 1
    rows, hidden = x.shape
    if out is None:
        out = torch.empty_like(x)
    rc = _cabi.load().mvb_add_rmsnorm(_ptr(x), _ptr(y), y.stride(0), _ptr(y_weight), _ptr(weight), _ptr(out), rows,
                                      hidden, float(eps), 1 if unit_offset else 0, _stream())
    _cabi.check(rc, "mvb_add_rmsnorm")
    LaunchCounter.add(1)
    return out


def add_rmsnorm_last_tokens(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, unit_offset: bool,
                            cu_seqlens_q: torch.Tensor, y_weight: torch.Tensor | None = None) -> torch.Tensor:
    """``rmsnorm(x + y)`` (or ``x + rmsnorm(y, y_weight)``) for the last token of every sequence only:
    ``[num_seqs, hidden]``, row r from source row ``cu_seqlens_q[r + 1] - 1``.  ``x`` is left untouched."""
    _need(x, torch.bfloat16, "x"); _need(y, torch.bfloat16, "y"); _need(weight, torch.bfloat16, "weight")
    _need(cu_seqlens_q, torch.int32, "cu_seqlens_q")
    assert x.dim() == 2 and x.is_contiguous() and y.shape == x.shape and y.stride(1) == 1
    num_seqs, hidden = cu_seqlens_q.numel() - 1, x.shape[1]
    out = torch.empty(num_seqs, hidden, dtype=torch.bfloat16, device=x.device)
    rc = _cabi.load().mvb_add_rmsnorm_last_tokens(_ptr(x), _ptr(y), y.stride(0), _ptr(y_weight), _ptr(weight), _ptr(out),
                                                  _ptr(cu_seqlens_q), num_seqs, hidden, float(eps),
                                                  1 if unit_offset else 0, _stream())
    _cabi.check(rc, "mvb_add_rmsnorm_last_tokens")
    LaunchCounter.add(1)
    return out


def lm_head_argmax_scratch(max_rows: int, device) -> torch.Tensor:
    """Zeroed scratch for ``lm_head_argmax`` (every call leaves it zeroed again)."""
    n = _cabi.load().mvb_lm_head_argmax_scratch_bytes(max_rows)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def lm_head_argmax(hidden_states: torch.Tensor, weight: torch.Tensor, scratch: torch.Tensor,
                   out: torch.Tensor | None = None, scatter_table: torch.Tensor | None = None,
                   scatter_index: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """``argmax(hidden_states @ weight.T)`` per row over bf16-rounded logits, without materialising them."""
    _need(hidden_states, torch.bfloat16, "hidden_states"); _need(weight, torch.bfloat16, "weight")
    assert hidden_states.dim() == 2 and weight.dim() == 2 and hidden_states.stride(1) == 1 and weight.stride(1) == 1
    rows, hidden = hidden_states.shape
    vocab = weight.shape[0]
    assert weight.shape[1] == hidden
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=hidden_states.device)
    if scatter_table is not None:
        _need(scatter_table, torch.int64, "scatter_table"); _need(scatter_index, torch.int32, "scatter_index")
        assert scatter_index.numel() >= rows
    rc = _cabi.load().mvb_lm_head_argmax(_ptr(hidden_states), hidden_states.stride(0), _ptr(weight), weight.stride(0), rows,
                                         hidden, vocab, _ptr(out), _ptr(scatter_table), _ptr(scatter_index), _ptr(scratch),
                                         scratch.numel(), _ptr(status), _stream())
    _cabi.check(rc, "mvb_lm_head_argmax")
    LaunchCounter.add(1)
    return out
