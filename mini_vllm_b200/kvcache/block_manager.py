"""Paged KV-cache block allocator with an optional hash-chained prefix cache.

Behaviourally identical to ``minivllm/kvcache/block_manager.py`` (the block ids it hands out
decide every slot mapping and block table downstream, so they must match exactly):

* free blocks form an ordered list initialised ``0..capacity-1``; allocation takes the LAST
  entry (``:119``), so a fresh pool hands out ``capacity-1, capacity-2, ...``; freeing walks a
  request's blocks in reverse and appends each block whose refcount drops to zero (``:100-109``);
* a full block's hash is ``xxh64(prefix_hash as 8 LE bytes (omitted for the first block) ||
  tokens as signed 32-bit LE)`` (``:23-30``); a hit needs the hash to map to a block whose stored
  tokens are equal, and the first miss turns every later block of that prompt into a miss
  (``:60-73``); a hit on a live block bumps its refcount, a hit on a freed but intact block takes
  exactly that id out of the free list (``:76-81``);
* stale hash entries are never purged (the reference resets a block's hash before testing it,
  ``:125-128``); the token comparison keeps that safe.

Implementation differences (not observable): the free list is an insertion-ordered dict, which
gives O(1) pop-last, append and remove-by-id instead of ``deque.remove``; hashing feeds xxhash one
``int32`` buffer per block instead of one 4-byte update per token; block contents are kept as the
hashed byte string.
"""
from __future__ import annotations

import numpy as np
import xxhash

from ..engine.request import Request
from ..utils import cdiv

NO_HASH = -1


def block_hash(tokens, prefix: int = NO_HASH) -> int:
    h = xxhash.xxh64()
    if prefix != NO_HASH:
        h.update(int(prefix).to_bytes(8, "little"))
    h.update(np.asarray(tokens, dtype="<i4").tobytes())
    return h.intdigest()


class KVCacheBlock:
    """Kept for API parity; ``compute_hash`` is the reference's static helper."""
    compute_hash = staticmethod(block_hash)


class KVCacheBlockManager:
    def __init__(self, capacity: int, block_size: int, support_prefix_cache: bool = False,
                 keep_last_block_uncached: bool = False):
        self.block_size = block_size
        self.capacity = capacity
        self.support_prefix_cache = support_prefix_cache
        # When a whole prompt is found in the cache the reference marks every token cached, which
        # leaves the prefill with zero query tokens and no logits for that request
        # (executor.py:96, qwen3.py:216).  With this flag the last block of such a prompt is
        # prefilled again so the request always has a last-token row.
        self.keep_last_block_uncached = keep_last_block_uncached
        self._free: dict[int, None] = dict.fromkeys(range(capacity))
        self._refcount = [0] * capacity
        self._hash = [NO_HASH] * capacity
        self._content: list[bytes] = [b""] * capacity
        self.used_block_ids: set[int] = set()
        self.hash_to_block_id: dict[int, int] = {}

    # ---- views used by tests and the scheduler ------------------------------------------------
    @property
    def free_block_ids(self) -> list[int]:
        return list(self._free)

    @property
    def num_free_blocks(self) -> int:
        return len(self._free)

    def request_required_blocks(self, req: Request) -> int:
        return cdiv(len(req.tokens), self.block_size) - len(req.blocks)

    def can_allocate_new_block(self, req: Request) -> bool:
        return len(self._free) >= self.request_required_blocks(req)

    # ---- allocation ----------------------------------------------------------------------------
    def _take(self, bid: int = -1) -> int:
        if not self._free:
            raise RuntimeError("KV cache exhausted")
        if bid < 0:
            bid, _ = self._free.popitem()
        else:
            del self._free[bid]
        assert self._refcount[bid] == 0
        self._refcount[bid] = 1
        self._hash[bid] = NO_HASH
        self._content[bid] = b""
        self.used_block_ids.add(bid)
        return bid

    def _publish(self, bid: int, h: int, content: bytes) -> None:
        self._hash[bid] = h
        self._content[bid] = content
        self.hash_to_block_id[h] = bid

    def allocate_blocks_for_prefill(self, req: Request) -> None:
        assert req.state == Request.WAITING and not req.blocks
        bs, n = self.block_size, len(req.tokens)
        toks = np.asarray(req.tokens, dtype="<i4")
        chain, missed = NO_HASH, False
        # A negative id stands for a sampled token that has not reached the host yet (the pipelined engine's
        # placeholder).  A block holding one is neither looked up nor published, and neither is any block
        # behind it: its hash would chain over content that is not the request's.
        unknown = np.flatnonzero(toks < 0)
        first_unknown = int(unknown[0]) if unknown.size else n
        for start in range(0, n, bs):
            full = start + bs <= n
            if not (full and self.support_prefix_cache) or start + bs > first_unknown:
                req.blocks.append(self._take())
                continue
            content = toks[start:start + bs].tobytes()
            h = xxhash.xxh64()
            if chain != NO_HASH:
                h.update(chain.to_bytes(8, "little"))
            h.update(content)
            chain = h.intdigest()
            hit = self.hash_to_block_id.get(chain, -1)
            if hit < 0 or self._content[hit] != content:
                missed = True
            if not missed and self.keep_last_block_uncached and start + bs == n:
                missed = True
            if missed:
                bid = self._take()
            else:
                req.num_cached_tokens += bs
                if hit in self.used_block_ids:
                    self._refcount[hit] += 1
                    bid = hit
                else:
                    bid = self._take(hit)
            self._publish(bid, chain, content)
            req.blocks.append(bid)

    def allocate_block_for_decode(self, req: Request) -> None:
        assert req.state == Request.RUNNING and req.blocks
        if self.request_required_blocks(req) > 0:
            req.blocks.append(self._take())

    def deallocate(self, req: Request) -> None:
        for bid in reversed(req.blocks):
            assert self._refcount[bid] > 0
            self._refcount[bid] -= 1
            if self._refcount[bid] == 0:
                self.used_block_ids.discard(bid)
                self._free[bid] = None
        req.blocks = []
        req.num_cached_tokens = 0

    def cache_block_at(self, req: Request, index: int) -> None:
        """Publish block ``index`` of the request, which has become full some steps ago (the pipelined
        engine learns a block's last tokens late).  Nothing happens if the request has lost the block in
        the meantime (finished or preempted) or the block before it was never published."""
        if not self.support_prefix_cache or index >= len(req.blocks) or len(req.tokens) < (index + 1) * self.block_size:
            return
        bid = req.blocks[index]
        if self._hash[bid] != NO_HASH:
            return
        prefix = self._hash[req.blocks[index - 1]] if index > 0 else NO_HASH
        if index > 0 and prefix == NO_HASH:
            return
        content = np.asarray(req.tokens[index * self.block_size:(index + 1) * self.block_size], dtype="<i4").tobytes()
        h = xxhash.xxh64()
        if prefix != NO_HASH:
            h.update(prefix.to_bytes(8, "little"))
        h.update(content)
        self._publish(bid, h.intdigest(), content)

    def cache_block_if_needed(self, req: Request) -> None:
        """Publish the request's last block once it is full (block_manager.py:144-158)."""
        if not self.support_prefix_cache or len(req.tokens) % self.block_size:
            return
        last = req.blocks[-1]
        assert self._hash[last] == NO_HASH
        prefix = self._hash[req.blocks[-2]] if len(req.blocks) > 1 else NO_HASH
        content = np.asarray(req.tokens[-self.block_size:], dtype="<i4").tobytes()
        h = xxhash.xxh64()
        if prefix != NO_HASH:
            h.update(prefix.to_bytes(8, "little"))
        h.update(content)
        self._publish(last, h.intdigest(), content)
