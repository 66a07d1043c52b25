"""Paged KV-cache bookkeeping (host side) and the device tensors behind it.

Layout of one layer's cache: K and V tensors of shape
``[num_blocks, local_kv_heads, block_size, head_dim]``. ``local_kv_heads`` is the
per-rank share under TP*SP head sharding and is identical in sequence-parallel
and tensor-parallel mode, which is what lets shift parallelism switch modes
without moving KV (reference: arctic_inference/vllm/ulysses.py:60-70,402-416 and
arctic_inference/vllm/model_runner.py:1758-1772). Every rank runs this manager
with the same inputs, so block ids agree across ranks without communication.

Prefix caching: full blocks are keyed by a hash chained over the tokens they
hold; a finished request's blocks stay in an LRU pool and are revived when a
later prompt hashes to the same chain.
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional

import torch


def hash_block(parent_hash: Optional[bytes], tokens) -> bytes:
    h = hashlib.blake2b(digest_size=16)
    h.update(parent_hash or b"root")
    h.update(struct.pack("%di" % len(tokens), *tokens))
    return h.digest()


@dataclass
class _Block:
    block_id: int
    ref: int = 0
    hash: Optional[bytes] = None


class BlockPool:
    """Fixed pool of KV blocks with reference counts and an LRU of cached-but-free blocks."""

    def __init__(self, num_blocks: int, enable_prefix_caching: bool = True):
        # block 0 is reserved as the "null" block that padding slots may point at
        self.num_blocks = num_blocks
        self.enable_prefix_caching = enable_prefix_caching
        self.blocks = [_Block(i) for i in range(num_blocks)]
        self.free: OrderedDict[int, None] = OrderedDict((i, None) for i in range(1, num_blocks))
        self.cached: dict[bytes, int] = {}

    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def usage(self) -> float:
        usable = self.num_blocks - 1
        return 1.0 - len(self.free) / usable if usable > 0 else 0.0

    def lookup(self, h: bytes) -> Optional[int]:
        return self.cached.get(h) if self.enable_prefix_caching else None

    def touch(self, block_id: int) -> None:
        """Take a reference on a block found through the prefix cache."""
        b = self.blocks[block_id]
        if b.ref == 0:
            self.free.pop(block_id, None)
        b.ref += 1

    def allocate(self, n: int) -> list[int]:
        if n > len(self.free):
            raise RuntimeError("out of KV blocks")
        out = []
        for _ in range(n):
            bid, _ = self.free.popitem(last=False)  # least recently freed first
            b = self.blocks[bid]
            if b.hash is not None:  # evict its cached identity
                if self.cached.get(b.hash) == bid:
                    del self.cached[b.hash]
                b.hash = None
            b.ref = 1
            out.append(bid)
        return out

    def release(self, block_ids) -> None:
        # free in reverse so that the tail of a sequence is evicted before its head
        for bid in reversed(list(block_ids)):
            b = self.blocks[bid]
            b.ref -= 1
            assert b.ref >= 0
            if b.ref == 0:
                self.free[bid] = None

    def set_hash(self, block_id: int, h: bytes) -> None:
        if not self.enable_prefix_caching:
            return
        b = self.blocks[block_id]
        if b.hash is None and h not in self.cached:
            b.hash = h
            self.cached[h] = block_id

    def reset_prefix_cache(self) -> None:
        for b in self.blocks:
            b.hash = None
        self.cached.clear()


class KVCacheManager:
    """Per-request block tables on top of a :class:`BlockPool`."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = True):
        self.block_size = block_size
        self.pool = BlockPool(num_blocks, enable_prefix_caching)
        self._hashes: dict[str, list[bytes]] = {}

    # -- prefix cache -------------------------------------------------------------------
    def match_prefix(self, request) -> int:
        """Attach cached blocks covering a prefix of the prompt; returns cached token count.
        The last prompt token is never served from cache (its logits are needed)."""
        if not self.pool.enable_prefix_caching or request.block_ids:
            return 0
        bs = self.block_size
        toks = request.prompt_token_ids
        max_blocks = (len(toks) - 1) // bs
        parent = None
        hashes = []
        got = []
        for i in range(max_blocks):
            h = hash_block(parent, toks[i * bs:(i + 1) * bs])
            bid = self.pool.lookup(h)
            if bid is None:
                break
            hashes.append(h)
            got.append(bid)
            parent = h
        for bid in got:
            self.pool.touch(bid)
        request.block_ids = list(got)
        self._hashes[request.request_id] = hashes
        return len(got) * bs

    def _publish_full_blocks(self, request, num_computed: int) -> None:
        if not self.pool.enable_prefix_caching:
            return
        bs = self.block_size
        hashes = self._hashes.setdefault(request.request_id, [])
        full = num_computed // bs
        while len(hashes) < full:
            i = len(hashes)
            toks = [request.token_at(j) for j in range(i * bs, (i + 1) * bs)]
            h = hash_block(hashes[-1] if hashes else None, toks)
            hashes.append(h)
            self.pool.set_hash(request.block_ids[i], h)

    # -- allocation ---------------------------------------------------------------------
    def blocks_needed(self, request, num_new_tokens: int) -> int:
        total = request.num_computed_tokens + num_new_tokens
        need = (total + self.block_size - 1) // self.block_size
        return max(0, need - len(request.block_ids))

    def can_allocate(self, request, num_new_tokens: int) -> bool:
        return self.blocks_needed(request, num_new_tokens) <= self.pool.num_free

    def allocate(self, request, num_new_tokens: int) -> None:
        n = self.blocks_needed(request, num_new_tokens)
        if n:
            request.block_ids.extend(self.pool.allocate(n))

    def commit(self, request, num_computed: int) -> None:
        """Called after a step: tokens below ``num_computed`` now have valid KV."""
        self._publish_full_blocks(request, num_computed)

    def free(self, request) -> None:
        self.pool.release(request.block_ids)
        request.block_ids = []
        request._block_array = None
        self._hashes.pop(request.request_id, None)

    def slot(self, request, position: int) -> int:
        return request.block_ids[position // self.block_size] * self.block_size + \
            position % self.block_size

    @property
    def usage(self) -> float:
        return self.pool.usage

    def reset_prefix_cache(self) -> None:
        self.pool.reset_prefix_cache()


class KVCacheTensors:
    """Device memory of the cache: one (K, V) pair per layer."""

    def __init__(self, num_layers: int, num_blocks: int, local_kv_heads: int, block_size: int,
                 head_dim: int, dtype: torch.dtype, device, layers: Optional[range] = None):
        """``layers``: the layers this rank runs (a pipeline stage); the others get no memory."""
        self.shape = (num_blocks, local_kv_heads, block_size, head_dim)
        own = range(num_layers) if layers is None else layers
        self.k = [torch.zeros(self.shape, dtype=dtype, device=device) if l in own else None
                  for l in range(num_layers)]
        self.v = [torch.zeros(self.shape, dtype=dtype, device=device) if l in own else None
                  for l in range(num_layers)]
        self._tables: dict = {}

    def pointer_tables(self, first: int, count: int):
        """Device tables (int64) of the K and V base addresses of ``count`` consecutive layers,
        for kernels that write several layers in one launch. Built once per range."""
        key = (first, count)
        t = self._tables.get(key)
        if t is None:
            dev = self.k[first].device
            t = (torch.tensor([c.data_ptr() for c in self.k[first:first + count]],
                              dtype=torch.int64, device=dev),
                 torch.tensor([c.data_ptr() for c in self.v[first:first + count]],
                              dtype=torch.int64, device=dev))
            self._tables[key] = t
        return t

    @staticmethod
    def bytes_per_block(num_layers, local_kv_heads, block_size, head_dim, elem_bytes=2) -> int:
        return 2 * num_layers * local_kv_heads * block_size * head_dim * elem_bytes

    def free(self) -> None:
        self.k, self.v = [], []
        self._tables = {}
