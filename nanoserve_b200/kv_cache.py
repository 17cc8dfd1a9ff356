"""Paged KV cache: block pool, allocators (plain and prefix-caching) and per-request block tables.

Public names and behaviour follow the reference (nanoserve/kv_cache.py:75-288): `NoFreeBlocks`,
`BlockAllocator`, `PrefixCachingAllocator`, `BlockTable`, `PagedKVCache`. All of it is host-side integer
bookkeeping whose results (block ids, slots, eviction order) must equal the reference's exactly; the pool
tensors themselves live in HBM and are only touched by the CUDA kernels.

Layout of the pool (API-visible, tests index it): k, v : [n_layers, num_blocks, block_size, n_kv_heads, head_dim],
zero-filled; slot of token t of a request = table[t // block_size] * block_size + t % block_size.
"""
from __future__ import annotations

from collections import OrderedDict

import torch


class NoFreeBlocks(Exception):
    """The pool is exhausted: the scheduler must preempt someone or wait."""


class BlockAllocator:
    """Free list handing out block ids 0, 1, 2, ... first; freed blocks are reused most-recent-first
    [kv_cache.py:79-101]."""

    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._free: list[int] = list(reversed(range(num_blocks)))     # pop() from the tail
        self._used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise NoFreeBlocks()
        b = self._free.pop()
        self._used.add(b)
        return b

    def free(self, blocks: list[int]) -> None:
        for b in blocks:
            if b not in self._used:
                raise ValueError(f"block {b} freed twice (or never allocated)")
            self._used.discard(b)
            self._free.append(b)


class PrefixCachingAllocator:
    """Reference-counted allocator that keeps FULL blocks findable by their exact token prefix
    [kv_cache.py:104-204].

    key(block i of a request) = (node id of block i-1's key, tuple of block i's token ids); every new key gets
    a fresh node id, so keys form a trie and lookups are exact. A registered block whose last holder lets go is
    parked in an LRU list: still cached, but counted as free capacity; allocate() prefers truly free blocks and
    otherwise evicts the least recently released cached block.
    """

    def __init__(self, base: BlockAllocator, block_size: int):
        self.base = base
        self.block_size = block_size
        self.ref: dict[int, int] = {}
        self.block_of: dict[tuple, int] = {}
        self.key_of: dict[int, tuple] = {}
        self.node_of: dict[int, int] = {}
        self.evictable: OrderedDict[int, None] = OrderedDict()
        self._next_node = 1                      # node 0 is the empty prefix

    @property
    def num_free(self) -> int:
        return self.base.num_free + len(self.evictable)

    @property
    def num_evictable(self) -> int:
        return len(self.evictable)

    @property
    def num_blocks(self) -> int:
        return self.base.num_blocks

    def _forget(self, block: int) -> None:
        self.block_of.pop(self.key_of.pop(block))
        self.node_of.pop(block)

    def allocate(self) -> int:
        if self.base.num_free > 0:
            block = self.base.allocate()
        elif self.evictable:
            block = next(iter(self.evictable))   # least recently released
            del self.evictable[block]
            self._forget(block)
        else:
            raise NoFreeBlocks()
        self.ref[block] = 1
        return block

    def free(self, blocks: list[int]) -> None:
        # tail first, so a request's prefix outlives its suffix in the LRU order [kv_cache.py:158-168]
        for b in blocks[::-1]:
            count = self.ref.get(b, 0)
            if count <= 0:
                raise ValueError(f"block {b} freed twice (or never allocated)")
            if count > 1:
                self.ref[b] = count - 1
                continue
            del self.ref[b]
            if b in self.key_of:
                self.evictable[b] = None
            else:
                self.base.free([b])

    def lookup(self, token_ids: list[int], max_blocks: int | None = None) -> list[int]:
        """Blocks holding the longest cached whole-block prefix of token_ids; no side effects."""
        bs = self.block_size
        limit = len(token_ids) // bs
        if max_blocks is not None:
            limit = min(limit, max_blocks)
        found: list[int] = []
        node = 0
        for i in range(limit):
            block = self.block_of.get((node, tuple(token_ids[i * bs:i * bs + bs])))
            if block is None:
                break
            found.append(block)
            node = self.node_of[block]
        return found

    def pin(self, blocks: list[int]) -> None:
        for b in blocks:
            held = self.ref.get(b, 0)
            if held == 0:
                del self.evictable[b]
            self.ref[b] = held + 1

    def register(self, table: "BlockTable", token_ids: list[int]) -> None:
        """Make every block of `table` that became full since the last call findable. When the same prefix was
        registered meanwhile by someone else, theirs stays the cached copy [kv_cache.py:190-204]."""
        bs = self.block_size
        for i in range(table.num_hashed, table.num_tokens // bs):
            key = (table.prefix_node, tuple(token_ids[i * bs:i * bs + bs]))
            other = self.block_of.get(key)
            if other is not None:
                node = self.node_of[other]
            else:
                mine = table.blocks[i]
                node = self._next_node
                self._next_node += 1
                self.block_of[key] = mine
                self.key_of[mine] = key
                self.node_of[mine] = node
            table.prefix_node = node
            table.num_hashed = i + 1


class BlockTable:
    """One request's blocks, in order, and how many of its tokens have K/V stored [kv_cache.py:207-248]."""

    def __init__(self, block_size: int):
        self.block_size = block_size
        self.blocks: list[int] = []
        self.num_tokens = 0
        self.num_hashed = 0
        self.prefix_node = 0

    def blocks_needed(self, n_new: int) -> int:
        total = -(-(self.num_tokens + n_new) // self.block_size)
        return max(0, total - len(self.blocks))

    def reserve(self, n_new: int, allocator) -> None:
        for _ in range(self.blocks_needed(n_new)):
            self.blocks.append(allocator.allocate())

    def slots(self, n_new: int) -> list[int]:
        bs, blocks = self.block_size, self.blocks
        start = self.num_tokens
        return [blocks[p // bs] * bs + p % bs for p in range(start, start + n_new)]

    def commit(self, n: int) -> None:
        self.num_tokens += n

    def truncate(self, n_tokens: int, allocator) -> None:
        keep = -(-n_tokens // self.block_size)
        allocator.free(self.blocks[keep:])
        del self.blocks[keep:]
        self.num_tokens = n_tokens

    def rewind(self, n_tokens: int) -> None:
        assert n_tokens <= self.num_tokens
        self.num_tokens = n_tokens

    def release(self, allocator) -> None:
        allocator.free(self.blocks)
        self.blocks = []
        self.num_tokens = 0


class PagedKVCache:
    """The shared block pool, allocated once [kv_cache.py:251-288]."""

    def __init__(self, cfg, num_blocks: int, block_size: int = 16, device="cuda", dtype=torch.bfloat16):
        shape = (cfg.n_layers, num_blocks, block_size, cfg.n_kv_heads, cfg.head_dim)
        self.k = torch.zeros(shape, device=device, dtype=dtype)
        self.v = torch.zeros(shape, device=device, dtype=dtype)
        self.cfg = cfg
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.allocator = BlockAllocator(num_blocks)
        self.reserved_bytes = num_blocks * block_size * cfg.kv_bytes_per_token(dtype)

    @classmethod
    def from_token_budget(cls, cfg, num_tokens: int, block_size: int = 16, device="cuda",
                          dtype=torch.bfloat16) -> "PagedKVCache":
        return cls(cfg, -(-num_tokens // block_size), block_size, device, dtype)

    @staticmethod
    def tokens_for_bytes(cfg, nbytes: int, dtype=torch.bfloat16) -> int:
        return nbytes // cfg.kv_bytes_per_token(dtype)

    def write(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        """Store this step's K/V ([N, n_kv_heads, head_dim]) at their slots: one scatter kernel for all
        requests (ns_kv_write)."""
        from nanoserve_b200.kernels.fused import kv_write
        kv_write(k_new.contiguous(), v_new.contiguous(), self.k[layer], self.v[layer], slot_mapping)

    def gather(self, layer: int, block_table: torch.Tensor, length: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Dense copy of one request's first `length` tokens, [1, n_kv_heads, length, head_dim]. Inspection
        helper only: the attention kernel reads the blocks in place."""
        kvh, hd = self.cfg.n_kv_heads, self.cfg.head_dim
        idx = block_table.long()
        k = self.k[layer][idx].reshape(-1, kvh, hd)[:length]
        v = self.v[layer][idx].reshape(-1, kvh, hd)[:length]
        return k.transpose(0, 1)[None], v.transpose(0, 1)[None]
