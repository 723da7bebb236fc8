"""Cache and state manager: pages of the key/value cache and slots of recurrent state.

The reference's block manager (backends/vllm/src/block_manager.rs, block_allocator.rs) hands out
fixed-size physical blocks from a free list and keeps one block table per sequence; this is the same
bookkeeping for one device pool, plus what a model with recurrent layers needs beside it: a small pool
of state slots, one per live sequence, handed out at admission and given back with the pages.

Pure host logic.  Pages and slots are reused in LIFO order (the most recently freed first), so a
short-lived request's pages are the next request's — stale contents are the normal case and the model
code must never read a row it has not written for the sequence at hand.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


class OutOfPages(RuntimeError):
    pass


class OutOfStateSlots(RuntimeError):
    pass


class FreeList:
    """LIFO pool of integer handles 0..n-1."""

    def __init__(self, n: int):
        self.capacity = int(n)
        self._free = list(range(self.capacity - 1, -1, -1))
        self._used = set()

    def take(self) -> int:
        if not self._free:
            raise IndexError("pool is empty")
        h = self._free.pop()
        self._used.add(h)
        return h

    def give_back(self, h: int) -> None:
        if h not in self._used:
            raise ValueError(f"handle {h} is not in use")
        self._used.remove(h)
        self._free.append(h)

    @property
    def num_free(self) -> int:
        return len(self._free)


@dataclass
class SequenceCache:
    """What one live sequence holds."""
    block_table: List[int] = field(default_factory=list)
    state_slot: Optional[int] = None
    num_tokens: int = 0            # tokens whose keys / values / state are in the cache


class CacheManager:
    """Pages + state slots for the live sequences of one engine."""

    def __init__(self, num_blocks: int, block_size: int, num_state_slots: int = 0):
        if block_size <= 0 or num_blocks <= 0:
            raise ValueError("block_size and num_blocks must be positive")
        self.block_size = int(block_size)
        self.blocks = FreeList(num_blocks)
        self.state_slots = FreeList(num_state_slots)
        self.needs_state = num_state_slots > 0
        self._seqs: Dict[str, SequenceCache] = {}

    # ---- queries ----
    def blocks_needed(self, seq_id: str, new_total_tokens: int) -> int:
        have = len(self._seqs[seq_id].block_table) if seq_id in self._seqs else 0
        return max(0, -(-new_total_tokens // self.block_size) - have)

    def can_admit(self, first_chunk_tokens: int) -> bool:
        if self.needs_state and self.state_slots.num_free == 0:
            return False
        return -(-first_chunk_tokens // self.block_size) <= self.blocks.num_free

    def can_grow(self, seq_id: str, new_total_tokens: int) -> bool:
        return self.blocks_needed(seq_id, new_total_tokens) <= self.blocks.num_free

    def __contains__(self, seq_id: str) -> bool:
        return seq_id in self._seqs

    def get(self, seq_id: str) -> SequenceCache:
        return self._seqs[seq_id]

    @property
    def live(self) -> int:
        return len(self._seqs)

    # ---- transitions ----
    def admit(self, seq_id: str) -> SequenceCache:
        if seq_id in self._seqs:
            raise ValueError(f"sequence {seq_id} is already live")
        sc = SequenceCache()
        if self.needs_state:
            if self.state_slots.num_free == 0:
                raise OutOfStateSlots(f"no state slot for sequence {seq_id} ({self.state_slots.capacity} in use)")
            sc.state_slot = self.state_slots.take()
        self._seqs[seq_id] = sc
        return sc

    def grow(self, seq_id: str, new_total_tokens: int) -> SequenceCache:
        """Make room for the sequence's first `new_total_tokens` tokens (all-or-nothing)."""
        sc = self._seqs[seq_id]
        need = self.blocks_needed(seq_id, new_total_tokens)
        if need > self.blocks.num_free:
            raise OutOfPages(f"sequence {seq_id} needs {need} more pages, {self.blocks.num_free} free")
        for _ in range(need):
            sc.block_table.append(self.blocks.take())
        return sc

    def commit(self, seq_id: str, new_total_tokens: int) -> None:
        self._seqs[seq_id].num_tokens = int(new_total_tokens)

    def free(self, seq_id: str) -> None:
        sc = self._seqs.pop(seq_id)
        for b in reversed(sc.block_table):
            self.blocks.give_back(b)
        if sc.state_slot is not None:
            self.state_slots.give_back(sc.state_slot)
