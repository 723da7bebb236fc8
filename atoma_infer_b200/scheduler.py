"""Continuous-batching scheduler with chunked prefill.

The reference's scheduler (backends/vllm/src/scheduler.rs: `Scheduler::schedule_chunked_prefill`, the
`SchedulingBudget` of max_num_batched_tokens / max_num_sequences, policy FCFS, preemption by recompute)
decides per step which sequences run and how many tokens of each.  This is the same decision for one
device: running sequences first (a decoded token each, or the next portion of a prompt that is still
being prefilled), then waiting ones while the token budget, the page pool and the state slots last.
A step is therefore a MIXED batch: portions of prompts beside single decoded tokens.

`plan_forced` takes the step's composition from the caller (a trace replay, a test) and makes the
same allocations through the same cache manager — nothing else differs from a scheduled step.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Iterable, List, Optional, Sequence as Seq_, Tuple

from .cache import CacheManager, OutOfPages


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    stop_token_ids: Tuple[int, ...] = ()
    greedy: bool = True


@dataclass
class Sequence:
    seq_id: str
    tokens: List[int]                       # prompt + generated so far
    prompt_len: int
    params: SamplingParams = field(default_factory=SamplingParams)
    num_computed: int = 0                   # tokens already run through the model (in cache / state)
    finished: bool = False
    arrival: int = 0

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.num_computed


@dataclass
class ScheduledChunk:
    seq: Sequence
    start: int                              # position of the chunk's first token
    count: int
    want: Tuple[int, ...] = ()              # offsets inside the chunk whose logits are wanted
    block_table: Seq_[int] = ()
    state_slot: Optional[int] = None

    @property
    def is_decode(self) -> bool:
        return self.count == 1 and self.start > 0 and self.start >= self.seq.prompt_len


@dataclass
class StepPlan:
    chunks: List[ScheduledChunk]
    preempted: List[str] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(c.count for c in self.chunks)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_batched_tokens: int = 2048, max_num_seqs: int = 64):
        self.cache = cache
        self.max_tokens = int(max_num_batched_tokens)
        self.max_seqs = int(max_num_seqs)
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self._clock = 0

    # ---- queue ----
    def add(self, seq: Sequence) -> None:
        self._clock += 1
        seq.arrival = self._clock
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def finish(self, seq: Sequence) -> None:
        seq.finished = True
        if seq in self.running:
            self.running.remove(seq)
        if seq.seq_id in self.cache:
            self.cache.free(seq.seq_id)

    def _preempt_one(self, keep: Sequence) -> Optional[Sequence]:
        """Recompute-preemption: the youngest running sequence gives its pages and state back and waits again."""
        victims = [s for s in self.running if s is not keep]
        if not victims:
            return None
        v = max(victims, key=lambda s: s.arrival)
        self.running.remove(v)
        self.cache.free(v.seq_id)
        v.num_computed = 0
        self.waiting.appendleft(v)
        return v

    def _chunk(self, seq: Sequence, count: int, want_last: bool) -> ScheduledChunk:
        sc = self.cache.grow(seq.seq_id, seq.num_computed + count)
        return ScheduledChunk(seq, seq.num_computed, count, (count - 1,) if want_last else (), tuple(sc.block_table), sc.state_slot)

    # ---- policy ----
    def plan(self) -> StepPlan:
        budget = self.max_tokens
        chunks: List[ScheduledChunk] = []
        preempted: List[str] = []
        # running sequences, oldest first: decodes cost one token, unfinished prompts take what is left
        for seq in sorted(self.running, key=lambda s: s.arrival):
            if seq not in self.running or budget <= 0:
                continue
            count = min(seq.pending, budget)
            while not self.cache.can_grow(seq.seq_id, seq.num_computed + count):
                v = self._preempt_one(seq)
                if v is None:
                    break
                preempted.append(v.seq_id)
                chunks = [c for c in chunks if c.seq is not v]
            if not self.cache.can_grow(seq.seq_id, seq.num_computed + count):
                continue
            chunks.append(self._chunk(seq, count, seq.num_computed + count == len(seq.tokens)))
            budget -= count
        # admissions
        while self.waiting and budget > 0 and len(self.running) < self.max_seqs:
            seq = self.waiting[0]
            if seq.seq_id in preempted:
                break
            count = min(seq.pending, budget)
            if not self.cache.can_admit(count):
                break
            self.waiting.popleft()
            self.cache.admit(seq.seq_id)
            self.running.append(seq)
            chunks.append(self._chunk(seq, count, count == len(seq.tokens)))
            budget -= count
        return StepPlan(chunks, preempted)

    # ---- caller-given composition ----
    def plan_forced(self, entries: Iterable[Tuple[Sequence, int, Seq_[int]]]) -> StepPlan:
        """entries: (sequence, token count, wanted offsets).  A sequence is admitted at its first entry."""
        chunks: List[ScheduledChunk] = []
        for seq, count, want in entries:
            if count <= 0 or count > seq.pending:
                raise ValueError(f"sequence {seq.seq_id}: {count} tokens asked, {seq.pending} pending")
            if seq.seq_id not in self.cache:
                if seq in self.waiting:
                    self.waiting.remove(seq)
                self.cache.admit(seq.seq_id)
                self.running.append(seq)
            try:
                sc = self.cache.grow(seq.seq_id, seq.num_computed + count)
            except OutOfPages:
                raise
            chunks.append(ScheduledChunk(seq, seq.num_computed, count, tuple(int(w) for w in want), tuple(sc.block_table),
                                         sc.state_slot))
        return StepPlan(chunks)

    def commit(self, plan: StepPlan) -> None:
        """The step ran: its tokens are in the cache / state."""
        for c in plan.chunks:
            c.seq.num_computed = c.start + c.count
            self.cache.commit(c.seq.seq_id, c.seq.num_computed)
