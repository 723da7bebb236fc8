"""The serving engine: requests in, scheduled mixed batches through the model's step function, tokens out.

The reference's `LlmEngine::step` (backends/vllm/src/llm_engine.rs) asks the scheduler for the step's
sequence groups, hands them to the model executor, samples, and appends the new tokens; this is the
same loop for one device.  `step()` runs whatever the scheduler plans; `step_forced()` runs a
composition given by the caller (trace replay, tests) through the same cache manager, executor and
sampling.  Sampling is greedy on the device (the step's last kernel).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence as Seq_, Tuple

import torch

from . import checkpoint, models
from .cache import CacheManager
from .models import CacheConfig
from .ops import AtomaError
from .scheduler import SamplingParams, Scheduler, Sequence, StepPlan


@dataclass
class RequestOutput:
    seq_id: str
    new_token: Optional[int]
    finished: bool
    generated: List[int] = field(default_factory=list)


class Engine:
    def __init__(self, executor, cache: CacheManager, max_num_batched_tokens: int = 2048, max_num_seqs: int = 64):
        self.executor = executor
        self.cache = cache
        self.scheduler = Scheduler(cache, max_num_batched_tokens, max_num_seqs)
        self.sequences: Dict[str, Sequence] = {}
        self._auto = 0

    @classmethod
    def from_model_dir(cls, model_dir, dtype=torch.bfloat16, device="cuda:0", max_tokens: int = 8192, block_size: int = 16,
                       max_live_requests: int = 4, max_num_batched_tokens: int = 2048) -> "Engine":
        """`max_tokens`: the most tokens live requests hold at any time (the page pool is made for that many)."""
        cfg = checkpoint.read_config(model_dir)
        entry = models.resolve(cfg)
        needs_state = entry.needs_state(cfg)
        num_blocks = -(-int(max_tokens) // block_size) + max_live_requests   # a partly filled last page per request
        cc = CacheConfig(num_blocks=num_blocks, block_size=block_size, num_state_slots=max_live_requests if needs_state else 0)
        executor = entry.build(cfg, checkpoint.open_checkpoint(model_dir), dtype, device, cc)
        cache = CacheManager(cc.num_blocks, cc.block_size, cc.num_state_slots)
        return cls(executor, cache, max_num_batched_tokens, max_live_requests)

    # ---- requests ----
    def add_request(self, prompt: Seq_[int], params: Optional[SamplingParams] = None, seq_id: Optional[str] = None) -> str:
        if seq_id is None:
            self._auto += 1
            seq_id = f"req-{self._auto}"
        if seq_id in self.sequences:
            raise AtomaError(f"request {seq_id} already exists")
        if not len(prompt):
            raise AtomaError("empty prompts are not accepted")
        seq = Sequence(seq_id, [int(t) for t in prompt], len(prompt), params or SamplingParams())
        self.sequences[seq_id] = seq
        self.scheduler.add(seq)
        return seq_id

    def finish_request(self, seq_id: str) -> None:
        """Ends a request and gives its pages and state slot back."""
        seq = self.sequences.pop(seq_id)
        if seq in self.scheduler.waiting:
            self.scheduler.waiting.remove(seq)
        self.scheduler.finish(seq)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # ---- steps ----
    def _run(self, plan: StepPlan, **kw):
        out = self.executor.execute(plan, **kw)
        self.scheduler.commit(plan)
        return out

    def step(self) -> List[RequestOutput]:
        """One scheduled step; sampled tokens are appended to their sequences."""
        plan = self.scheduler.plan()
        if not plan.chunks:
            if self.scheduler.has_work():
                raise AtomaError("nothing can be scheduled: the page pool or the state slots are too small for the next request")
            return []
        out = self._run(plan)
        results: List[RequestOutput] = []
        if out.next_tokens is not None:
            toks = out.next_tokens.cpu().tolist()      # the step's one device-to-host read
            for (seq_id, _), tok in zip(out.rows, toks):
                seq = self.sequences[seq_id]
                seq.tokens.append(int(tok))
                done = len(seq.generated) >= seq.params.max_new_tokens or int(tok) in seq.params.stop_token_ids
                results.append(RequestOutput(seq_id, int(tok), done, list(seq.generated)))
                if done:
                    self.finish_request(seq_id)
        return results

    def step_forced(self, entries: Iterable[Tuple[str, Seq_[int], Seq_[int]]], end: Iterable[str] = (), **kw):
        """Runs the given composition: per entry a request id, its NEXT tokens and the offsets among them whose
        logits are wanted.  Unknown ids are admitted.  Nothing is sampled or appended; returns the executor's
        StepOutput (logits rows in the order of the entries and their wanted offsets)."""
        forced = []
        for seq_id, tokens, want in entries:
            seq = self.sequences.get(seq_id)
            if seq is None:
                seq = Sequence(seq_id, [], 0)
                self.sequences[seq_id] = seq
            if seq.pending:
                raise AtomaError(f"request {seq_id} has tokens that were never run")
            seq.tokens.extend(int(t) for t in tokens)
            seq.prompt_len = len(seq.tokens)
            forced.append((seq, len(tokens), want))
        plan = self.scheduler.plan_forced(forced)
        out = self._run(plan, **kw)
        for seq_id in end:
            if seq_id in self.sequences:
                self.finish_request(seq_id)
        return out

    def generate(self, prompts: Seq_[Seq_[int]], max_new_tokens: int = 16, stop_token_ids: Tuple[int, ...] = ()) -> List[List[int]]:
        """Greedy continuation of every prompt, through the scheduler (continuous batching)."""
        ids = [self.add_request(p, SamplingParams(max_new_tokens, tuple(stop_token_ids))) for p in prompts]
        done: Dict[str, List[int]] = {}
        while self.has_unfinished():
            for r in self.step():
                if r.finished:
                    done[r.seq_id] = r.generated
        return [done[i] for i in ids]
