"""Iteration-level scheduler: which requests run in the next engine step, and how many tokens each.

Same public surface and the same decisions as the reference scheduler (nanoserve/scheduler.py:25-200):
`SeqStatus`, `Sequence`, `SchedulerOutput`, `Scheduler.add / finish / abort / schedule / has_unfinished`,
the `waiting` deque, the `running` list and `num_preemptions`. The decisions are pure integer logic and are
checked step by step against traces recorded from the reference (tests/golden/).

Rules (reference file:line in brackets):
  * policy "continuous" admits at every step, "static" only between batches, once the batch is full or the
    oldest request waited batch_wait_s [scheduler.py:153-159];
  * before anything else every running request gets room for one more token; when the pool is out of blocks
    the most recently admitted request is preempted (KV freed, outputs kept, back to the FRONT of the queue)
    until the rest fit [scheduler.py:128-148];
  * budget order: running decodes (1 token each, always) -> running partial prefills (min(remaining, budget)
    with chunked prefill) -> FCFS admissions while a seat is free, budget is left (chunked) or the whole
    prompt fits (unchunked), and the KV manager accepts the head of the queue; nobody overtakes the head
    [scheduler.py:161-200].
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field


class SeqStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)
class Sequence:
    """One request inside the engine [scheduler.py:31-77]."""
    seq_id: int
    prompt_ids: list[int]
    max_new_tokens: int
    ignore_eos: bool = False
    arrival_time: float = 0.0
    output_ids: list[int] = field(default_factory=list)
    status: SeqStatus = SeqStatus.WAITING
    cache: object | None = None          # unused here (contiguous cache of the reference's early milestones)
    block_table: object | None = None    # BlockTable, set on admission
    num_cached: int = 0                  # tokens whose K/V are stored; 0 => must (re)prefill
    sampling: object | None = None       # None = greedy
    seed: int = 0
    seat: int = -1                       # row of the device block-table mirror while admitted (not in the reference)
    token_on_device: bool = False        # the newest output token is in the device's last_tokens[seat]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def remaining(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids) - self.num_cached

    @property
    def is_prefill(self) -> bool:
        # nothing cached yet (new or preempted), or part-way through a chunked prefill [scheduler.py:56-60]
        # (written out: this runs for every running sequence in every step)
        return self.num_cached == 0 or len(self.prompt_ids) + len(self.output_ids) - self.num_cached > 1

    @property
    def step_cost(self) -> int:
        return self.remaining

    def token_at(self, pos: int) -> int:
        n = len(self.prompt_ids)
        return self.prompt_ids[pos] if pos < n else self.output_ids[pos - n]

    def step_tokens(self, n: int | None = None) -> tuple[list[int], list[int]]:
        """(token ids, positions) of the next n uncached tokens (default: all) [scheduler.py:62-73]."""
        start = self.num_cached
        count = self.remaining if n is None else n
        if count == 1 and self.remaining == 1 and self.output_ids:
            return [self.output_ids[-1]], [self.num_tokens - 1]
        stop = start + count
        n_prompt = len(self.prompt_ids)
        if stop <= n_prompt:
            toks = self.prompt_ids[start:stop]
        elif start >= n_prompt:
            toks = self.output_ids[start - n_prompt:stop - n_prompt]
        else:
            toks = self.prompt_ids[start:] + self.output_ids[:stop - n_prompt]
        return toks, list(range(start, start + len(toks)))


@dataclass
class SchedulerOutput:
    scheduled: list[Sequence]                 # batch order: decodes, partial prefills, new admissions
    admitted: list[Sequence]                  # newly admitted this step
    chunks: list[int] = field(default_factory=list)   # tokens each scheduled sequence feeds this step


class Scheduler:
    def __init__(self, policy: str = "continuous", max_num_seqs: int = 8, max_num_batched_tokens: int = 8192,
                 batch_wait_s: float = 0.02, kv=None, chunked_prefill: bool = False):
        if policy not in ("static", "continuous"):
            raise ValueError(f"unknown policy {policy!r}")
        self.policy = policy
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.batch_wait_s = batch_wait_s
        self.kv = kv
        self.chunked_prefill = chunked_prefill
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    # ---- queue management ------------------------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        n_prompt = len(seq.prompt_ids)
        if not self.chunked_prefill and n_prompt > self.max_num_batched_tokens:
            raise ValueError(f"prompt of {n_prompt} tokens exceeds the per-step token budget "
                             f"({self.max_num_batched_tokens}) and chunked prefill is off")
        worst = n_prompt + seq.max_new_tokens
        if self.kv is not None and not self.kv.can_ever_fit(worst):
            raise ValueError(f"request needs up to {worst} tokens of KV, more than the whole KV budget: "
                             f"it could never finish")
        seq.status = SeqStatus.WAITING
        self.waiting.append(seq)

    def finish(self, seq: Sequence) -> None:
        seq.status = SeqStatus.FINISHED
        self.running.remove(seq)
        if self.kv is not None:
            self.kv.free(seq)

    def abort(self, seq: Sequence) -> None:
        if seq in self.running:
            self.finish(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
            seq.status = SeqStatus.FINISHED

    def has_unfinished(self) -> bool:
        return bool(self.running) or bool(self.waiting)

    # ---- one scheduling decision -----------------------------------------------------------------------
    def _evict_newest(self) -> None:
        victim = self.running.pop()
        self.kv.free(victim)
        victim.num_cached = 0
        victim.status = SeqStatus.WAITING
        self.waiting.appendleft(victim)
        self.num_preemptions += 1

    def _make_room_for_decodes(self) -> None:
        idx = 0
        while idx < len(self.running):
            if self.kv.try_append(self.running[idx]):
                idx += 1
            else:
                self._evict_newest()      # may evict running[idx] itself; the loop condition then ends or moves on

    def _admission_open(self, now: float) -> bool:
        if self.policy == "continuous":
            return True
        if self.running or not self.waiting:
            return False
        return len(self.waiting) >= self.max_num_seqs or now - self.waiting[0].arrival_time >= self.batch_wait_s

    def schedule(self, now: float) -> SchedulerOutput:
        if self.kv is not None:
            self._make_room_for_decodes()
        budget = self.max_num_batched_tokens
        decodes: list[Sequence] = []
        partial: list[Sequence] = []
        for s in self.running:
            (partial if s.is_prefill else decodes).append(s)
        scheduled: list[Sequence] = list(decodes)
        chunks: list[int] = [1] * len(decodes)
        budget -= len(decodes)
        for seq in partial:
            n = min(seq.remaining, budget) if self.chunked_prefill else seq.remaining
            if n > 0:
                scheduled.append(seq)
                chunks.append(n)
                budget -= n
        admitted: list[Sequence] = []
        if self._admission_open(now):
            seats_left = self.max_num_seqs - len(self.running)
            while self.waiting and len(admitted) < seats_left:
                head = self.waiting[0]
                if self.chunked_prefill:
                    if budget <= 0:
                        break
                elif head.step_cost > budget:
                    break
                if self.kv is not None and not self.kv.can_admit(head):
                    break
                self.waiting.popleft()
                if self.kv is not None:
                    self.kv.admit(head)          # a prefix-cache hit moves num_cached ahead: size the chunk after
                n = min(head.step_cost, budget) if self.chunked_prefill else head.step_cost
                budget -= n
                head.status = SeqStatus.RUNNING
                admitted.append(head)
                scheduled.append(head)
                chunks.append(n)
            self.running.extend(admitted)
        return SchedulerOutput(scheduled=scheduled, admitted=admitted, chunks=chunks)
