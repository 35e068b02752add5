"""Continuous batching: which requests run in a step and how many of their pending tokens.

The decisions are the reference's BatchScheduler (src/engine/batch_scheduler.cpp:78-174),
restated over this engine's cache manager (several page groups, state slots):

  1. every running request with exactly one pending token decodes, oldest first; one that
     needs a page when none is free preempts the NEWEST request admitted after it that is
     idle and holds pages; if there is none but a newer one is in flight it waits this
     step; only then does it preempt itself;
  2. running requests in the middle of a prompt continue, in admission order, with as many
     tokens as the budget and the free pages allow;
  3. waiting requests are admitted in policy order while `free - pages(chunk) >= watermark`
     (no watermark when nothing runs); admission stops at the first that does not fit, and
     a request preempted in this very step sits one step out;
  4. if nothing could run, the oldest running request preempts newer ones until it can
     take a portion (the engine never stalls).

When pages run out, a request is preempted BY RECOMPUTE: its pages and state go back, its
tokens (prompt and generated) stay, and it is prefilled again later
(src/engine/batch_scheduler.cpp:67-76). An older request is never preempted for a newer one.
The scheduler owns pages while requests run: every (request, n) it returns already has
pages reserved for num_computed + n tokens. Deciding a step (`schedule`) is separate from
finishing it (`complete` / `abandon`); requests of a batch that is neither are skipped by the next
decision. The engine calls `complete` as soon as a step is queued when it decides the next one while that
step is still on the GPU: the requests' bookkeeping is then already past it.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.manager import CacheManager, blocks_for
from ..errors import InvalidArgument
from .sequence import SeqState, Sequence


@dataclass
class ServingConfig:
    """The shape of one step, shared by step function, scheduler and engine
    (src/engine/serving_config.h:12-22)."""
    max_tokens_per_step: int = 512
    max_seqs: int = 64
    run_ahead: bool = True      # decide and queue the next step before the host has seen this one's tokens

    def validate(self) -> None:
        if self.max_tokens_per_step <= 0:
            raise InvalidArgument(f"max_tokens_per_step must be positive, got {self.max_tokens_per_step}")
        if self.max_seqs <= 0:
            raise InvalidArgument(f"max_seqs must be positive, got {self.max_seqs}")
        if self.max_seqs > self.max_tokens_per_step:
            raise InvalidArgument(f"max_seqs ({self.max_seqs}) cannot exceed max_tokens_per_step "
                                  f"({self.max_tokens_per_step}): every sequence must decode each step")


POLICIES = ("fcfs", "srpt-aging")


@dataclass
class SchedulerConfig:
    serving: ServingConfig = field(default_factory=ServingConfig)
    policy: str = "srpt-aging"     # "fcfs": by arrival; "srpt-aging": least remaining prefill first, minus aging per step waited
    aging: int = 16
    watermark_pages: int = -1      # pages admission leaves free; -1 = max(1, 1% of the pool)


@dataclass
class ScheduledBatch:
    id: int = 0
    seqs: list[tuple[Sequence, int]] = field(default_factory=list)

    def empty(self) -> bool:
        return not self.seqs


class Scheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig | None = None):
        self.cache = cache
        self.config = config or SchedulerConfig()
        self.config.serving.validate()
        if self.config.policy not in POLICIES:
            raise InvalidArgument(f"scheduling policy must be fcfs or srpt-aging, got '{self.config.policy}'")
        if self.config.aging < 0:
            raise InvalidArgument(f"aging must be non-negative, got {self.config.aging}")
        wm = self.config.watermark_pages
        if wm < -1 or wm >= cache.num_pages:
            raise InvalidArgument(f"watermark of {wm} pages must be -1 (auto) or below the pool's {cache.num_pages} pages")
        self.watermark = wm if wm >= 0 else max(1, cache.num_pages // 100)
        self.waiting: list[Sequence] = []
        self.running: list[Sequence] = []     # admission order, oldest first
        self._in_flight: set[int] = set()
        self.step_no = 0
        self._next_batch = 1
        self.num_preemptions = 0

    # -- queue
    def add(self, seq: Sequence) -> None:
        seq.state = SeqState.WAITING
        seq.waiting_since_step = self.step_no
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _busy(self, seq: Sequence) -> bool:
        return seq.id in self._in_flight

    def _order_key(self, s: Sequence):
        if self.config.policy == "srpt-aging":
            return (s.num_pending - self.config.aging * (self.step_no - s.waiting_since_step), s.waiting_since_step, s.id)
        return (0, s.waiting_since_step, s.id)

    def _fit(self, seq: Sequence, want: int) -> int:
        """The most of `want` tokens `seq` can run next with the pages it holds plus the free ones."""
        return max(0, min(want, self.cache.room(seq.cache, seq.num_computed)))

    def _holds_pages(self, seq: Sequence) -> bool:
        return any(len(t) > t.released for t in seq.cache.tables)

    def _newest_after(self, index: int):
        for j in range(len(self.running) - 1, index, -1):
            s = self.running[j]
            if not self._busy(s) and self._holds_pages(s):
                return s
        return None

    def _newer_busy(self, index: int) -> bool:
        return any(self._busy(s) for s in self.running[index + 1:])

    def _preempt(self, seq: Sequence) -> None:
        self.cache.reset(seq.cache)
        seq.num_computed = 0
        seq.state = SeqState.WAITING
        seq.waiting_since_step = self.step_no
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(seq)
        self.waiting.append(seq)

    # -- one decision
    def schedule(self) -> ScheduledBatch:
        self.step_no += 1
        batch = ScheduledBatch(id=self._next_batch)
        self._next_batch += 1
        budget = self.config.serving.max_tokens_per_step
        max_seqs = self.config.serving.max_seqs
        page = self.cache.page_size

        def full() -> bool:
            return budget == 0 or len(batch.seqs) == max_seqs

        def take(seq: Sequence, n: int) -> None:
            nonlocal budget
            if not self.cache.reserve(seq.cache, seq.num_computed + n):
                raise InvalidArgument(f"scheduler bug: {n} tokens of sequence {seq.id} do not fit the pages it counted")
            batch.seqs.append((seq, n))
            budget -= n

        # 1. decodes, oldest first
        i = 0
        while i < len(self.running) and not full():
            seq = self.running[i]
            if self._busy(seq) or seq.num_pending != 1:
                i += 1
                continue
            preempted_self = deferred = False
            while self._fit(seq, 1) == 0:
                victim = self._newest_after(i)
                if victim is None and self._newer_busy(i):
                    deferred = True
                    break
                self._preempt(victim if victim is not None else seq)
                if victim is None:
                    preempted_self = True
                    break
            if deferred:
                i += 1
                continue
            if preempted_self:
                continue  # running[i] is now the next sequence
            take(seq, 1)
            i += 1

        # 2. prompts in progress
        for seq in self.running:
            if full():
                break
            if self._busy(seq) or seq.num_pending <= 1:
                continue
            n = self._fit(seq, min(seq.num_pending, budget))
            if n > 0:
                take(seq, n)

        # 3. admission in policy order
        self.waiting.sort(key=self._order_key)
        admitted = []
        for seq in self.waiting:
            if full() or len(self.running) >= max_seqs:
                break
            if seq.num_preemptions > 0 and seq.waiting_since_step == self.step_no:
                continue
            n = min(seq.num_pending, budget)
            keep_free = self.watermark if self.running else 0
            if self.cache.min_free() - blocks_for(n, page) < keep_free:
                break
            seq.state = SeqState.PREFILLING
            self.running.append(seq)
            take(seq, n)
            admitted.append(seq)
        if admitted:
            ids = {s.id for s in admitted}
            self.waiting = [s for s in self.waiting if s.id not in ids]

        # 4. never stall
        if batch.empty():
            for i, seq in enumerate(self.running):
                if self._busy(seq):
                    continue
                want = min(seq.num_pending, budget)
                while self._fit(seq, want) == 0:
                    victim = self._newest_after(i)
                    if victim is None:
                        break
                    self._preempt(victim)
                n = self._fit(seq, want)
                if n > 0:
                    take(seq, n)
                break

        for seq, _ in batch.seqs:
            self._in_flight.add(seq.id)
        return batch

    def complete(self, batch: ScheduledBatch) -> None:
        """The engine advanced num_computed of every sequence of the batch (when the step's tokens are back, or,
        to decide the next step while this one is still on the GPU, as soon as it is queued)."""
        for seq, _ in batch.seqs:
            self._in_flight.discard(seq.id)

    def abandon(self, batch: ScheduledBatch) -> None:
        """The step failed; tables were trimmed back to num_computed."""
        for seq, _ in batch.seqs:
            self._in_flight.discard(seq.id)

    def requeue(self, seq: Sequence) -> None:
        """The engine gave the request's pages back and set num_computed to 0 after a failed step: it waits
        again, wherever it was (running, waiting, or already taken out because its last token was in flight)."""
        if seq in self.running:
            self.running.remove(seq)
        if seq not in self.waiting:
            self.waiting.append(seq)
        seq.state = SeqState.WAITING
        seq.waiting_since_step = self.step_no
        self._in_flight.discard(seq.id)

    def finish(self, seq: Sequence) -> None:
        """Done or cancelled: forget it."""
        if seq in self.waiting:
            self.waiting.remove(seq)
        if seq in self.running:
            self.running.remove(seq)
        self._in_flight.discard(seq.id)
