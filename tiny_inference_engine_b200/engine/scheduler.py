"""Continuous batching: which requests run in a step and how many of their pending tokens.

The rules are those of the reference's BatchScheduler (src/engine/batch_scheduler.cpp:78-174); the
code is built around what this engine schedules over: a cache manager with several page groups of
different sizes, state slots that are a resource like pages, and steps decided while the one before
is still on the GPU. A decision is a `_Draft` that four passes fill in turn:

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

When pages (or state slots) run out, a request is preempted BY RECOMPUTE: its pages and state slot
go back, its tokens (prompt and generated) stay, and it is prefilled again later
(src/engine/batch_scheduler.cpp:67-76). A waiting request holds neither pages nor a slot; both are
taken when it is admitted, by the same all-or-nothing `CacheManager.reserve`. An older request is
never preempted for a newer one.
The scheduler owns pages while requests run: every (request, n) it returns already has
pages reserved for num_computed + n tokens. Deciding a step (`schedule`) is separate from
finishing it (`complete` / `abandon`); requests of a batch that is neither are skipped by the next
decision. The engine calls `complete` as soon as a step is queued when it decides the next one while that
step is still on the GPU: the requests' bookkeeping is then already past it.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.manager import CacheManager
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


class _Draft:
    """A step while it is being decided: what has been granted and what is left of the step's limits."""

    def __init__(self, number: int, tokens: int, seqs: int):
        self.batch = ScheduledBatch(id=number)
        self.tokens_left = tokens
        self.seq_limit = seqs
        self.evicted: set[int] = set()      # requests preempted while this step was decided

    @property
    def closed(self) -> bool:
        return self.tokens_left == 0 or len(self.batch.seqs) == self.seq_limit


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
        smallest = min((p.num_blocks for p in cache.pools), default=cache.num_pages)
        if wm < -1 or wm >= smallest:
            raise InvalidArgument(f"watermark of {wm} pages must be -1 (auto) or below the pool's {smallest} pages")
        # pages that admission leaves free, per group (src/engine/batch_scheduler.cpp:15-23: 1 % of the pool)
        self._margins = [wm if wm >= 0 else max(1, p.num_blocks // 100) for p in cache.pools]
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

    def _priority(self, s: Sequence):
        """Admission order (src/engine/batch_scheduler.cpp:31-40): arrival, or least pending work made
        smaller by `aging` for every step waited; ties by arrival, then id."""
        waited = self.step_no - s.waiting_since_step
        score = s.num_pending - self.config.aging * waited if self.config.policy == "srpt-aging" else 0
        return (score, s.waiting_since_step, s.id)

    def _room(self, seq: Sequence, want: int) -> int:
        """How many of `want` tokens `seq` can run next with what it holds plus what is free."""
        return max(0, min(want, self.cache.room(seq.cache, seq.num_computed)))

    def _evict(self, seq: Sequence, draft: _Draft) -> None:
        self.cache.reset(seq.cache)
        seq.num_computed = 0
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(seq)
        self.add(seq)
        draft.evicted.add(seq.id)

    def _make_room(self, seq: Sequence, want: int, draft: _Draft) -> int:
        """Preempts, newest first, idle requests admitted after `seq` that hold a page or a state slot, until
        some of `want` tokens of `seq` fit or no such request is left. Returns how many fit."""
        fit = self._room(seq, want)
        while fit == 0:
            behind = self.running[self.running.index(seq) + 1:]
            victim = next((s for s in reversed(behind) if not self._busy(s) and self.cache.holds(s.cache)), None)
            if victim is None:
                break
            self._evict(victim, draft)
            fit = self._room(seq, want)
        return fit

    def _grant(self, draft: _Draft, seq: Sequence, n: int) -> None:
        if not self.cache.reserve(seq.cache, seq.num_computed + n):
            raise InvalidArgument(f"sequence {seq.id}: {n} more tokens were counted as fitting, "
                                  f"but their pages could not be reserved")
        draft.batch.seqs.append((seq, n))
        draft.tokens_left -= n

    # -- one decision
    def schedule(self) -> ScheduledBatch:
        self.step_no += 1
        draft = _Draft(self._next_batch, self.config.serving.max_tokens_per_step, self.config.serving.max_seqs)
        self._next_batch += 1
        self._decode_pass(draft)
        self._prompt_pass(draft)
        self._admission_pass(draft)
        if draft.batch.empty():
            self._rescue_pass(draft)
        self._in_flight.update(seq.id for seq, _ in draft.batch.seqs)
        return draft.batch

    def _decode_pass(self, draft: _Draft) -> None:
        """Rule 1. The candidates are fixed up front; one that an older candidate preempted is passed over."""
        for seq in [s for s in self.running if s.num_pending == 1 and not self._busy(s)]:
            if draft.closed:
                return
            if seq.id in draft.evicted:
                continue
            if self._make_room(seq, 1, draft):
                self._grant(draft, seq, 1)
            elif any(self._busy(s) for s in self.running[self.running.index(seq) + 1:]):
                pass        # a newer request is on the GPU: what it holds can be had in the next decision
            else:
                self._evict(seq, draft)

    def _prompt_pass(self, draft: _Draft) -> None:
        """Rule 2."""
        for seq in self.running:
            if draft.closed:
                return
            if seq.num_pending > 1 and not self._busy(seq):
                n = self._room(seq, min(seq.num_pending, draft.tokens_left))
                if n:
                    self._grant(draft, seq, n)

    def _admission_pass(self, draft: _Draft) -> None:
        """Rule 3. Whether a portion fits is asked of every page group and of the state slots at once."""
        self.waiting.sort(key=self._priority)
        nothing_kept = [0] * len(self._margins)
        for seq in list(self.waiting):
            if draft.closed or len(self.running) >= draft.seq_limit:
                return
            if seq.id in draft.evicted:
                continue
            n = min(seq.num_pending, draft.tokens_left)
            if not self.cache.admits(n, self._margins if self.running else nothing_kept):
                return
            self.waiting.remove(seq)
            self.running.append(seq)
            seq.state = SeqState.PREFILLING
            self._grant(draft, seq, n)

    def _rescue_pass(self, draft: _Draft) -> None:
        """Rule 4: the oldest request that is not on the GPU takes what it can, at the cost of newer ones."""
        seq = next((s for s in self.running if not self._busy(s)), None)
        if seq is None:
            return
        n = self._make_room(seq, min(seq.num_pending, draft.tokens_left), draft)
        if n:
            self._grant(draft, seq, n)

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
