"""The engine: admits requests, asks the scheduler for a batch, runs the step function, samples, finishes.

The Python entry point follows the reference's Engine (src/engine/engine.h:18-86,
src/engine/engine.cpp:11-235): add_request, step, generate, cancel, release, stats,
set_token_callback, with the same meanings, errors and finish reasons.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Sequence as Seq

from ..cache.manager import CacheManager, blocks_for
from ..cache.state_slots import StateSlots
from ..errors import CapacityError, InvalidArgument
from ..sampling.params import SamplingParams
from .scheduler import ScheduledBatch, Scheduler, SchedulerConfig, ServingConfig
from .sequence import FinishReason, SeqState, Sequence
from .step import StepEntry, StepRunner


@dataclass
class EngineStats:
    steps: int = 0
    seqs_scheduled: int = 0    # summed over steps; divided by steps it is the mean batch size
    prefill_tokens: int = 0    # prompt tokens, and tokens recomputed after preemption
    decode_tokens: int = 0
    step_seconds: float = 0.0  # time in the step function and sampling
    preemptions: int = 0
    steps_ahead: int = 0       # steps queued before the tokens of the step ahead of them were read


PLACEHOLDER = -1      # stands in a request's tokens for the one that a step in flight is sampling
UNSAMPLABLE = -2      # what the sampling kernels answer for a row with a NaN or with nothing finite (csrc/sampling.cu)


@dataclass
class _Pending:
    """A step on the GPU whose tokens have not been read yet."""
    batch: ScheduledBatch
    sampled: list            # the requests that get a token from this step, in the order of its sampled rows
    tokens: object           # StepRunner.fetch's handle
    prefill: int
    decode: int
    advanced: bool = False   # the requests' bookkeeping is already past this step (a step was decided behind it)
    token_at: dict = field(default_factory=dict)   # request id -> where in its tokens the placeholder stands


class Engine:
    def __init__(self, model, cache: CacheManager, scheduler: Scheduler, serving: ServingConfig,
                 stop_tokens: Seq[int] = (), states: StateSlots | None = None, runner: StepRunner | None = None):
        serving.validate()
        self.model, self.cache, self.scheduler, self.serving = model, cache, scheduler, serving
        self.stop_tokens = set(int(t) for t in stop_tokens)
        self.states = states
        self.runner = runner or StepRunner(model, cache, serving.max_tokens_per_step, serving.max_seqs,
                                           serving.max_seqs, states=states)
        if self.runner.max_tokens < serving.max_tokens_per_step or self.runner.max_seqs < serving.max_seqs or \
                self.runner.max_logit_rows < serving.max_seqs:
            raise InvalidArgument(f"serving config ({serving.max_tokens_per_step} tokens, {serving.max_seqs} sequences "
                                  f"per step) exceeds the step function's limits ({self.runner.max_tokens} tokens, "
                                  f"{self.runner.max_seqs} sequences, {self.runner.max_logit_rows} logit rows)")
        self.sequences: dict[int, Sequence] = {}
        self._next_id = 0
        self._stepping = False
        self._ahead: _Pending | None = None      # a step queued before the tokens of the one ahead of it were read
        self._on_token: Callable[[int, int], None] | None = None
        self._stats = EngineStats()
        self.max_blocks_per_seq = blocks_for(model.spec.max_positions, cache.page_size)

    # -- requests
    def add_request(self, prompt: Seq[int], params: SamplingParams | None = None) -> int:
        """Queues a request and returns its id. Only a prompt that can never run is rejected
        (CapacityError) before any compute; otherwise max_tokens is clamped to what the
        context and the pool can hold (src/engine/engine.cpp:26-63)."""
        params = SamplingParams(**vars(params)) if params is not None else SamplingParams()
        params.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise InvalidArgument("prompt is empty")
        vocab = self.model.spec.vocab_size
        for t in prompt:
            if not 0 <= t < vocab:
                raise InvalidArgument(f"prompt token {t} outside vocabulary of {vocab}")
        page = self.cache.page_size
        context_cap = self.model.spec.max_positions
        pool_cap = self.cache.max_tokens_per_request()
        n = len(prompt)
        if n >= context_cap:
            raise CapacityError(f"prompt of {n} tokens leaves no room to generate in the model context of {context_cap}")
        if n >= pool_cap:
            raise CapacityError(f"prompt of {n} tokens plus one generated token needs {blocks_for(n + 1, page)} KV pages "
                                f"but the cache holds {pool_cap // page}; raise --kv-mem")
        params.max_tokens = min(params.max_tokens, min(context_cap, pool_cap) - n)
        # A waiting request holds no page and no state slot: both are taken when the scheduler admits it.
        seq = Sequence(id=self._next_id, tokens=prompt, prompt_len=n, params=params, cache=self.cache.new_request())
        self._next_id += 1
        self.scheduler.add(seq)
        self.sequences[seq.id] = seq
        return seq.id

    def sequence(self, seq_id: int) -> Sequence:
        try:
            return self.sequences[seq_id]
        except KeyError:
            raise InvalidArgument(f"no sequence with id {seq_id}") from None

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._ahead is not None

    def set_token_callback(self, callback: Callable[[int, int], None] | None) -> None:
        """`callback(request id, token)` is called for every generated token, in the order of the step's rows.
        It may cancel requests. While it runs, the tokens of other requests of the step may still end in
        PLACEHOLDER (their id is handed out next); its own token is in place."""
        self._on_token = callback

    # -- one step
    def _check_batch(self, batch: ScheduledBatch) -> None:
        """A scheduler bug must fail loudly before any compute (src/engine/engine.cpp:65-92)."""
        if len(batch.seqs) > self.serving.max_seqs:
            raise InvalidArgument(f"scheduler gave {len(batch.seqs)} sequences; a step allows at most {self.serving.max_seqs}")
        total, seen = 0, set()
        for seq, n in batch.seqs:
            if n <= 0 or n > seq.num_pending:
                raise InvalidArgument(f"scheduler gave sequence {seq.id} {n} tokens; it has {seq.num_pending} pending")
            if seq.id in seen:
                raise InvalidArgument(f"scheduler gave sequence {seq.id} twice in one step")
            seen.add(seq.id)
            end = seq.num_computed + n
            for t in seq.cache.tables:
                if len(t) < blocks_for(end, self.cache.page_size):
                    raise InvalidArgument(f"sequence {seq.id} has {len(t)} KV pages reserved; {end} tokens need "
                                          f"{blocks_for(end, self.cache.page_size)}")
            total += n
        if total > self.serving.max_tokens_per_step:
            raise InvalidArgument(f"scheduler gave {total} tokens; a step allows at most {self.serving.max_tokens_per_step}")

    def step(self) -> None:
        """One step: a batch is decided, run, and its tokens are handed out. With `serving.run_ahead` the
        step after it is decided and queued on the GPU before this one's tokens are read: the requests'
        bookkeeping is moved past the step in flight (`_advance`: its tokens count as computed, and a
        placeholder stands for every token it is sampling), the scheduler decides as it always does, and a
        request that goes on decoding takes its input token from the device. The host's work (deciding,
        index arrays, launches) then overlaps the GPU's step. Tokens come out in the same order with the same
        values either way, since a request's tokens do not depend on what it is batched with; a request that
        stops on a stop token or is cancelled runs at most one step in vain."""
        if self._stepping:
            raise InvalidArgument("step() called during a step (e.g. from a token callback)")
        self._stepping = True
        try:
            pending, self._ahead = self._ahead, None
            if pending is not None and all(seq.state == SeqState.FINISHED for seq, _ in pending.batch.seqs):
                self._complete(pending)      # queued ahead for requests that have all ended since: nothing to hand out
                pending = None
            if pending is None:
                batch = self.scheduler.schedule()
                if batch.empty():
                    return
                pending = self._launch(batch)
            launch_error = None
            if self.serving.run_ahead:
                self._advance(pending)
                nxt = self.scheduler.schedule()
                if not nxt.empty():
                    try:
                        self._ahead = self._launch(nxt, behind=pending)
                        self._stats.steps_ahead += 1
                    except Exception as e:       # its reservation has been given back; the step in flight still counts
                        launch_error = e
            try:
                self._complete(pending)
            except BaseException:
                self._drop_ahead()
                raise
            if launch_error is not None:
                raise launch_error
        finally:
            self._stepping = False

    def _launch(self, batch: ScheduledBatch, behind: "_Pending | None" = None) -> "_Pending":
        """Queues the batch on the GPU and the copy of its sampled ids to the host. A request whose next token
        is a placeholder gets it from the row of the step in flight (`behind`) that samples it."""
        sampled: list[Sequence] = []
        prefill = decode = 0
        try:
            self._check_batch(batch)
            rows = {seq.id: r for r, seq in enumerate(behind.sampled)} if behind is not None else {}
            entries = []
            for seq, n in batch.seqs:
                begin, end = seq.num_computed, seq.num_computed + n
                tokens, device_row = seq.tokens[begin:end], None
                if tokens[0] == PLACEHOLDER:
                    tokens, device_row = [0] + tokens[1:], rows[seq.id]
                if PLACEHOLDER in tokens:
                    raise InvalidArgument(f"sequence {seq.id} was scheduled past a token that is not known yet")
                samples = end == len(seq.tokens)   # its whole pending input is in the cache after this step
                entries.append(StepEntry(seq.cache, tokens, begin, (n - 1,) if samples else (), device_row))
                if samples:
                    sampled.append(seq)
                if seq.state == SeqState.DECODING and n == 1:
                    decode += n
                else:
                    prefill += n
            t0 = time.perf_counter()
            sampling = [(s.params, s.num_generated) for s in sampled]
            logits, ids = self.runner.run(entries, sampling)
            tokens = self.runner.fetch(logits, ids, sampling)
            self._stats.step_seconds += time.perf_counter() - t0
        except BaseException:
            self._give_back(batch)
            raise
        return _Pending(batch, sampled, tokens, prefill, decode)

    def _advance(self, pending: "_Pending") -> None:
        """Moves the requests' bookkeeping past a step that is still in flight, so that the next one can be
        decided: its tokens count as computed and a placeholder stands for each token it is sampling. A request
        that reaches its max_tokens with that token leaves the scheduler now and is finished when the token
        is there. Pages that a window has passed, or that a preemption in the next decision takes away, may
        still be read by the step in flight: whoever gets them next is queued behind it on the same stream."""
        for seq, n in pending.batch.seqs:
            if seq.state == SeqState.FINISHED:
                continue
            seq.num_computed += n
            self.cache.advance_window(seq.cache, seq.num_computed)
        for seq in pending.sampled:
            if seq.state == SeqState.FINISHED:
                continue
            pending.token_at[seq.id] = len(seq.tokens)
            seq.tokens.append(PLACEHOLDER)
            seq.state = SeqState.DECODING
            if seq.num_generated >= seq.params.max_tokens:
                self.scheduler.finish(seq)
        self.scheduler.complete(pending.batch)
        pending.advanced = True

    def _give_back(self, batch: ScheduledBatch) -> None:
        """The step did not run: give back what the scheduler reserved and let it be scheduled again.
        State of fixed size may be half-updated, so requests that keep some start over."""
        for seq, _ in batch.seqs:
            if seq.state == SeqState.FINISHED:
                continue
            if self.cache.needs_state_slot:
                self.cache.reset(seq.cache)
                seq.num_computed = 0
            else:
                self.cache.truncate(seq.cache, seq.num_computed)
        self.scheduler.abandon(batch)

    def _drop_ahead(self) -> None:
        """Forgets the step queued ahead (its results will never be read) once the GPU is done with it."""
        ahead, self._ahead = self._ahead, None
        if ahead is None:
            return
        self.runner.synchronize()
        self._give_back(ahead.batch)

    def _start_over(self, pending: "_Pending") -> None:
        """A step whose bookkeeping had been moved on failed: its requests lose their placeholders and are
        computed again from their first token, like preempted ones."""
        for seq, _ in pending.batch.seqs:
            if seq.state == SeqState.FINISHED:
                continue
            if seq.tokens and seq.tokens[-1] == PLACEHOLDER:
                seq.tokens.pop()
            self.cache.reset(seq.cache)
            seq.num_computed = 0
            self.scheduler.requeue(seq)
        self.scheduler.abandon(pending.batch)

    def _complete(self, pending: "_Pending") -> None:
        """Waits for the step's tokens and hands them out; finishes what ends."""
        batch, sampled = pending.batch, pending.sampled
        try:
            t0 = time.perf_counter()
            tokens = pending.tokens.result()
            self._stats.step_seconds += time.perf_counter() - t0
            self._stats.steps += 1
            self._stats.seqs_scheduled += len(batch.seqs)
            self._stats.prefill_tokens += pending.prefill
            self._stats.decode_tokens += pending.decode
        except BaseException:
            self._drop_ahead()
            if pending.advanced:
                self._start_over(pending)
            else:
                self._give_back(batch)
            raise

        if not pending.advanced:
            for seq, n in batch.seqs:
                if seq.state == SeqState.FINISHED:
                    continue   # it ended while this step, queued ahead, was in flight: the step ran in vain for it
                seq.num_computed += n
                self.cache.advance_window(seq.cache, seq.num_computed)
            self.scheduler.complete(batch)

        for i, seq in enumerate(sampled):
            if seq.state == SeqState.FINISHED:
                continue  # cancelled by an earlier token callback of this step, or ended a step ago
            token = tokens[i]
            if token < 0:
                # The sampler refused the row (src/sampling/sampler.cpp:18-26): this request ends with an error,
                # the step's other requests go on (src/engine/engine.cpp:157-174).
                self._finish(seq, FinishReason.ERROR)
                continue
            try:
                if pending.advanced:
                    seq.tokens[pending.token_at[seq.id]] = token
                else:
                    seq.tokens.append(token)
                    seq.state = SeqState.DECODING
                if self._on_token is not None:
                    self._on_token(seq.id, token)
            except BaseException:
                # The sequences after it count this step as computed but will never get their token.
                for later in sampled[i:]:
                    if later.state != SeqState.FINISHED:
                        self._finish(later, FinishReason.ERROR)
                raise
            if seq.state == SeqState.FINISHED:
                continue  # its own callback cancelled it
            if token in self.stop_tokens:
                self._finish(seq, FinishReason.STOP)
            elif seq.num_generated >= seq.params.max_tokens:
                self._finish(seq, FinishReason.LENGTH)

    def _finish(self, seq: Sequence, reason: FinishReason) -> None:
        if seq.tokens and seq.tokens[-1] == PLACEHOLDER:
            seq.tokens.pop()       # ended while the token was still being sampled: it is never handed out
        seq.state = SeqState.FINISHED
        seq.finish_reason = reason
        self.cache.release(seq.cache)
        self.scheduler.finish(seq)

    def cancel(self, seq_id: int) -> None:
        """Finishes a waiting, running or preempted request as CANCELLED; safe from a token callback."""
        seq = self.sequence(seq_id)
        if seq.state != SeqState.FINISHED:
            self._finish(seq, FinishReason.CANCELLED)

    def release(self, seq_id: int) -> None:
        """Forgets a finished request; not allowed during step()."""
        if self._stepping:
            raise InvalidArgument(f"cannot release sequence {seq_id} during a step")
        if self.sequence(seq_id).state != SeqState.FINISHED:
            raise InvalidArgument(f"sequence {seq_id} is still running")
        del self.sequences[seq_id]

    def stats(self) -> EngineStats:
        s = EngineStats(**vars(self._stats))
        s.preemptions = self.scheduler.num_preemptions
        return s

    def generate(self, prompt: Seq[int], params: SamplingParams | None = None) -> list[int]:
        """Runs one request to completion and returns its generated tokens, a final stop token included."""
        seq_id = self.add_request(prompt, params)
        try:
            while self.sequence(seq_id).state != SeqState.FINISHED:
                self.step()
        except BaseException:
            seq = self.sequences.get(seq_id)
            if seq is not None:
                if seq.state != SeqState.FINISHED:
                    self._finish(seq, FinishReason.ERROR)
                del self.sequences[seq_id]
            raise
        seq = self.sequence(seq_id)
        out = seq.tokens[seq.prompt_len:]
        self.release(seq_id)
        return out

    def generate_batch(self, prompts: Seq[Seq[int]], params: SamplingParams | Seq[SamplingParams] | None = None) -> list[list[int]]:
        """Runs several requests together through the scheduler; returns their generated tokens in order."""
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        ids = [self.add_request(p, q) for p, q in zip(prompts, plist)]
        while any(self.sequence(i).state != SeqState.FINISHED for i in ids):
            self.step()
        outs = []
        for i in ids:
            seq = self.sequence(i)
            outs.append(seq.tokens[seq.prompt_len:])
            self.release(i)
        return outs
