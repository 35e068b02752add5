"""The step function: one batch of (request, its next tokens), run from the cache.

A step takes portions of prompts beside single decoded tokens, cut anywhere, runs only the
tokens it is given as one flat unpadded batch, appends their keys and values to the pages
the requests hold, and returns float32 logits at the wanted places only. It is the one way
into the model: generation, the scheduler's batches and trace replay all come through here.

The flat batch is the reference's BatchInput (src/model/qwen3.h:24-32, built in
src/engine/engine.cpp:114-135): tokens, positions and slots per row, query_start and
context_lens (length AFTER the step) per sequence, zero-padded block tables, logit rows.
Here rows are ordered so that sequences bringing several tokens come first and sequences
bringing one token last (the attention kernels differ), all index arrays travel in one
pinned buffer and one copy, and block-table rows are as long as this step's longest
sequence needs, not as long as the longest a model could have.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache, blocks_for
from ..errors import CapacityError, InvalidArgument
from ..ops.library import check_device
from .workspace import Workspace


@dataclass
class StepEntry:
    """`tokens` are the request's next tokens; `start` tokens of it are already in the cache;
    `want` are the places among `tokens` whose logits are asked for."""
    cache: RequestCache
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = ()


@dataclass
class GroupStep:
    slots: torch.Tensor          # int32 [T]
    block_tables: torch.Tensor   # int32 [S, MB]


@dataclass
class StepContext:
    """Everything a part may read about the step. Device tensors are int32."""
    T: int
    S: int
    R: int
    tokens: torch.Tensor
    positions: torch.Tensor
    seq_of_row: torch.Tensor
    query_start: torch.Tensor
    context_lens: torch.Tensor
    logit_rows: torch.Tensor
    state_slots: torch.Tensor        # [S] slot of each sequence's fixed-size state
    single_seqs: torch.Tensor        # [single_count] sequences that bring one token
    groups: list[GroupStep]
    multi_rows: int                  # rows [0, multi_rows) belong to sequences that bring several tokens
    single_count: int
    single_max_context: int
    max_context: int
    max_seqs: int
    ws: Workspace                    # buffers of max_tokens rows
    logit_ws: Workspace              # buffers of max_logit_rows rows (final norm, logits)
    host: "HostStep"
    layer_hook: Callable | None = None


@dataclass
class HostStep:
    """Host copies for parts that decide on the host (and for toy parts in tests)."""
    query_start: np.ndarray
    context_lens: np.ndarray
    starts: np.ndarray            # position of each sequence's first token in this step
    state_slots: np.ndarray


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class StepRunner:
    """Owns the workspace and the pinned staging buffer; `run(entries)` is the step function."""

    def __init__(self, model, cache: CacheManager, max_tokens: int, max_seqs: int, max_logit_rows: int | None = None,
                 states=None, device="cuda"):
        check_device()
        if max_tokens <= 0 or max_seqs <= 0:
            raise InvalidArgument("step limits must be positive")
        self.model, self.cache, self.states = model, cache, states
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.max_logit_rows = max_logit_rows if max_logit_rows is not None else max_seqs
        self.device = device
        self.ws = Workspace(max_tokens, device)
        self.logit_ws = Workspace(self.max_logit_rows, device)
        self.vocab = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self._staging_bufs = [None, None]   # two pinned buffers, used in turn, each with the event of its last copy
        self._staging_turn = 0
        self._dev = None
        self.layer_hook = None
        self.fail_hook = None     # tests: called after the batch is built, may raise

    def _staging(self, n: int):
        """A pinned host buffer that no copy in flight still reads, and the device buffer it goes to."""
        self._staging_turn ^= 1
        slot = self._staging_bufs[self._staging_turn]
        if slot is None or slot[0].numel() < n:
            if slot is not None:
                slot[2].synchronize()
            size = max(n, 1 << 14)
            host = torch.empty(size, dtype=torch.int32, pin_memory=True)
            slot = [host, host.numpy(), torch.cuda.Event()]
            self._staging_bufs[self._staging_turn] = slot
        else:
            slot[2].synchronize()
        if self._dev is None or self._dev.numel() < n:
            self._dev = torch.empty(max(n, 1 << 14), dtype=torch.int32, device=self.device)
        return slot

    def run(self, entries: Sequence[StepEntry], return_context: bool = False):
        """Runs one step. Returns float32 logits [R, V] on the device in the order of the entries
        and of their `want` (None when nothing is wanted)."""
        ctx, order = self.prepare(entries)
        logits = self.model.forward(ctx, self.cache, self.states)
        return (logits, ctx) if return_context else logits

    def prepare(self, entries: Sequence[StepEntry]):
        S = len(entries)
        if not 1 <= S <= self.max_seqs:
            raise CapacityError(f"step has {S} sequences; the step function allows 1 to {self.max_seqs}")
        page = self.cache.page_size
        counts = [len(e.tokens) for e in entries]
        T = sum(counts)
        if min(counts) < 1:
            raise InvalidArgument("a step entry brings no token")
        if T > self.max_tokens:
            raise CapacityError(f"step has {T} tokens; the step function allows 1 to {self.max_tokens}")
        R = sum(len(e.want) for e in entries)
        if R > self.max_logit_rows:
            raise CapacityError(f"step requests {R} logit rows; the step function allows 0 to {self.max_logit_rows}")
        seen = set()
        for e in entries:
            if id(e.cache) in seen:
                raise InvalidArgument("a request appears twice in one step")
            seen.add(id(e.cache))
            if not e.cache.live:
                raise InvalidArgument("a step entry names a released request")
            end = e.start + len(e.tokens)
            if e.start < 0 or end > self.max_positions:
                raise CapacityError(f"positions [{e.start}, {end}) do not fit the model's {self.max_positions}")
            for t in e.cache.tables:
                if blocks_for(end, page) > len(t):
                    raise InvalidArgument(f"a request has {len(t)} pages reserved; {end} tokens need "
                                          f"{blocks_for(end, page)}")
        # Sequences that bring several tokens first, then those that bring one (stable).
        order = sorted(range(S), key=lambda i: counts[i] == 1)
        n_multi = sum(1 for c in counts if c > 1)
        multi_rows = sum(c for c in counts if c > 1)
        max_ctx = max(e.start + c for e, c in zip(entries, counts))
        MB = _round_up(blocks_for(max_ctx, page), 4)
        G = len(self.cache.groups)

        # layout of the staging buffer (int32 words)
        sizes = [("tokens", T), ("positions", T), ("seq_of_row", T), ("query_start", S + 1), ("context_lens", S),
                 ("logit_rows", max(R, 1)), ("state_slots", S), ("single_seqs", max(S, 1))]
        for g in range(G):
            sizes += [(f"slots{g}", T), (f"tables{g}", S * MB)]
        offs, total = {}, 0
        for name, n in sizes:
            offs[name] = (total, n)
            total += _round_up(n, 4)  # 16-byte aligned sections
        slot = self._staging(total)
        host, dev = slot[1], self._dev

        def sec(name):
            o, n = offs[name]
            return host[o:o + n]

        tokens, positions, seq_of_row = sec("tokens"), sec("positions"), sec("seq_of_row")
        query_start, context_lens = sec("query_start"), sec("context_lens")
        state_slots = sec("state_slots")
        row_of = {}  # (original entry index) -> first row
        row = 0
        query_start[0] = 0
        starts = np.empty(S, dtype=np.int64)
        tables = [sec(f"tables{g}").reshape(S, MB) for g in range(G)]
        for g in range(G):
            tables[g][:] = 0
        for s, i in enumerate(order):
            e, n = entries[i], counts[i]
            tok = np.asarray(e.tokens, dtype=np.int64)
            if tok.min() < 0 or tok.max() >= self.vocab:
                bad = int(tok[(tok < 0) | (tok >= self.vocab)][0])
                raise InvalidArgument(f"token id {bad} outside vocabulary of {self.vocab}")
            tokens[row:row + n] = tok
            positions[row:row + n] = np.arange(e.start, e.start + n)
            seq_of_row[row:row + n] = s
            row_of[i] = row
            starts[s] = e.start
            context_lens[s] = e.start + n
            state_slots[s] = e.cache.state_slot
            for g in range(G):
                sec(f"slots{g}")[row:row + n] = self.cache.slots(e.cache, g, e.start, e.start + n)
                t = e.cache.tables[g]
                k = min(len(t), MB)
                tables[g][s, :k] = np.maximum(t.ids[:k], 0)  # pages below a window are never read
            row += n
            query_start[s + 1] = row
        logit_rows = sec("logit_rows")
        r = 0
        for i, e in enumerate(entries):
            for wpos in e.want:
                if not 0 <= wpos < counts[i]:
                    raise InvalidArgument(f"wanted place {wpos} outside the {counts[i]} tokens of its entry")
                logit_rows[r] = row_of[i] + wpos
                r += 1
        single = sec("single_seqs")
        n_single = S - n_multi
        single[:n_single] = np.arange(n_multi, S)
        single_max_ctx = int(context_lens[n_multi:S].max()) if n_single else 0

        dev[:total].copy_(slot[0][:total], non_blocking=True)
        slot[2].record()

        def dsec(name, n=None):
            o, full = offs[name]
            return dev[o:o + (full if n is None else n)]

        groups = [GroupStep(dsec(f"slots{g}"), dsec(f"tables{g}").view(S, MB)) for g in range(G)]
        hs = HostStep(query_start.copy(), context_lens.copy(), starts, state_slots.copy())
        ctx = StepContext(T=T, S=S, R=R, tokens=dsec("tokens"), positions=dsec("positions"),
                          seq_of_row=dsec("seq_of_row"), query_start=dsec("query_start"),
                          context_lens=dsec("context_lens"), logit_rows=dsec("logit_rows", R),
                          state_slots=dsec("state_slots"), single_seqs=dsec("single_seqs"), groups=groups,
                          multi_rows=multi_rows, single_count=n_single, single_max_context=single_max_ctx,
                          max_context=max_ctx, max_seqs=self.max_seqs, ws=self.ws, logit_ws=self.logit_ws, host=hs,
                          layer_hook=self.layer_hook)
        if self.fail_hook is not None:
            self.fail_hook(ctx)
        return ctx, order
