"""The step function: one batch of (request, its next tokens), run from the cache.

A step takes portions of prompts beside single decoded tokens, cut anywhere, runs only the
tokens it is given as one flat unpadded batch, appends their keys and values to the pages
the requests hold, and returns float32 logits at the wanted places only (and, when asked,
the token sampled from each of those rows). It is the one way into the model: generation,
the scheduler's batches and trace replay all come through here.

The flat batch is the reference's BatchInput (src/model/qwen3.h:24-32, built in
src/engine/engine.cpp:114-135): tokens, positions and slots per row, query_start and
context_lens (length AFTER the step) per sequence, zero-padded block tables, logit rows.
Here rows are ordered so that sequences bringing several tokens come first and sequences
bringing one token last (the attention kernels differ), all index arrays and sampling
parameters travel in one pinned buffer and one copy, and block-table rows are as long as
this step's longest sequence needs, not as long as the longest a model could have.

Steps in which every sequence brings one token (decoding) are launch-bound when issued
kernel by kernel, so they are captured once per (batch bucket, table-length bucket) as a
CUDA graph over fixed buffers and replayed; sequences that pad a bucket have no keys and
write nothing.
"""
from __future__ import annotations

import gc

from dataclasses import dataclass, field
from typing import Callable, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, RequestCache, blocks_for
from ..errors import CapacityError, InvalidArgument, TieError
from ..ops import gemm_select
from ..ops.library import check_device
from ..sampling.params import SamplingParams
from .workspace import Workspace


@dataclass
class StepEntry:
    """`tokens` are the request's next tokens; `start` tokens of it are already in the cache;
    `want` are the places among `tokens` whose logits are asked for. With `device_row` the first of
    `tokens` is a placeholder: the real one is the id that the step before this one sampled for its
    row `device_row`, still on the device (perhaps not computed yet)."""
    cache: RequestCache
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = ()
    device_row: int | None = None


@dataclass
class GroupStep:
    slots: torch.Tensor          # int32 [T]
    block_tables: torch.Tensor   # int32 [S, MB]


@dataclass
class HostStep:
    """Host copies for parts that decide on the host (and for toy parts in tests)."""
    query_start: np.ndarray
    context_lens: np.ndarray
    starts: np.ndarray            # position of each sequence's first token in this step
    state_slots: np.ndarray


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
    multi_seqs: int                  # sequences [0, multi_seqs) are those
    multi_max_queries: int           # the most tokens one of them brings
    single_count: int
    single_max_context: int
    max_context: int
    max_seqs: int
    ws: Workspace                    # buffers of max_tokens rows
    logit_ws: Workspace              # buffers of max_logit_rows rows (final norm, logits)
    host: HostStep
    layer_hook: Callable | None = None
    ws_dtype: torch.dtype | None = None   # the model's compute dtype (set by Model.forward)
    # sampling parameters per logit row (None when the step does not sample)
    inv_temperature: torch.Tensor | None = None
    seeds: torch.Tensor | None = None
    counters: torch.Tensor | None = None
    top_k: torch.Tensor | None = None              # given only when a row filters (top-k, top-p)
    top_p: torch.Tensor | None = None
    single_contexts: tuple | None = None   # context lengths of the sequences that bring one token, when the step is not a captured graph
    memo: dict = field(default_factory=dict)   # what a part works out once per step and every layer of its kind uses again


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def _bucket(n: int, limit: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return min(b, limit) if n <= limit else n


class PendingTokens:
    """The sampled ids of a step on their way to the host."""

    def __init__(self, runner, host, event, logits, sampling):
        self.runner, self.host, self.event, self.logits, self.sampling = runner, host, event, logits, sampling

    def result(self) -> list[int]:
        """Waits for the copy and checks the kernels' status words."""
        R = len(self.sampling)
        if R == 0:
            return []
        self.event.synchronize()
        gemm_select.check_status()
        return self.host[:R].tolist()


class StepRunner:
    """Owns the workspace, the staging buffers and the decode graphs; `run(entries)` is the step function."""

    def __init__(self, model, cache: CacheManager, max_tokens: int, max_seqs: int, max_logit_rows: int | None = None,
                 states=None, device="cuda", use_graphs: bool = True):
        check_device()
        if max_tokens <= 0 or max_seqs <= 0:
            raise InvalidArgument("step limits must be positive")
        self.model, self.cache, self.states = model, cache, states
        self.max_tokens, self.max_seqs = max_tokens, max(1, min(max_seqs, max_tokens))
        self.max_logit_rows = max_logit_rows if max_logit_rows is not None else self.max_seqs
        self.device = device
        self.ws = Workspace(max_tokens, device)
        self.logit_ws = Workspace(self.max_logit_rows, device)
        self.vocab = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self._staging_bufs = [None, None]   # two pinned buffers, used in turn, each with the event of its last copy
        self._staging_turn = 0
        # The device copy of the index arrays never moves: captured graphs read it at fixed offsets.
        G = len(cache.groups)
        mb = self._table_cap = _round_up(blocks_for(self.max_positions, cache.page_size), 4)
        words = 4 * max_tokens + 6 * self.max_seqs + 6 * self.max_logit_rows + G * (max_tokens + self.max_seqs * mb) + 64 * (8 + 2 * G)
        self._dev = torch.zeros(words, dtype=torch.int32, device=device)
        self._ids = torch.zeros(self.max_logit_rows, dtype=torch.int32, device=device)
        self.last_h2d_bytes = 0
        self._ids_host = [(torch.zeros(self.max_logit_rows, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                          for _ in range(2)]
        self._ids_turn = 0
        self.layer_hook = None
        self.fail_hook = None     # tests: called after the batch is built, may raise
        # A mixer with state of its own may be plain torch code that reads the step on the host: decode steps are
        # captured as graphs only if every such mixer says that it can be (`Mixer.graph_safe`).
        stateful = [model.layers[e.layer].mixer for i, e in enumerate(model.spec.run_order)
                    if states is not None and states.tensor(i) is not None]
        self.use_graphs = use_graphs and all(getattr(m, "graph_safe", False) for m in stateful)
        self._graphs: dict[tuple, tuple] = {}
        self.graph_replays = 0
        self.kernels_in_graph: dict[tuple, int] = {}

    # -- staging
    def _staging(self, n: int):
        """A pinned host buffer that no copy in flight still reads."""
        self._staging_turn ^= 1
        slot = self._staging_bufs[self._staging_turn]
        if slot is None or slot[0].numel() < n:
            if slot is not None:
                slot[2].synchronize()
            host = torch.empty(max(n, 1 << 14), dtype=torch.int32, pin_memory=True)
            slot = [host, host.numpy(), torch.cuda.Event()]
            self._staging_bufs[self._staging_turn] = slot
        else:
            slot[2].synchronize()
        if self._dev.numel() < n:
            raise CapacityError(f"step needs {n} index words; the step function was sized for {self._dev.numel()}")
        return slot

    # -- the step function
    def run(self, entries: Sequence[StepEntry], sampling: Sequence[tuple[SamplingParams, int]] | None = None,
            device_tokens: bool = False):
        """Runs one step. Returns float32 logits [R, V] on the device in the order of the entries and
        of their `want` (None when nothing is wanted). With `sampling` (one (parameters, index of
        the generated token) per wanted row) returns (logits, ids): ids is an int32 device tensor
        [R] picked by the sampling kernels (greedy, temperature, top-k, top-p).

        An entry with `device_row`, and with `device_tokens` every entry i as if it had `device_row` i,
        takes its first token from the ids that the step before sampled (still on the device, perhaps not
        computed yet): the step can be queued before the host has seen those ids."""
        if device_tokens and any(len(e.tokens) != 1 for e in entries):
            raise InvalidArgument("device_tokens is for steps in which every entry brings one token")
        graph_key = self._graph_key(entries, sampling)
        if graph_key is not None:
            return self._run_graph(entries, sampling, graph_key, device_tokens)
        ctx = self.prepare(entries, sampling, device_tokens=device_tokens)
        logits = self.model.forward(ctx, self.cache, self.states)
        if sampling is None:
            return logits
        return logits, self._sample(ctx, logits)

    def _sample(self, ctx: StepContext, logits):
        if logits is None:
            return None
        ops.sample(logits, self._ids, ctx.inv_temperature, ctx.seeds, ctx.counters, ctx.top_k, ctx.top_p)
        return self._ids[:ctx.R]

    def fetch(self, logits, ids, sampling) -> "PendingTokens":
        """Queues the copy of a step's sampled ids to the host (into one of two pinned buffers used in
        turn) and returns a handle; `result()` waits for it. Another step may be queued in between."""
        R = len(sampling)
        self._ids_turn ^= 1
        host, event = self._ids_host[self._ids_turn]
        if R > 0:
            host[:R].copy_(ids[:R], non_blocking=True)
        event.record()
        return PendingTokens(self, host, event, logits, list(sampling))

    def tokens_of(self, logits, ids, sampling) -> list[int]:
        """Brings the sampled ids to the host (one copy, one synchronize) and samples rows that need
        Checks the kernels' status words."""
        return self.fetch(logits, ids, sampling).result()

    def synchronize(self) -> None:
        """Waits until the GPU is done with every step queued so far."""
        torch.cuda.current_stream().synchronize()

    def check(self) -> None:
        """After a synchronize: raises if a kernel of an earlier step gave up a bounded wait."""
        gemm_select.check_status()

    # -- decode graphs
    def _graph_key(self, entries, sampling):
        if not self.use_graphs or self.layer_hook is not None or self.fail_hook is not None:
            return None
        S = len(entries)
        if S > self.max_seqs or any(len(e.tokens) != 1 for e in entries):
            return None
        if any(len(e.want) != 1 for e in entries) or S > self.max_logit_rows:
            return None
        if sampling is not None and len(sampling) != S:
            return None
        page = self.cache.page_size
        need = max(blocks_for(e.start + 1, page) for e in entries)
        sb = _bucket(S, self.max_seqs)
        if sb > self.max_logit_rows or sb > self.max_tokens:
            return None
        # table lengths come in powers of two, but never longer than the longest table a request can have:
        # the index buffer is sized for that
        mb = min(max(16, _bucket(need, 1 << 30)), max(self._table_cap, need))
        filtered = sampling is not None and any(p.filters for p, _ in sampling)   # one more kernel in the graph
        return (sb, mb, sampling is not None, filtered)

    def _run_graph(self, entries, sampling, key, device_tokens=False):
        sb, mb, sampled, _ = key
        ctx = self.prepare(entries, sampling, pad_seqs=sb, table_len=mb, device_tokens=device_tokens)
        if key not in self._graphs:
            # The first step of a shape runs kernel by kernel: that allocates every buffer, loads every kernel and is
            # the step's own execution (a second run would update the state of mixers that keep some a second
            # time). The capture behind it records the same launches over the same buffers and executes nothing.
            logits = self.model.forward(ctx, self.cache, self.states)
            if sampled:
                self._sample(ctx, logits)
            torch.cuda.synchronize()
            before = ops.library.launch_count()
            graph = torch.cuda.CUDAGraph()
            # No garbage collection while capturing: collecting an older runner's graphs frees their memory
            # pools, a CUDA call that is not allowed during a capture and invalidates it.
            gc_was_on = gc.isenabled()
            gc.collect()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    captured = self.model.forward(ctx, self.cache, self.states)
                    if sampled:
                        self._sample(ctx, captured)
            finally:
                if gc_was_on:
                    gc.enable()
            if captured.data_ptr() != logits.data_ptr():
                raise TieError("a decode step's logits moved between its first run and its capture")
            self.kernels_in_graph[key] = ops.library.launch_count() - before
            self._graphs[key] = (graph, captured)
        else:
            graph, logits = self._graphs[key]
            graph.replay()
            self.graph_replays += 1
        S = len(entries)
        if sampling is None:
            return logits[:S]
        return logits[:S], self._ids[:S]

    # -- building the flat batch
    def prepare(self, entries: Sequence[StepEntry], sampling=None, pad_seqs: int | None = None,
                table_len: int | None = None, device_tokens: bool = False) -> StepContext:
        S_real = len(entries)
        if not 1 <= S_real <= self.max_seqs:
            raise CapacityError(f"step has {S_real} sequences; the step function allows 1 to {self.max_seqs}")
        page = self.cache.page_size
        counts = [len(e.tokens) for e in entries]
        T_real = sum(counts)
        if min(counts) < 1:
            raise InvalidArgument("a step entry brings no token")
        if T_real > self.max_tokens:
            raise CapacityError(f"step has {T_real} tokens; the step function allows 1 to {self.max_tokens}")
        R_real = sum(len(e.want) for e in entries)
        if R_real > self.max_logit_rows:
            raise CapacityError(f"step requests {R_real} logit rows; the step function allows 0 to {self.max_logit_rows}")
        if sampling is not None and len(sampling) != R_real:
            raise InvalidArgument(f"{len(sampling)} sampling entries for {R_real} wanted rows")
        seen = set()
        for e in entries:
            if id(e.cache) in seen:
                raise InvalidArgument("a request appears twice in one step")
            seen.add(id(e.cache))
            if not e.cache.live:
                raise InvalidArgument("a step entry names a released request")
            if self.cache.needs_state_slot and e.cache.state_slot < 0:
                raise InvalidArgument("a step entry names a request without a state slot (nothing was reserved for it)")
            end = e.start + len(e.tokens)
            if e.start < 0 or end > self.max_positions:
                raise CapacityError(f"positions [{e.start}, {end}) do not fit the model's {self.max_positions}")
            for t in e.cache.tables:
                if blocks_for(end, page) > len(t):
                    raise InvalidArgument(f"a request has {len(t)} pages reserved; {end} tokens need "
                                          f"{blocks_for(end, page)}")
        # Sequences that bring several tokens first, then those that bring one (stable).
        order = sorted(range(S_real), key=lambda i: counts[i] == 1)
        n_multi = sum(1 for c in counts if c > 1)
        multi_rows = sum(c for c in counts if c > 1)
        max_ctx = max(e.start + c for e, c in zip(entries, counts))
        pad = (pad_seqs or S_real) - S_real          # padding sequences: one row each, no keys, no slot
        S, T, R = S_real + pad, T_real + pad, R_real + pad
        MB = table_len if table_len is not None else _round_up(blocks_for(max_ctx, page), 4)
        G = len(self.cache.groups)

        # layout of the staging buffer (int32 words); 64-bit sections are 8-byte aligned because every section is 16-byte aligned
        sizes = [("tokens", T), ("positions", T), ("seq_of_row", T), ("query_start", S + 1), ("context_lens", S),
                 ("logit_rows", max(R, 1)), ("state_slots", S), ("single_seqs", max(S, 1)),
                 ("inv_t", max(R, 1)), ("seeds", 2 * max(R, 1)), ("counters", 2 * max(R, 1)),
                 ("top_k", max(R, 1)), ("top_p", max(R, 1)), ("ids_dst", S), ("ids_src", S)]
        for g in range(G):
            sizes += [(f"slots{g}", T), (f"tables{g}", S * MB)]
        offs, total = {}, 0
        for name, n in sizes:
            offs[name] = (total, n)
            total += _round_up(n, 4)
        slot = self._staging(total)
        host, dev = slot[1], self._dev

        def sec(name):
            o, n = offs[name]
            return host[o:o + n]

        tokens, positions, seq_of_row = sec("tokens"), sec("positions"), sec("seq_of_row")
        query_start, context_lens = sec("query_start"), sec("context_lens")
        state_slots = sec("state_slots")
        row_of = {}
        row = 0
        query_start[0] = 0
        starts = np.zeros(S, dtype=np.int64)
        tables = [sec(f"tables{g}").reshape(S, MB) for g in range(G)]
        for g in range(G):
            tables[g][:] = 0
        windowed = [g.kind == "window" for g in self.cache.groups]
        if T_real == S_real:
            # Every sequence brings one token (decode): plain Python numbers, one array assignment per section.
            toks = [0] * S_real if device_tokens else [int(e.tokens[0]) for e in entries]
            if min(toks) < 0 or max(toks) >= self.vocab:
                bad = next(t for t in toks if t < 0 or t >= self.vocab)
                raise InvalidArgument(f"token id {bad} outside vocabulary of {self.vocab}")
            begin = [e.start for e in entries]
            tokens[:S_real] = toks
            positions[:S_real] = begin
            seq_of_row[:S_real] = query_start[:S_real] = np.arange(S_real, dtype=np.int32)
            query_start[S_real] = S_real
            starts[:S_real] = begin
            context_lens[:S_real] = [b + 1 for b in begin]
            state_slots[:S_real] = [e.cache.state_slot for e in entries]
            for g in range(G):
                slots_g = []
                for s, e in enumerate(entries):
                    t = e.cache.tables[g]
                    page_id = int(t.ids[e.start // page])
                    if page_id < 0:
                        raise InvalidArgument("a position below the window was asked for: its page has been given back")
                    slots_g.append(page_id * page + e.start % page)
                    k = min(len(t), MB)
                    tables[g][s, :k] = np.maximum(t.ids[:k], 0) if windowed[g] else t.ids[:k]
                sec(f"slots{g}")[:S_real] = slots_g
            row_of = {i: i for i in range(S_real)}
            row = S_real
        else:
            for s, i in enumerate(order):
                e, n = entries[i], counts[i]
                if n == 1:
                    # one token beside others' portions: plain numbers, no array per sequence
                    t0 = int(e.tokens[0])
                    if not 0 <= t0 < self.vocab:
                        raise InvalidArgument(f"token id {t0} outside vocabulary of {self.vocab}")
                    tokens[row], positions[row], seq_of_row[row] = t0, e.start, s
                    row_of[i] = row
                    starts[s] = e.start
                    context_lens[s] = e.start + 1
                    state_slots[s] = e.cache.state_slot
                    for g in range(G):
                        t = e.cache.tables[g]
                        page_id = int(t.ids[e.start // page])
                        if page_id < 0:
                            raise InvalidArgument("a position below the window was asked for: its page has been given back")
                        sec(f"slots{g}")[row] = page_id * page + e.start % page
                        k = min(len(t), MB)
                        tables[g][s, :k] = np.maximum(t.ids[:k], 0) if windowed[g] else t.ids[:k]
                    row += 1
                    query_start[s + 1] = row
                    continue
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
                    tables[g][s, :k] = np.maximum(t.ids[:k], 0) if windowed[g] else t.ids[:k]  # pages below a window are never read
                row += n
                query_start[s + 1] = row
        for s in range(S_real, S):                  # padding
            tokens[row], positions[row], seq_of_row[row] = 0, 0, s
            context_lens[s], state_slots[s] = 0, -1
            for g in range(G):
                sec(f"slots{g}")[row] = -1
            row += 1
            query_start[s + 1] = row
        logit_rows = sec("logit_rows")
        r = 0
        for i, e in enumerate(entries):
            for wpos in e.want:
                if not 0 <= wpos < counts[i]:
                    raise InvalidArgument(f"wanted place {wpos} outside the {counts[i]} tokens of its entry")
                logit_rows[r] = row_of[i] + wpos
                r += 1
        for s in range(S_real, S):
            logit_rows[r] = T_real + (s - S_real)
            r += 1
        single = sec("single_seqs")
        n_single = S - n_multi
        single[:n_single] = np.arange(n_multi, S)
        if table_len is not None:
            single_max_ctx = MB * page               # a captured graph must hold for every context of its bucket
        else:
            single_max_ctx = int(context_lens[n_multi:S].max()) if n_single else 0
        if sampling is not None:
            inv_t = sec("inv_t").view(np.float32)
            seeds, counters = sec("seeds").view(np.uint64), sec("counters").view(np.int64)
            inv_t[:], seeds[:], counters[:] = 0.0, 0, 0
            for r, (p, index) in enumerate(sampling):
                inv_t[r], seeds[r], counters[r] = p.inv_temperature(), p.seed, index
            filtered = any(p.filters for p, _ in sampling)
            if filtered:
                top_k, top_p = sec("top_k"), sec("top_p").view(np.float32)
                top_k[:], top_p[:] = 0, 1.0
                for r, (p, _) in enumerate(sampling):
                    top_k[r], top_p[r] = min(p.top_k, 2 ** 31 - 1), p.top_p

        # tokens that are still on the device: (row of the token in this step, row of the step before that samples it)
        from_device = [(row_of[i], i if device_tokens else e.device_row) for i, e in enumerate(entries)
                       if device_tokens or e.device_row is not None]
        if from_device:
            if any(not 0 <= src < self.max_logit_rows for _, src in from_device):
                raise InvalidArgument(f"a device row outside the {self.max_logit_rows} rows a step samples")
            ids_dst, ids_src = sec("ids_dst"), sec("ids_src")
            ids_dst[:len(from_device)] = [d for d, _ in from_device]
            ids_src[:len(from_device)] = [r for _, r in from_device]

        dev[:total].copy_(slot[0][:total], non_blocking=True)
        slot[2].record()
        self.last_h2d_bytes = 4 * total        # what this step copied to the device (bench.py reports it)

        def dsec(name, n=None):
            o, full = offs[name]
            return dev[o:o + (full if n is None else n)]

        if from_device:
            ops.scatter_ids(dsec("tokens"), dsec("ids_dst"), dsec("ids_src"), self._ids, len(from_device))

        groups = [GroupStep(dsec(f"slots{g}"), dsec(f"tables{g}").view(S, MB)) for g in range(G)]
        hs = HostStep(query_start.copy(), context_lens.copy(), starts, state_slots.copy())
        ctx = StepContext(T=T, S=S, R=R, tokens=dsec("tokens"), positions=dsec("positions"),
                          seq_of_row=dsec("seq_of_row"), query_start=dsec("query_start"),
                          context_lens=dsec("context_lens"), logit_rows=dsec("logit_rows", R),
                          state_slots=dsec("state_slots"), single_seqs=dsec("single_seqs"), groups=groups,
                          multi_rows=multi_rows, multi_seqs=n_multi,
                          multi_max_queries=max((c for c in counts if c > 1), default=0), single_count=n_single, single_max_context=single_max_ctx,
                          single_contexts=None if table_len is not None else tuple(int(c) for c in context_lens[n_multi:S]),
                          max_context=max_ctx, max_seqs=self.max_seqs, ws=self.ws, logit_ws=self.logit_ws, host=hs,
                          layer_hook=self.layer_hook)
        if sampling is not None:
            ctx.inv_temperature = dsec("inv_t", R).view(torch.float32)
            ctx.seeds = dsec("seeds", 2 * R).view(torch.int64)
            ctx.counters = dsec("counters", 2 * R).view(torch.int64)
            if filtered:
                ctx.top_k, ctx.top_p = dsec("top_k", R), dsec("top_p", R).view(torch.float32)
        if self.fail_hook is not None:
            self.fail_hook(ctx)
        return ctx
