"""The cache manager: keys and values in pages, a block table per request and group, slots of fixed-size state.

Layers are put into groups by what they need of the cache (kv heads, head size, all keys or a
window of them). Each group has its own page pool and its own storage
`[planes][2 (K, V)][pages][kv_heads][page_size][head_dim]`, one plane per run entry of the
group; within a group a page id addresses the same token slots in every plane, as in the
reference's single group (src/kv/paged_kv_cache.h:27-30). A request holds one block table
per group: token j lives in page table[j // page_size] at offset j % page_size
(src/kv/paged_kv_cache.h:14-16).

Pages go back to the pool when a request is released (finished, cancelled or preempted),
when a table is truncated after a failed step, and, in a window group, when the window has
passed them: their table entry becomes -1 and no later query reads below the window.
`reserve` is all-or-nothing over all groups (src/kv/paged_kv_cache.cpp:41-49).

A request that only waits holds nothing (src/engine/sequence.h:15-30: an empty block table):
pages and, for models whose mixers keep state of fixed size, the state slot are taken by
`reserve`, that is when the scheduler admits the request, and go back on `reset`
(preemption) and `release`.

Groups may differ in size. A window group never holds more than the pages of a window plus
one step per request, so with `window_requests` and `window_step_tokens` given it gets only
that many pages and the byte budget goes to the groups that keep every key.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..errors import CapacityError, InvalidArgument
from .block_pool import BlockPool

FREED = -1


def blocks_for(tokens: int, page_size: int) -> int:
    return (tokens + page_size - 1) // page_size


class BlockTable:
    """Page ids of one request in one group, in a numpy array so that a step can copy it fast."""
    __slots__ = ("ids", "n", "released")

    def __init__(self):
        self.ids = np.empty(16, dtype=np.int32)
        self.n = 0          # entries in use (positional: entry i covers tokens [i*page, (i+1)*page))
        self.released = 0   # leading entries already given back (window groups)

    def append(self, block: int) -> None:
        if self.n == len(self.ids):
            self.ids = np.concatenate([self.ids, np.empty(len(self.ids), dtype=np.int32)])
        self.ids[self.n] = block
        self.n += 1

    def view(self) -> np.ndarray:
        return self.ids[:self.n]

    def held(self) -> list[int]:
        return [int(b) for b in self.ids[self.released:self.n]]

    def __len__(self) -> int:
        return self.n


@dataclass
class RequestCache:
    """What one request holds: a table per group and a state slot (-1 if the model keeps no state)."""
    tables: list[BlockTable]
    state_slot: int = -1
    live: bool = True


@dataclass(frozen=True)
class GroupSpec:
    kind: str            # "full" | "window"
    kv_heads: int
    head_dim: int
    window: int
    entries: tuple[int, ...]   # run entries whose planes live in this group


class CacheManager:
    """`needs[i]` is what run entry i wants (a parts.CacheNeed or None). With `device` None no
    storage is allocated (host-side tests and the scheduler's arithmetic)."""

    def __init__(self, needs, page_size: int, num_pages: int | None = None, budget_bytes: int | None = None,
                 dtype=None, device=None, state_slots=None, window_requests: int | None = None,
                 window_step_tokens: int = 0):
        """`num_pages` (or what `budget_bytes` buys) is the page count of the groups that keep every key.
        With `window_requests` a window group holds only what that many requests can use at once:
        the pages of `window + window_step_tokens` tokens, and two more for the edges, per request."""
        if page_size <= 0:
            raise InvalidArgument(f"page size must be positive, got {page_size}")
        self.page_size = page_size
        self.dtype = dtype
        keyed: dict[tuple, list[int]] = {}
        for i, need in enumerate(needs):
            if need is None:
                continue
            if need.kv_heads <= 0 or need.head_dim <= 0 or need.kind not in ("full", "window") or \
                    (need.kind == "window" and need.window <= 0):
                raise InvalidArgument(f"bad cache need of run entry {i}: {need}")
            keyed.setdefault((need.kind, need.kv_heads, need.head_dim, need.window if need.kind == "window" else 0),
                             []).append(i)
        self.groups = [GroupSpec(k[0], k[1], k[2], k[3], tuple(v)) for k, v in keyed.items()]
        self._entry_group = {e: gi for gi, g in enumerate(self.groups) for e in g.entries}
        self._entry_plane = {e: pi for g in self.groups for pi, e in enumerate(g.entries)}
        elem = 4 if dtype is None else _elem_size(dtype)
        group_bytes = [2 * len(g.entries) * g.kv_heads * page_size * g.head_dim * elem for g in self.groups]
        # what a window group can ever use (None: as many pages as the other groups)
        bounded = [None] * len(self.groups)
        if window_requests is not None:
            if window_requests <= 0 or window_step_tokens < 0:
                raise InvalidArgument(f"bad window sizing: {window_requests} requests, {window_step_tokens} tokens a step")
            for gi, g in enumerate(self.groups):
                if g.kind == "window":
                    bounded[gi] = window_requests * (blocks_for(g.window + window_step_tokens, page_size) + 2)
        self.bytes_per_page = sum(b for b, fixed in zip(group_bytes, bounded) if fixed is None) or sum(group_bytes)
        if num_pages is None:
            if budget_bytes is None:
                raise InvalidArgument("give num_pages or budget_bytes")
            left = budget_bytes - sum(b * fixed for b, fixed in zip(group_bytes, bounded) if fixed is not None)
            if all(fixed is not None for fixed in bounded) and bounded:
                left = budget_bytes       # window groups only: the budget caps them all alike
            num_pages = left // max(1, self.bytes_per_page)
            if num_pages <= 0:
                raise CapacityError(f"KV budget of {budget_bytes} bytes is smaller than one {self.bytes_per_page}-byte page"
                                    + (" beside the window groups' pages" if any(f is not None for f in bounded) else ""))
        num_pages = int(min(num_pages, (2 ** 31 - 1) // page_size))  # slots are 32-bit
        if num_pages <= 0:
            raise InvalidArgument(f"the cache needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self.group_pages = [num_pages if fixed is None else int(min(fixed, num_pages)) for fixed in bounded]
        self.pools = [BlockPool(n) for n in self.group_pages]
        self.storage = []
        if device is not None:
            import torch
            for g, n in zip(self.groups, self.group_pages):
                self.storage.append(torch.zeros((len(g.entries), 2, n, g.kv_heads, page_size, g.head_dim),
                                                dtype=dtype, device=device))
        self.state_slots = state_slots
        self._live: set[int] = set()

    @property
    def needs_state_slot(self) -> bool:
        """True when some mixer of the model keeps per-request state: a request then runs only with a slot."""
        return self.state_slots is not None and self.state_slots.has_state

    # -- requests
    def new_request(self) -> RequestCache:
        """A request that holds nothing yet: empty tables, no state slot."""
        req = RequestCache([BlockTable() for _ in self.groups], -1)
        self._live.add(id(req))
        return req

    def num_free(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def min_free(self) -> int:
        return min((p.num_free for p in self.pools), default=self.num_pages)

    def pages_needed(self, req: RequestCache, new_len: int) -> list[int]:
        want = blocks_for(new_len, self.page_size)
        return [max(0, want - len(t)) for t in req.tables]

    def _lacks_slot(self, req: RequestCache) -> bool:
        return self.needs_state_slot and req.state_slot < 0

    def holds(self, req: RequestCache) -> bool:
        """Whether preempting the request would give anything back: a page or a state slot."""
        return req.state_slot >= 0 or any(len(t) > t.released for t in req.tables)

    def room(self, req: RequestCache, computed: int) -> int:
        """How many more tokens `req` could hold with its pages plus all free ones
        (src/engine/batch_scheduler.cpp:42-48, the minimum over groups); none if it needs a state slot,
        has none and none is free."""
        if self._lacks_slot(req) and self.state_slots.num_free == 0:
            return 0
        if not self.groups:
            return 2 ** 31
        return min((len(t) + p.num_free) * self.page_size - computed for t, p in zip(req.tables, self.pools))

    def admits(self, tokens: int, keep_free) -> bool:
        """Whether a request that holds nothing can take `tokens` tokens and leave `keep_free[g]` pages of
        every group free (a state slot, where the model needs one, must be free too)."""
        if self.needs_state_slot and self.state_slots.num_free == 0:
            return False
        pages = blocks_for(tokens, self.page_size)
        return all(p.num_free - pages >= keep for p, keep in zip(self.pools, keep_free))

    def reserve(self, req: RequestCache, new_len: int) -> bool:
        """Grows every table to cover new_len tokens and takes a state slot (zeroed) if the request needs one
        and has none; or changes nothing and returns False."""
        if new_len < 0:
            raise InvalidArgument(f"cannot reserve pages for {new_len} tokens")
        if not req.live:
            raise InvalidArgument("cannot reserve for a released request")
        need = self.pages_needed(req, new_len)
        if any(n > p.num_free for n, p in zip(need, self.pools)):
            return False
        if self._lacks_slot(req):
            if self.state_slots.num_free == 0:
                return False
            req.state_slot = self.state_slots.allocate()
        for n, t, p in zip(need, req.tables, self.pools):
            for _ in range(n):
                t.append(p.allocate())
        return True

    def slots(self, req: RequestCache, group: int, old_len: int, new_len: int) -> np.ndarray:
        """Cache slot (page * page_size + offset) of every position in [old_len, new_len); never allocates."""
        if old_len < 0 or new_len < old_len:
            raise InvalidArgument(f"bad token range [{old_len}, {new_len})")
        t = req.tables[group]
        if blocks_for(new_len, self.page_size) > len(t):
            raise InvalidArgument(f"block table of {len(t)} pages cannot hold {new_len} tokens")
        pos = np.arange(old_len, new_len, dtype=np.int64)
        pages = t.ids[pos // self.page_size].astype(np.int64)
        if (pages < 0).any():
            raise InvalidArgument("a position below the window was asked for: its page has been given back")
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def truncate(self, req: RequestCache, length: int) -> None:
        """Gives back the pages beyond those `length` tokens need (a step that did not run)."""
        if length < 0:
            raise InvalidArgument(f"cannot truncate a block table to {length} tokens")
        keep = blocks_for(length, self.page_size)
        for t, p in zip(req.tables, self.pools):
            while t.n > max(keep, t.released):
                t.n -= 1
                p.release(int(t.ids[t.n]))

    def advance_window(self, req: RequestCache, computed: int) -> None:
        """After `computed` tokens are in the cache, window groups give back every page that no
        later query can read: the next query is at position >= computed and reads keys
        > position - window."""
        for g, t, p in zip(self.groups, req.tables, self.pools):
            if g.kind != "window":
                continue
            first_needed = max(0, computed - g.window + 1)
            upto = min(first_needed // self.page_size, t.n)
            while t.released < upto:
                p.release(int(t.ids[t.released]))
                t.ids[t.released] = FREED
                t.released += 1

    def release(self, req: RequestCache) -> None:
        """Everything the request holds goes back: pages of every group and its state slot."""
        if not req.live:
            raise InvalidArgument("request released twice")
        for t, p in zip(req.tables, self.pools):
            for b in t.held():
                p.release(b)
            t.n = 0
            t.released = 0
        if self.state_slots is not None and req.state_slot >= 0:
            self.state_slots.release(req.state_slot)
        req.state_slot = -1
        req.live = False
        self._live.discard(id(req))

    def reset(self, req: RequestCache) -> None:
        """Preemption: pages and state slot go back, the request stays; its next `reserve` starts it again
        from token 0 with a slot handed out zeroed."""
        for t, p in zip(req.tables, self.pools):
            for b in t.held():
                p.release(b)
            t.n = 0
            t.released = 0
        if self.state_slots is not None and req.state_slot >= 0:
            self.state_slots.release(req.state_slot)
        req.state_slot = -1

    # -- what the model sees
    def group_of(self, entry: int) -> int:
        return self._entry_group[entry]

    def has_cache(self, entry: int) -> bool:
        return entry in self._entry_group

    def layer_cache(self, entry: int, writes: bool):
        from ..parts.model import LayerCache
        if entry not in self._entry_group:
            return LayerCache(None, None, -1, False)
        gi, pi = self._entry_group[entry], self._entry_plane[entry]
        st = self.storage[gi]
        return LayerCache(st[pi, 0], st[pi, 1], gi, writes)

    def max_tokens_per_request(self) -> int:
        """The longest a lone request can get: what the groups that keep every key can hold (a window
        group gives pages back as it goes and bounds nothing)."""
        full = [n for g, n in zip(self.groups, self.group_pages) if g.kind == "full"]
        return min(full) * self.page_size if full else 2 ** 31 - 1


def _elem_size(dtype) -> int:
    import torch
    return torch.empty((), dtype=dtype).element_size()
