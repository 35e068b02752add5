"""Sampling: the device kernel for greedy and temperature, and the host path with top-k and top-p.

The host path restates the reference's sampler (src/sampling/sampler.cpp:18-81): NaN or empty
logits and all -inf are errors, a +inf logit is certain, greedy is the first maximum,
otherwise shift by the maximum and scale by 1/T, keep the top_k most likely (ties by id),
then the smallest prefix whose weight reaches top_p of the total, and walk the candidates
with a uniform draw in [0, total).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..errors import InvalidArgument
from .params import SamplingParams
from .philox import uniform


def sample_host(logits: np.ndarray, params: SamplingParams, index: int) -> int:
    z = np.asarray(logits, dtype=np.float32)
    if z.size == 0:
        raise InvalidArgument("cannot sample from empty logits")
    nan = np.flatnonzero(np.isnan(z))
    if nan.size:
        raise InvalidArgument(f"logit {int(nan[0])} is NaN")
    best = int(np.argmax(z))  # first maximum
    if z[best] == -np.inf:
        raise InvalidArgument("all logits are -inf")
    inv_t = params.inv_temperature()
    if inv_t == 0.0 or z[best] == np.inf:
        return best
    scaled = (z - z[best]) * np.float32(inv_t)
    n, keep = z.size, z.size
    order = None
    if 0 < params.top_k < n or params.top_p < 1.0:
        order = np.lexsort((np.arange(n), -scaled))  # most likely first, ties by id
        if 0 < params.top_k < n:
            keep = params.top_k
        cand = scaled[order[:keep]]
    else:
        cand = scaled
    weights = np.exp(cand - cand.max()).astype(np.float32).astype(np.float64)
    total = float(weights.sum())
    if params.top_p < 1.0:
        cum = np.cumsum(weights)
        keep = min(int(np.searchsorted(cum, np.float32(params.top_p) * total, side="left")) + 1, weights.size)
        weights, total = weights[:keep], float(cum[keep - 1])
    r = uniform(params.seed, index) * total
    cum = np.cumsum(weights)
    pick = min(int(np.searchsorted(cum, r, side="right")), weights.size - 1)
    return int(order[pick]) if order is not None else pick


class Sampler:
    """Samples one token for each row of a step's logits; rows of requests with top-k or top-p
    come back to the host, the others are picked by the kernel and only their ids come back."""

    def __init__(self, max_rows: int, device="cuda"):
        self.max_rows = max_rows
        self._ids = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._ids_host = torch.empty(max_rows, dtype=torch.int32, pin_memory=True)
        self._inv_t = torch.empty(max_rows, dtype=torch.float32, pin_memory=True)
        self._seeds = torch.empty(max_rows, dtype=torch.int64, pin_memory=True)
        self._counters = torch.empty(max_rows, dtype=torch.int64, pin_memory=True)
        self._inv_t_d = torch.empty(max_rows, dtype=torch.float32, device=device)
        self._seeds_d = torch.empty(max_rows, dtype=torch.int64, device=device)
        self._counters_d = torch.empty(max_rows, dtype=torch.int64, device=device)

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], indices: list[int]) -> list[int]:
        """logits [R, V] float32 on the device; params[r] and indices[r] (how many tokens request r
        has generated so far) per row."""
        R = logits.shape[0]
        if R == 0:
            return []
        greedy_only = all(p.temperature == 0.0 for p in params)
        inv_np, seeds_np, ctr_np = self._inv_t.numpy(), self._seeds.numpy(), self._counters.numpy()
        if greedy_only:
            ops.sample(logits, self._ids)
        else:
            for r, (p, i) in enumerate(zip(params, indices)):
                inv_np[r] = p.inv_temperature()
                seeds_np[r] = np.array(p.seed, dtype=np.uint64).view(np.int64)
                ctr_np[r] = i
            self._inv_t_d[:R].copy_(self._inv_t[:R], non_blocking=True)
            self._seeds_d[:R].copy_(self._seeds[:R], non_blocking=True)
            self._counters_d[:R].copy_(self._counters[:R], non_blocking=True)
            ops.sample(logits, self._ids, self._inv_t_d, self._seeds_d, self._counters_d)
        self._ids_host[:R].copy_(self._ids[:R], non_blocking=True)
        host_rows = [r for r, p in enumerate(params) if not p.on_device]
        host_logits = logits[host_rows].cpu().numpy() if host_rows else None   # synchronizes
        torch.cuda.current_stream().synchronize()
        out = self._ids_host[:R].tolist()
        for j, r in enumerate(host_rows):
            out[r] = sample_host(host_logits[j], params[r], indices[r])
        return out
