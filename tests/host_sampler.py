"""The sampler on the host: what the sampling kernels compute, restated with numpy in the kernels' own
precision (float32 weights, sums in double). The engine samples on the device (greedy, temperature, top-k
and top-p run in kernels inside the step); this function is what the tests hold those kernels against.

It restates the reference's sampler (src/sampling/sampler.cpp:18-81): NaN or empty
logits and all -inf are errors, a +inf logit is certain, greedy is the first maximum,
otherwise shift by the maximum and scale by 1/T, keep the top_k most likely (ties by id),
then the smallest prefix whose weight reaches top_p of the total, and walk the candidates
with a uniform draw in [0, total).
"""
from __future__ import annotations

import numpy as np

from tiny_inference_engine_b200.errors import InvalidArgument
from tiny_inference_engine_b200.sampling import SamplingParams, uniform


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
        keep = min(int(np.searchsorted(cum, float(np.float32(params.top_p)) * total, side="left")) + 1, weights.size)
        weights, total = weights[:keep], float(cum[keep - 1])
    r = uniform(params.seed, index) * total
    cum = np.cumsum(weights)
    pick = min(int(np.searchsorted(cum, r, side="right")), weights.size - 1)
    return int(order[pick]) if order is not None else pick
