"""Philox4x32-10 on the host, the same generator the sampling kernel runs: key = the request's
seed (low and high word), counter = the index of the generated token. A draw needs no state,
so it cannot depend on batching, on how a prompt was cut, or on a preemption in between.
(The reference keeps one std::mt19937_64 per sequence: src/engine/sequence.h:22.)"""
from __future__ import annotations

_M0, _M1, _W0, _W1, _MASK = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF


def philox4x32(counter, key, rounds: int = 10):
    c0, c1, c2, c3 = (int(v) & _MASK for v in counter)
    k0, k1 = (int(v) & _MASK for v in key)
    for _ in range(rounds):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def uniform(seed: int, index: int) -> float:
    """Uniform in [0, 1) with 24 bits, for generated token `index` of a request seeded `seed`."""
    r = philox4x32((index & _MASK, (index >> 32) & _MASK, 0, 0), (seed & _MASK, (seed >> 32) & _MASK))
    return (r[0] >> 8) * (1.0 / (1 << 24))
