"""Standard normal values from a counter: value i of stream (seed, ordinal) is a pure function of
(seed, ordinal, i), the same bits on the CPU and on the GPU.

Philox4x32-10 (the generator the sampling kernels use) keyed by (seed, ordinal), counter = i // 4, gives
four 32-bit words, that is two pairs of uniforms, and Box-Muller turns each pair into two normal values:
sqrt(-2 ln u1) * (cos, sin)(2 pi u2). So that both devices agree to the last bit, ln, cos and sin are
worked out here from additions, multiplications, divisions and a square root in float64, each its own
torch operation (no fused multiply-add), which IEEE 754 rounds the same way everywhere; the math
libraries of a CPU and a GPU do not promise that for their own log and cos.
"""
from __future__ import annotations

import math

import torch

_M0, _M1, _W0, _W1, _MASK = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF


def _philox4x32_10(counter: torch.Tensor, key0: int, key1: int):
    """counter: int64 tensor of values below 2^63 -> four int64 tensors holding 32-bit words.
    Products of two 32-bit values wrap in int64 with the bit pattern of the unsigned product."""
    c0, c1 = counter & _MASK, (counter >> 32) & _MASK
    c2, c3 = torch.zeros_like(c0), torch.zeros_like(c0)
    k0, k1 = key0 & _MASK, key1 & _MASK
    for _ in range(10):
        p0, p1 = c0 * _M0, c2 * _M1
        c0, c1, c2, c3 = ((p1 >> 32) & _MASK) ^ c1 ^ k0, p1 & _MASK, ((p0 >> 32) & _MASK) ^ c3 ^ k1, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def _ln(u: torch.Tensor) -> torch.Tensor:
    """Natural logarithm of float64 values in (0, 1): u = m * 2^e with m in [sqrt(1/2), sqrt(2)),
    ln m = 2 atanh(z), z = (m - 1) / (m + 1), |z| < 0.172, by its series in z^2."""
    m, e = torch.frexp(u)                       # m in [0.5, 1), exact
    low = m < math.sqrt(0.5)
    m = torch.where(low, m * 2.0, m)
    e = (e - low.to(e.dtype)).to(torch.float64)
    z = (m - 1.0) / (m + 1.0)
    z2 = z * z
    s = torch.full_like(z, 1.0 / 25.0)
    for k in range(23, 0, -2):                  # 1/23, 1/21, ..., 1: z^24 / 25 is below 2e-20
        s = s * z2 + (1.0 / k)
    return e * math.log(2.0) + (z * s) * 2.0


def _cos_sin_turns(u: torch.Tensor):
    """(cos, sin)(2 pi u) for float64 u in [0, 1): the quarter turn is taken off exactly, the rest
    (an angle in [0, pi/2)) goes through the Taylor series of both."""
    t = u * 4.0
    q = torch.floor(t)
    x = (t - q) * (math.pi / 2.0)
    x2 = x * x
    c = torch.full_like(x, 1.0 / math.factorial(22))
    s = torch.full_like(x, 1.0 / math.factorial(23))
    for k in range(20, -1, -2):
        sign = -1.0                              # alternating series, Horner from the far end
        c = c * x2 * sign + (1.0 / math.factorial(k))
        s = s * x2 * sign + (1.0 / math.factorial(k + 1))
    s = s * x
    qi = q.to(torch.int64)
    cos = torch.where(qi == 0, c, torch.where(qi == 1, -s, torch.where(qi == 2, -c, s)))
    sin = torch.where(qi == 0, s, torch.where(qi == 1, c, torch.where(qi == 2, -s, -c)))
    return cos, sin


def standard_normal(seed: int, ordinal: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """Values start .. start + count - 1 of stream (seed, ordinal) as float64 on `device`."""
    if count <= 0:
        return torch.empty(0, dtype=torch.float64, device=device)
    first, last = start // 4, (start + count - 1) // 4
    counter = torch.arange(first, last + 1, dtype=torch.int64, device=device)
    key0 = (seed ^ (ordinal * 0x9E3779B1)) & _MASK
    key1 = ((seed >> 32) ^ (ordinal >> 3) ^ 0x5851F42D) & _MASK
    words = _philox4x32_10(counter, key0, key1)
    out = torch.empty((last - first + 1, 4), dtype=torch.float64, device=device)
    for pair in range(2):
        u1 = (words[2 * pair].to(torch.float64) + 0.5) * (1.0 / 4294967296.0)
        u2 = words[2 * pair + 1].to(torch.float64) * (1.0 / 4294967296.0)
        r = torch.sqrt(_ln(u1) * -2.0)
        c, s = _cos_sin_turns(u2)
        out[:, 2 * pair], out[:, 2 * pair + 1] = r * c, r * s
    return out.reshape(-1)[start - 4 * first:start - 4 * first + count]
