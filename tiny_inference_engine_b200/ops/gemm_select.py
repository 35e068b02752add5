"""Which matrix-product kernel runs for which operands, and with which tiling.

float32 always runs on the CUDA cores: the 32-bit path has no reduced-precision matrix mode.
bfloat16 runs on the tensor cores (tcgen05) whenever TMA can address the operands (K and the
row strides multiples of 8 elements, 16-byte aligned bases), else on the CUDA cores.
"""
from __future__ import annotations

import functools
import math
import os

import torch

from ..errors import TieError
from .library import call as _call, library as _library

NUM_SMS = 148
_scratch: dict = {}


def tc_takes(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    K = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# Microseconds on one B200, fitted to a sweep of Qwen3-4B's and 8B's products at 160 to 2,048 tokens (8 % mean
# error): a k-block of a 128 x 128 or 128 x 256 tile, the prologue and epilogue of a wave of tiles, and writing
# and reading back a million float partial sums.
_US_K_BLOCK = {128: 0.225, 256: 0.356}
_US_WAVE = {128: 3.2, 256: 7.0}
_US_MEGA_PARTIAL = 0.68


def _plain_cost(M: int, N: int, k_blocks: int, bn: int, splits: int) -> float:
    """Estimated time of the plain tiling: the launcher gives every split NUM_SMS // splits CTAs, each of which
    walks its tiles in turn."""
    per = math.ceil(k_blocks / splits)
    real = math.ceil(k_blocks / per)
    tiles = math.ceil(M / 128) * math.ceil(N / bn)
    ctas = tiles if tiles * real <= NUM_SMS else max(1, NUM_SMS // real)
    waves = math.ceil(tiles / min(ctas, tiles))
    return waves * (per * _US_K_BLOCK[bn] + _US_WAVE[bn]) + (real * M * N / 1e6 * _US_MEGA_PARTIAL if real > 1 else 0.0)


@functools.lru_cache(maxsize=None)
def plan(M: int, N: int, K: int, split_many: bool = True) -> tuple[int, int, int]:
    """(transposed, tile width, splits) for out[M, N] = a[M, K] w[N, K]^T on one CTA per tile.

    Up to 128 tokens the weights take the 128-row side of the MMA and the tokens the narrow side
    (width = the smallest of 16, 32, 64, 128 that holds them): the product is bound by streaming the
    weights, and k is cut into splits so that every SM has a CTA pulling bytes. More tokens: 128-token
    row tiles against 128- or 256-wide weight tiles with k cut into up to four splits, whichever the
    cost estimate above puts first: what matters there is how many waves of tiles the SMs need.
    `split_many` False keeps k whole above 128 tokens (for a consumer that wants the finished product)."""
    k_blocks = math.ceil(K / 64)
    if M <= 128:
        bn = next(b for b in (16, 32, 64, 128) if b >= M)
        tiles = math.ceil(N / 128)
        splits = 1
        if bn <= 64 and tiles < 2 * NUM_SMS:
            # Two CTAs share an SM (the ring is about 100 KB): as many splits as keep all CTAs
            # resident at once, while a split keeps 4 k-blocks and the float partial sums
            # (written and read once) stay well below the weight bytes.
            splits = max(1, min(2 * NUM_SMS // tiles, k_blocks // 4, K // (8 * M)))
        elif bn == 128 and tiles < NUM_SMS:
            splits = max(1, min(NUM_SMS // tiles, k_blocks // 16))      # one CTA per SM at this width
        return 1, bn, splits
    if N <= 128:
        tiles = math.ceil(M / 128)
        bn = next(b for b in (16, 32, 64, 128) if b >= N)
        return 0, bn, max(1, min(NUM_SMS // tiles, k_blocks // 16)) if split_many else 1
    best = None
    for bn in (128, 256):
        for splits in range(1, 5 if split_many else 2):
            if splits > 1 and k_blocks // splits < 8:
                break
            cost = _plain_cost(M, N, k_blocks, bn, splits)
            if best is None or cost < best[0] - 1e-6:
                best = (cost, bn, splits)
    return 0, best[1], best[2]


_retired: list = []


def _scratch_for(numel: int, device) -> torch.Tensor:
    """Scratch for split products whose caller gave none. An outgrown buffer is kept: a captured CUDA graph
    may still use its address."""
    buf = _scratch.get(device)
    if buf is None or buf.numel() < numel:
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(max(numel, 1 << 20, 2 * buf.numel() if buf is not None else 0), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


@functools.lru_cache(maxsize=None)
def partial_capacity(max_rows: int, N: int, K: int, split_many: bool = True) -> int:
    """The most float partial sums a product of up to `max_rows` tokens with these weights leaves
    (splits x tokens x N over every token count): what its scratch buffer is sized for once."""
    most = 0
    for M in range(1, max_rows + 1):
        splits = plan(M, N, K, split_many)[2]
        if splits > 1:
            most = max(most, splits * M * N)
    return most


PAIR_MIN_ROWS = 512     # from this many tokens on, 256 x 256 tiles on pairs of SMs (cta_group::2)


_NO_PAIR = os.environ.get("TIE_NO_PAIR_GEMM") == "1"
_ops = None


def pair_takes(M: int, N: int) -> bool:
    """Pairs of SMs once the 128 x 128 tiles of the product are more than one wave of CTAs."""
    return M >= PAIR_MIN_ROWS and N >= 256 and not _NO_PAIR and math.ceil(M / 128) * math.ceil(N / 128) > NUM_SMS


PAIR_WIDTHS = (256, 224, 192, 160, 128)
# Microseconds of a 256 x width tile per 64-deep k-block, measured at Qwen3-8B's widths: the MMAs of the full width,
# and what staging the operands from L2 costs at any width (the 256 rows of `a` are fetched whatever the width:
# narrow tiles are bound by that, which is why they only pay where they save a whole wave); and per tile the
# prologue and epilogue that nothing hides.
_PAIR_US_MMA, _PAIR_US_FEED, _PAIR_US_TILE = 0.45, 0.33, 3.0
_pairs = None


def resident_pairs() -> int:
    """Pairs of SMs that hold the pair kernel at once (asked of the library once; 74 without a GPU, for planning)."""
    global _pairs
    if _pairs is None:
        try:
            _pairs = int(_library().tie_gemm_tc2_pairs()) or NUM_SMS // 2
        except Exception:       # no GPU, no library: plans are still worth looking at
            return NUM_SMS // 2
    return _pairs


@functools.lru_cache(maxsize=None)
def pair_width(M: int, N: int, K: int, pairs: int) -> int:
    """The tile width of the pair kernel for out[M, N] = a[M, K] w^T: the one whose waves of tiles over `pairs` pairs
    of SMs take the least time by the estimate above; the widest on a tie."""
    tiles_m, k_blocks = math.ceil(M / 256), math.ceil(K / 64)
    best = None
    for bn in PAIR_WIDTHS:
        waves = math.ceil(tiles_m * math.ceil(N / bn) / pairs)
        cost = waves * (k_blocks * max(_PAIR_US_MMA * bn / 256, _PAIR_US_FEED) + _PAIR_US_TILE)
        if best is None or cost < best[0] - 1e-9:
            best = (cost, bn)
    return best[1]


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, transposed=None, bn=None, splits=None, scratch=None,
            silu: bool = False, partial_scratch=None, deep=None, pair=None, checked: bool = False):
    """The tensor-core product; the tiling can be forced (tests). Returns `out`, or a SplitSum when
    `partial_scratch` is given and k is split."""
    global _ops
    if _ops is None:
        from . import SplitSum, _need, _stream, dtype_code      # once: this runs hundreds of times in an eager step
        _ops = (SplitSum, _need, _stream, dtype_code)
    SplitSum, _need, _stream, dtype_code = _ops
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N // 2 if silu else N),
          f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm: last axes must be contiguous")
    _need(checked or tc_takes(a, w, out),
          "gemm_tc: operands must be bfloat16 with K and row strides multiples of 8, 16-byte aligned")
    if pair is None:
        pair = transposed is None and bn is None and splits is None and pair_takes(M, N)
    if pair:
        _call("tie_gemm_tc2", dtype_code(out), a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(0),
              w.stride(0), out.stride(0), 1 if silu else 0, 0, 0, bn if bn in PAIR_WIDTHS else pair_width(M, N, K, resident_pairs()),
              _stream())
        return out
    t, b, s = plan(M, N, K)
    transposed = t if transposed is None else int(transposed)
    bn = b if bn is None else bn
    splits = s if splits is None else splits
    if silu:
        splits = 1
        if not transposed:
            bn = max(bn, 32)
    leave = splits > 1 and partial_scratch is not None
    if leave:
        scratch = partial_scratch(splits * M * N)
    elif splits > 1 and scratch is None:
        scratch = _scratch_for(splits * M * N, a.device)
    _call("tie_gemm_tc", dtype_code(out), a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(0),
          w.stride(0), out.stride(0), transposed, bn, splits, scratch.data_ptr() if splits > 1 else 0, 1 if silu else 0,
          0 if leave else 1, int(deep if deep is not None else (not transposed or bn >= 128)), 0, 0, _stream())
    if leave:
        return SplitSum(scratch, _library().tie_gemm_tc_real_splits(K, splits), M, N)
    return out


def check_status() -> None:
    """After a synchronize: raises if a tensor-core kernel gave up a bounded wait."""
    code = _library().tie_kernel_status()
    if code:
        where = {1: "a matrix product's TMA producer waiting for a free stage", 2: "a matrix product's MMA issuer waiting "
                 "for operands", 3: "a matrix product's epilogue waiting for the accumulator",
                 4: "a CTA of a pair waiting for its partner before it frees its tensor memory",
                 11: "an attention kernel's TMA producer waiting for a free stage",
                 12: "an attention kernel waiting for keys and values"}.get(code, f"code {code}")
        if code == 13:
            raise TieError("decode attention was given fewer splits than a context needs; that sequence's output was not written")
        raise TieError(f"a kernel gave up after its wait limit ({where}); its output is invalid")


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, partial_scratch=None):
    from . import gemm_simt
    if a.shape[0] == 0:
        return out
    if tc_takes(a, w, out):
        return gemm_tc(a, w, out, partial_scratch=partial_scratch, checked=True)
    gemm_simt(a, w, out)
    return out


def gemm_silu(a: torch.Tensor, w_blocks: torch.Tensor, out: torch.Tensor) -> None:
    from . import _need
    _need(w_blocks.shape[0] % 32 == 0 and tc_takes(a, w_blocks, out),
          "gemm_silu: needs bfloat16 operands TMA can address and gate/up rows in blocks of 16")
    if a.shape[0] > 0:
        gemm_tc(a, w_blocks, out, silu=True)


class BoundGemm:
    """out = a . w^T for one weight matrix, checked once: what the parts call hundreds of times a step.

    The weight's address, sizes and kernel family are fixed when the part binds its tensors; a call looks up
    the tiling of its token count (computed once per count) and goes straight to the launcher. `a` and `out`
    come from the step's workspace: rows contiguous, 16-byte aligned, the compute dtype (the parts' contract);
    anything the tensor-core kernels do not take falls back to `gemm` with its full checks.

    A weight that the tensor-core kernels take is kept in k-blocks (`ops.pack_k_blocks`, with `pack`): `.w` is then
    [ceil(K / 64), rows, 64] and `packed_rows` its number of rows; `.rows(a, b)` gives the product with a slice of
    its rows (the q rows of a stacked q/k/v weight) over the same memory."""

    def __init__(self, w: torch.Tensor, silu: bool = False, split_many: bool = True, pack: bool = True, _slice=None):
        self.silu, self.split_many = silu, split_many
        if _slice is not None:              # rows [row0, row0 + N) of a packed weight
            parent, row0, n = _slice
            self.w, self.N, self.K, self.packed_rows, self.row0, self.fast = parent.w, n, parent.K, parent.packed_rows, row0, True
        else:
            self.N, self.K = w.shape
            self.fast = (w.dtype == torch.bfloat16 and w.stride(1) == 1 and self.K % 8 == 0 and w.stride(0) % 8 == 0
                         and w.data_ptr() % 16 == 0 and (not silu or self.N % 32 == 0))
            self.packed_rows = self.row0 = 0
            if pack and self.fast and w.is_cuda:
                from . import pack_k_blocks
                w = pack_k_blocks(w)
                self.packed_rows = self.N
            self.w = w
        self.w_ptr, self.ldw = self.w.data_ptr(), (64 if self.packed_rows else self.w.stride(0))
        self._plans: dict[int, tuple] = {}

    def rows(self, begin: int, end: int) -> "BoundGemm":
        """The product with rows begin..end-1 of this weight (no SiLU epilogue)."""
        if not 0 <= begin < end <= self.N:
            raise ValueError(f"rows {begin}..{end} of a weight of {self.N} rows")
        if self.packed_rows:
            return BoundGemm(None, False, self.split_many, _slice=(self, self.row0 + begin, end - begin))
        return BoundGemm(self.w[begin:end], False, self.split_many, pack=False)

    def row_major(self) -> torch.Tensor:
        """The weight as [N, K] (a copy if it is kept in k-blocks): for callers that need it the plain way."""
        if not self.packed_rows:
            return self.w
        from . import unpack_k_blocks
        return unpack_k_blocks(self.w, self.K)[self.row0:self.row0 + self.N]

    def _plan(self, M: int):
        pair = pair_takes(M, self.N)
        t, bn, splits = plan(M, self.N, self.K, self.split_many)
        if self.silu:
            splits = 1
            if not t:
                bn = max(bn, 32)
        real = _library().tie_gemm_tc_real_splits(self.K, splits) if splits > 1 else 1
        if pair:
            bn = pair_width(M, self.N, self.K, resident_pairs())
        p = (pair, t, bn, splits, int(not t or bn >= 128), real)
        self._plans[M] = p
        return p

    def __call__(self, a: torch.Tensor, out: torch.Tensor, partial_scratch=None):
        M = a.shape[0]
        if M == 0:
            return out
        if not (self.fast and a.dtype == torch.bfloat16 and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
                and out.stride(1) == 1 and a.shape[1] == self.K and out.shape[1] == (self.N // 2 if self.silu else self.N)
                and out.shape[0] == M and out.dtype in (torch.bfloat16, torch.float32)):
            w = self.row_major()
            if self.silu:
                gemm_silu(a, w, out)
                return out
            return gemm(a, w, out, partial_scratch)
        global _ops
        if _ops is None:
            from . import SplitSum, _need, _stream, dtype_code
            _ops = (SplitSum, _need, _stream, dtype_code)
        SplitSum, _, _stream, dtype_code = _ops
        pair, t, bn, splits, deep, real = self._plans.get(M) or self._plan(M)
        code = 1 if out.dtype == torch.bfloat16 else 0
        if pair:
            _call("tie_gemm_tc2", code, a.data_ptr(), self.w_ptr, out.data_ptr(), M, self.N, self.K, a.stride(0), self.ldw,
                  out.stride(0), 1 if self.silu else 0, self.packed_rows, self.row0, bn, _stream())
            return out
        leave = splits > 1 and partial_scratch is not None
        scratch = 0
        if leave:
            buf = partial_scratch(splits * M * self.N)
            scratch = buf.data_ptr()
        elif splits > 1:
            buf = _scratch_for(splits * M * self.N, a.device)
            scratch = buf.data_ptr()
        _call("tie_gemm_tc", code, a.data_ptr(), self.w_ptr, out.data_ptr(), M, self.N, self.K, a.stride(0), self.ldw, out.stride(0),
              t, bn, splits, scratch, 1 if self.silu else 0, 0 if leave else 1, deep, self.packed_rows, self.row0, _stream())
        if leave:
            return SplitSum(buf, real, M, self.N)
        return out
