"""Python faces of the CUDA kernels: shape and dtype checks, then one launch on the current stream.

Tensors are torch CUDA tensors used as typed device memory; nothing here computes with torch.
"""
from __future__ import annotations

import os

import torch

from ..errors import InvalidArgument
from . import library
from .library import call, check_device

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise InvalidArgument(f"dtype {t.dtype} is not one of float32, bfloat16") from None


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX = None


def _stream() -> int:
    """The current stream's handle. (torch.cuda.current_stream() builds a Stream object each time, several
    microseconds per kernel launch; the raw accessor does not.)"""
    global _DEVICE_INDEX
    if _RAW_STREAM is None:
        return torch.cuda.current_stream().cuda_stream
    if _DEVICE_INDEX is None:
        _DEVICE_INDEX = torch.cuda.current_device()
    return _RAW_STREAM(_DEVICE_INDEX)


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise InvalidArgument(msg)


def _dev(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise InvalidArgument("kernel arguments must be CUDA tensors: the engine has no CPU path")


class SplitSum:
    """The result of a matrix product whose k range was cut into splits, not yet added up:
    float32 partial sums [splits, M, N] in scratch memory. Kernels that consume it (the residual
    add + norm, the q/k norm + RoPE + append) add the splits in order while they read, which saves
    a reduction kernel and a rounding; `materialize` adds them into a tensor for everyone else."""

    def __init__(self, partial: torch.Tensor, splits: int, M: int, N: int):
        self.partial, self.splits, self.M, self.N = partial, splits, M, N

    @property
    def stride(self) -> int:
        return self.M * self.N

    def materialize(self, out: torch.Tensor) -> torch.Tensor:
        p = self.partial[:self.splits * self.stride].view(self.splits, self.M, self.N)
        out.copy_(p.sum(dim=0) if self.splits > 1 else p[0])   # off the product path: toy parts and tests only
        return out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = float(table[ids[t]]); out is the float32 residual stream [T, D]. The table is [V, D], or the
    same in k-blocks, [ceil(D / 64), V, 64] (`pack_k_blocks`: what a tied output table is stored as)."""
    _dev(table, ids, out)
    T, D = out.shape
    packed = table.dim() == 3
    _need(table.is_contiguous() and ((not packed and table.dim() == 2 and table.shape[1] == D) or
                                     (packed and table.shape[2] == 64 and table.shape[0] == (D + 63) // 64)),
          "embed: table must be [V, D] or [ceil(D / 64), V, 64], contiguous")
    _need(ids.dtype == torch.int32 and ids.numel() == T and ids.is_contiguous(), "embed: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.is_contiguous(), "embed: output must be float32 contiguous")
    V = table.shape[1] if packed else table.shape[0]
    call("tie_embed", dtype_code(table), table.data_ptr(), ids.data_ptr(), out.data_ptr(), T, D, V, V if packed else 0, _stream())


def pack_k_blocks(w: torch.Tensor) -> torch.Tensor:
    """[N, K] -> [ceil(K / 64), N, 64]: the rows' first 64 columns, then their next 64, and so on (zeros beyond K).
    The tensor-core products load a weight in boxes of 128 rows x 64 columns; stored like this a box is one piece
    of 16 KB instead of 128 pieces of 128 bytes a row apart, which is what the memory streams fastest."""
    N, K = w.shape
    kb = (K + 63) // 64
    if K % 64:
        w = torch.nn.functional.pad(w, (0, kb * 64 - K))
    return w.view(N, kb, 64).permute(1, 0, 2).contiguous()


def unpack_k_blocks(packed: torch.Tensor, K: int) -> torch.Tensor:
    """The inverse of pack_k_blocks: [ceil(K / 64), N, 64] -> [N, K] (a copy)."""
    kb, N, _ = packed.shape
    return packed.permute(1, 0, 2).reshape(N, kb * 64)[:, :K].contiguous()


def scatter_ids(tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, ids: torch.Tensor, n: int) -> None:
    """tokens[dst[i]] = ids[src[i]] for i < n (all int32): sampled ids of the step before become input tokens of
    this one without a trip to the host."""
    _dev(tokens, dst, src, ids)
    _need(all(t.dtype == torch.int32 and t.is_contiguous() for t in (tokens, dst, src, ids)) and
          0 <= n <= min(dst.numel(), src.numel()), "scatter_ids: int32 contiguous arrays, n within dst and src")
    call("tie_scatter_ids", tokens.data_ptr(), dst.data_ptr(), src.data_ptr(), ids.data_ptr(), n, _stream())


def add_rmsnorm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor, rows=None) -> None:
    """x += delta (when given; float32, in place), out = rmsnorm(x) * weight in out's dtype.
    With `rows` (int32 [R]), out[i] comes from row rows[i] and x is left as it is. `delta` may
    be a SplitSum: its splits are added in order while they are read."""
    part = None
    if isinstance(delta, SplitSum):
        part, delta = delta, None
        _need(part.M == x.shape[0] and part.N == x.shape[-1], "add_rmsnorm: partial sums do not match x")
    _dev(x, delta, weight, out, rows)
    D = x.shape[-1]
    n = out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_rmsnorm: x must be float32 contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == D, "add_rmsnorm: weight must be float32 [D]")
    _need(out.shape[-1] == D and out.is_contiguous(), "add_rmsnorm: out must be [n, D] contiguous")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.shape == x.shape and delta.is_contiguous(),
              "add_rmsnorm: delta must match x's shape and out's dtype")
    if rows is None:
        _need(n == x.shape[0], "add_rmsnorm: out must have x's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() == n, "add_rmsnorm: rows must be int32 [n]")
    call("tie_add_rmsnorm", dtype_code(out), x.data_ptr(), _ptr(delta), part.partial.data_ptr() if part else 0,
         part.stride if part else 0, part.splits if part else 0, _ptr(rows), weight.data_ptr(), float(eps), out.data_ptr(),
         n, D, _stream())


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """RMSNorm over the last axis of a 2-D view whose rows may be strided (last axis contiguous)."""
    _dev(x, weight, out)
    _need(x.dim() == 2 and out.shape == x.shape and x.dtype == out.dtype, "rmsnorm_rows: x and out must be 2-D alike")
    _need(x.stride(1) == 1 and out.stride(1) == 1, "rmsnorm_rows: last axis must be contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == x.shape[1], "rmsnorm_rows: weight must be float32 [size]")
    call("tie_rmsnorm_rows", dtype_code(x), x.data_ptr(), x.stride(0), weight.data_ptr(), float(eps), out.data_ptr(),
         out.stride(0), x.shape[1], x.shape[0], _stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _dev(gate_up, out)
    T, I = out.shape
    _need(gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous() and
          gate_up.dtype == out.dtype, "silu_mul: gate_up must be [T, 2I] and out [T, I], same dtype, contiguous")
    call("tie_silu_mul", dtype_code(out), gate_up.data_ptr(), out.data_ptr(), T, I, _stream())


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, heads: int, head_dim: int) -> None:
    """Rotate-half RoPE in place over the first 2*len(inv_freq) dims of each head of x [T, >= heads*head_dim]."""
    _dev(x, positions, inv_freq)
    _need(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= heads * head_dim, "rope: x must be [T, heads*head_dim]")
    _need(positions.dtype == torch.int32 and positions.numel() == x.shape[0], "rope: positions must be int32 [T]")
    _need(inv_freq.dtype == torch.float32, "rope: inv_freq must be float32")
    call("tie_rope", dtype_code(x), x.data_ptr(), x.stride(0), positions.data_ptr(), inv_freq.data_ptr(), x.shape[0],
         heads, head_dim, 2 * inv_freq.numel(), _stream())


def _check_planes(k_cache, v_cache, kv_heads, head_dim):
    _need(k_cache.dim() == 4 and k_cache.shape == v_cache.shape and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "cache planes must be [pages, kv_heads, page_size, head_dim] contiguous")
    _need(k_cache.shape[1] == kv_heads and k_cache.shape[3] == head_dim, "cache planes do not match the heads")
    _need(k_cache.numel() // head_dim < 2 ** 31, "cache plane too large for 32-bit row indices")


def kv_append(k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """k, v [T, kv_heads*head_dim] (rows may be strided) into the planes at slots[t]; slot < 0 writes nothing."""
    _dev(k, v, slots, k_cache, v_cache)
    kv_heads, page_size, head_dim = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    _check_planes(k_cache, v_cache, kv_heads, head_dim)
    _need(k.shape == v.shape and k.shape[1] == kv_heads * head_dim and k.stride(1) == 1 and v.stride(1) == 1,
          "kv_append: k and v must be [T, kv_heads*head_dim]")
    _need(k.dtype == k_cache.dtype and v.dtype == k_cache.dtype, "kv_append: dtype differs from the cache's")
    _need(slots.dtype == torch.int32 and slots.numel() == k.shape[0], "kv_append: slots must be int32 [T]")
    call("tie_kv_append", dtype_code(k), k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), slots.data_ptr(),
         k_cache.data_ptr(), v_cache.data_ptr(), k.shape[0], kv_heads, head_dim, page_size, _stream())


def qk_norm_rope_append(qkv: torch.Tensor, q_weight, k_weight, q_eps: float, k_eps: float, inv_freq,
                        positions: torch.Tensor, slots, k_cache, v_cache, q_heads: int, kv_heads: int,
                        head_dim: int, write_kv: bool = True, partial: SplitSum | None = None) -> None:
    """Per-head RMSNorm of q and k (weights may be None), RoPE (inv_freq may be None), q back in
    place, k and v into the cache planes. qkv is [T, (q_heads + 2 kv_heads) * head_dim]; with
    write_kv False it may hold q only and the planes are not touched. With `partial` the values
    are read from the split product's partial sums [splits, T, width] and only q is written to qkv."""
    _dev(qkv, q_weight, k_weight, inv_freq, positions, slots, k_cache, v_cache)
    T = qkv.shape[0]
    width = (q_heads + (2 * kv_heads if write_kv else 0)) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= width, "qk_norm_rope_append: qkv too narrow")
    _need(positions.dtype == torch.int32 and positions.numel() == T, "qk_norm_rope_append: positions must be int32 [T]")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == head_dim),
              "qk_norm_rope_append: norm weights must be float32 [head_dim]")
    rot = 0
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32, "qk_norm_rope_append: inv_freq must be float32")
        rot = 2 * inv_freq.numel()
    page_size = 1
    if write_kv:
        _check_planes(k_cache, v_cache, kv_heads, head_dim)
        _need(k_cache.dtype == qkv.dtype, "qk_norm_rope_append: dtype differs from the cache's")
        _need(slots.dtype == torch.int32 and slots.numel() == T, "qk_norm_rope_append: slots must be int32 [T]")
        page_size = k_cache.shape[2]
    if partial is not None:
        _need(partial.M == T and partial.N == width, "qk_norm_rope_append: partial sums do not match the rows")
    call("tie_qk_norm_rope_append", dtype_code(qkv), qkv.data_ptr(), qkv.stride(0),
         partial.partial.data_ptr() if partial else 0, partial.stride if partial else 0, partial.splits if partial else 0,
         partial.N if partial else 0, _ptr(q_weight), _ptr(k_weight),
         float(q_eps), float(k_eps), _ptr(inv_freq), rot, positions.data_ptr(), _ptr(slots) if write_kv else 0,
         _ptr(k_cache) if write_kv else 0, _ptr(v_cache) if write_kv else 0, T, q_heads, kv_heads, head_dim, page_size,
         1 if write_kv else 0, _stream())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] . w[N, K]^T on the CUDA cores with float accumulation (any sizes)."""
    _dev(a, w, out)
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm: operands must be 2-D")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm: last axes must be contiguous")
    _need(a.dtype == w.dtype, "gemm: a and w must have one dtype")
    call("tie_gemm_simt", dtype_code(a), dtype_code(out), a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K,
         a.stride(0), w.stride(0), out.stride(0), _stream())


def _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim):
    _check_planes(k_cache, v_cache, kv_heads, head_dim)
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= q_heads * head_dim, "attention: q too narrow")
    _need(out.shape == (q.shape[0], q_heads * head_dim) and out.is_contiguous(), "attention: out must be [T, Hq*Dh]")
    _need(q.dtype == k_cache.dtype and out.dtype == q.dtype, "attention: q, cache and out must have one dtype")
    S = context_lens.numel()
    _need(query_start.dtype == torch.int32 and query_start.numel() == S + 1, "attention: query_start must be int32 [S+1]")
    _need(context_lens.dtype == torch.int32, "attention: context_lens must be int32 [S]")
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.shape[0] == S and
          block_tables.is_contiguous(), "attention: block_tables must be int32 [S, max_blocks]")
    return S


def attention_rows(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_heads, kv_heads,
                   head_dim, scale: float, window: int = 0) -> None:
    """Causal attention of every row of the step over the paged cache (CUDA cores)."""
    _dev(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables)
    S = _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(seq_of_row.dtype == torch.int32 and seq_of_row.numel() == q.shape[0], "attention: seq_of_row must be int32 [T]")
    call("tie_attention_rows", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         out.data_ptr(), seq_of_row.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[1], q.shape[0], S, q_heads, kv_heads, head_dim, k_cache.shape[2], int(window), float(scale),
         _stream())


def attention_split_scratch_floats(n_list: int, q_heads: int, head_dim: int, max_splits: int) -> int:
    return n_list * q_heads * max_splits * (head_dim + 2)


def attention_split(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim,
                    scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch,
                    window: int = 0) -> None:
    """Attention of sequences that bring one token each, their keys cut into splits of `split_keys`."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch)
    S = _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "attention: seq_list must be int32 [n_list]")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    call("tie_attention_split", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
         S, q_heads, kv_heads, head_dim, k_cache.shape[2], int(window), float(scale), seq_list.data_ptr(), n_list,
         split_keys, max_splits, scratch.data_ptr(), _stream())


def attention_tc_takes(q: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernels take these operands (else the CUDA-core ones do)."""
    return (q.dtype == torch.bfloat16 and head_dim in (64, 128, 256) and q_heads // kv_heads <= 16 and
            q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_prompt_tc(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                        q_heads, kv_heads, head_dim, scale: float, window: int = 0) -> None:
    """Tensor-core attention of the first n_seqs sequences of the step (each brings several tokens;
    their rows come first); max_queries is the most tokens one of them brings."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    call("tie_attention_prompt_tc", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs,
         max_queries, q_heads, kv_heads, head_dim, k_cache.shape[2], int(window), float(scale), _stream())


def attention_decode_tc(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim,
                        scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch,
                        window: int = 0) -> None:
    """Tensor-core attention of sequences that bring one token each: split kernel, then the merge."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "attention: seq_list must be int32 [n_list]")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    call("tie_attention_decode_tc", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], q_heads, kv_heads,
         head_dim, k_cache.shape[2], int(window), float(scale), seq_list.data_ptr(), n_list, split_keys, max_splits,
         scratch.data_ptr(), _stream())
    call("tie_attention_merge", dtype_code(out), out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), q_heads,
         head_dim, int(window), seq_list.data_ptr(), n_list, split_keys, max_splits, scratch.data_ptr(), _stream())


def attention_decode_tma_takes(q: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the TMA-fed attention kernels (decode and prompt) take these operands."""
    return attention_tc_takes(q, q_heads, kv_heads, head_dim) and page_size >= 8 and page_size & (page_size - 1) == 0


def attention_prompt_tma(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                         q_heads, kv_heads, head_dim, scale: float, window: int = 0) -> None:
    """As attention_prompt_tc, keys and values fed by TMA (pages that are powers of two from 8 up)."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    call("tie_attention_prompt_tma", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs,
         max_queries, q_heads, kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _stream())


_NO_UMMA_ATTENTION = os.environ.get("TIE_NO_UMMA_ATTENTION") == "1"
UMMA_MIN_ROWS = 128     # rows (queries x heads of a group) from which the tcgen05 prompt kernel pays


def attention_prompt_umma_takes(q: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, page_size: int,
                                max_queries: int) -> bool:
    """Whether the tcgen05 prompt kernel takes these operands and the portions are long enough for its
    256-row tiles."""
    return (attention_decode_tma_takes(q, q_heads, kv_heads, head_dim, page_size) and head_dim in (64, 128)
            and max_queries * (q_heads // kv_heads) >= UMMA_MIN_ROWS and not _NO_UMMA_ATTENTION)


def attention_prompt_umma(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                          q_heads, kv_heads, head_dim, scale: float, window: int = 0) -> None:
    """As attention_prompt_tma with both products on tcgen05 and the accumulators in tensor memory
    (head sizes 64 and 128)."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(out.is_contiguous(), "attention: out must be contiguous")
    call("tie_attention_prompt_umma", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs,
         max_queries, q_heads, kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _stream())


CLUSTER_SPLITS = (2, 4, 8, 16)      # how many splits the decode attention merges as one thread-block cluster


def attention_decode_tma(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim,
                         scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch, counters,
                         window: int = 0, cluster: bool = False) -> None:
    """Attention of sequences that bring one token each, keys and values fed by TMA, splits merged by
    the last CTA to finish. `counters` (int32 [>= n_list * kv_heads]) must be zero; it is left zero.
    `cluster` (with max_splits in CLUSTER_SPLITS): the splits of a sequence and kv head run as one thread-block
    cluster and merge through shared memory, which is faster where all the launch's CTAs are resident at once.
    `seq_list`: int32 [n_list], or an int: the first of n_list sequences in a row (the kernel then has one load
    less to wait for before it can ask for keys)."""
    first = seq_list if isinstance(seq_list, int) else 0
    seq_list = None if isinstance(seq_list, int) else seq_list
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch, counters)
    S = _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need((seq_list is None and 0 <= first and first + n_list <= S) or
          (seq_list is not None and seq_list.dtype == torch.int32 and seq_list.numel() >= n_list),
          "attention: seq_list must be int32 [n_list], or the first of n_list sequences in a row")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    _need(counters.dtype == torch.int32 and counters.numel() >= n_list * kv_heads, "attention: counters too small")
    call("tie_attention_decode_tma", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], q_heads, kv_heads,
         head_dim, k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _ptr(seq_list), first, n_list, split_keys,
         max_splits, scratch.data_ptr(), counters.data_ptr(), 1 if cluster else 0, _stream())


def attention_decode_prep_takes(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, page_size: int, inv_freq) -> bool:
    """Whether the decode attention that prepares its own heads takes these operands: what the TMA-fed kernel takes,
    and a rotation (if any) over the whole head."""
    return (attention_decode_tma_takes(qkv, q_heads, kv_heads, head_dim, page_size)
            and (inv_freq is None or 2 * inv_freq.numel() == head_dim))


def attention_decode_prep(qkv, q_weight, k_weight, q_eps: float, k_eps: float, inv_freq, positions, k_cache, v_cache, out,
                          query_start, context_lens, block_tables, q_heads, kv_heads, head_dim, scale: float, seq_list,
                          n_list: int, split_keys: int, max_splits: int, scratch, counters, window: int = 0,
                          append: bool = True, partial: SplitSum | None = None, cluster: bool = False) -> None:
    """`attention_decode_tma` for a step in which every sequence brings one token, straight from the q/k/v product's
    output: qkv [T, (q_heads + 2 kv_heads) * head_dim] (or q only, with `append` False), or the product's partial sums.
    The kernel does what `qk_norm_rope_append` does to the group's query heads and, with `append`, to the newest
    key and value, which it stores in the cache planes and uses; qkv itself is left as it is."""
    first = seq_list if isinstance(seq_list, int) else 0
    seq_list = None if isinstance(seq_list, int) else seq_list
    _dev(qkv, q_weight, k_weight, inv_freq, positions, k_cache, v_cache, out, query_start, context_lens, block_tables,
         seq_list, scratch, counters)
    T = qkv.shape[0]
    width = (q_heads + (2 * kv_heads if append else 0)) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= width and qkv.dtype == torch.bfloat16,
          "attention_decode_prep: qkv must be bfloat16 rows of q (and k, v)")
    _need(out.shape == (T, q_heads * head_dim) and out.is_contiguous() and out.dtype == torch.bfloat16,
          "attention_decode_prep: out must be contiguous bfloat16 [T, q_heads * head_dim]")
    _check_planes(k_cache, v_cache, kv_heads, head_dim)
    _need(k_cache.dtype == torch.bfloat16, "attention_decode_prep: the cache must be bfloat16")
    _need(positions.dtype == torch.int32 and positions.numel() == T, "attention_decode_prep: positions must be int32 [T]")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == head_dim),
              "attention_decode_prep: norm weights must be float32 [head_dim]")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and 2 * inv_freq.numel() == head_dim),
          "attention_decode_prep: the rotation must cover the whole head")
    _need(query_start.dtype == torch.int32 and context_lens.dtype == torch.int32 and block_tables.dtype == torch.int32
          and block_tables.dim() == 2 and block_tables.stride(1) == 1, "attention: index tensors must be int32")
    _need((seq_list is None and 0 <= first and first + n_list <= context_lens.numel()) or
          (seq_list is not None and seq_list.dtype == torch.int32 and seq_list.numel() >= n_list),
          "attention: seq_list must be int32 [n_list], or the first of n_list sequences in a row")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    _need(counters.dtype == torch.int32 and counters.numel() >= n_list * kv_heads, "attention: counters too small")
    if partial is not None:
        _need(partial.M == T and partial.N == width, "attention_decode_prep: partial sums do not match the rows")
    call("tie_attention_decode_prep", qkv.data_ptr(), qkv.stride(0), partial.partial.data_ptr() if partial else 0,
         partial.stride if partial else 0, partial.splits if partial else 0, partial.N if partial else 0,
         _ptr(q_weight), _ptr(k_weight), float(q_eps), float(k_eps), _ptr(inv_freq), positions.data_ptr(),
         1 if append else 0, k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), query_start.data_ptr(),
         context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], q_heads, kv_heads, head_dim,
         k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _ptr(seq_list), first, n_list, split_keys,
         max_splits, scratch.data_ptr(), counters.data_ptr(), 1 if cluster else 0, _stream())


def sample(logits: torch.Tensor, out: torch.Tensor, inv_temperature=None, seeds=None, counters=None, top_k=None,
           top_p=None, one_cta: bool = False) -> None:
    """out[r] = first maximum of row r (inv_temperature None or 0), or a draw from softmax(logits * inv_temperature)
    with the Philox uniform of (seeds[r], counters[r]). With top_k (int32) and top_p (float32) the rows whose
    top_k is in (0, vocab) or whose top_p is below 1 draw from the candidates those keep, most likely first
    (`one_cta`: with the kernel that serves the largest vocabularies, whatever the size; for tests)."""
    _dev(logits, out, inv_temperature, seeds, counters, top_k, top_p)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be float32 rows")
    _need(out.dtype == torch.int32 and out.numel() >= R, "sample: out must be int32 [R]")
    if inv_temperature is not None:
        _need(inv_temperature.dtype == torch.float32 and seeds.dtype == torch.int64 and counters.dtype == torch.int64,
              "sample: inv_temperature float32, seeds and counters int64")
    call("tie_sample", logits.data_ptr(), logits.stride(0), R, V, _ptr(inv_temperature), _ptr(seeds), _ptr(counters),
         out.data_ptr(), _stream())
    if top_k is not None or top_p is not None:
        _need(inv_temperature is not None and top_k is not None and top_p is not None,
              "sample: top_k and top_p come together, with temperatures")
        _need(top_k.dtype == torch.int32 and top_p.dtype == torch.float32 and top_k.numel() >= R and top_p.numel() >= R,
              "sample: top_k int32 [R], top_p float32 [R]")
        call("tie_sample_filtered", logits.data_ptr(), logits.stride(0), R, V, inv_temperature.data_ptr(), top_k.data_ptr(),
             top_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(), out.data_ptr(), 1 if one_cta else 0, _stream())


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, partial_scratch=None):
    """The engine's matrix product: picks the kernel for the dtype and the sizes. With
    `partial_scratch` (a callable numel -> float32 buffer) a product whose k range is split may
    come back as a SplitSum (then `out` is untouched); else returns `out`.

    `w` is taken for a weight: the tensor-core kernels start fetching it before the kernel ahead of them
    in the stream has finished, so it must not be something that kernel writes."""
    from . import gemm_select
    return gemm_select.gemm(a, w, out, partial_scratch)


def bound_gemm(w: torch.Tensor, silu: bool = False, split_many: bool = True, pack: bool = True):
    """A matrix product bound to one weight (gemm_select.BoundGemm): checked once, called every step.
    `split_many` False: above 128 tokens k is never split (the consumer wants the finished product). With `pack`
    a weight that the tensor-core kernels take is stored in k-blocks (pack_k_blocks) from here on: the product
    keeps that copy (`.w`) and the caller lets go of its own. `.rows(a, b)` is the product with rows a..b-1 of
    the same weight, without a copy."""
    from . import gemm_select
    return gemm_select.BoundGemm(w, silu, split_many, pack)


def partial_capacity(max_rows: int, N: int, K: int, split_many: bool = True) -> int:
    """The largest scratch (floats) a split product of up to max_rows tokens with [N, K] weights asks for."""
    from . import gemm_select
    return gemm_select.partial_capacity(int(max_rows), int(N), int(K), bool(split_many))


def gemm_silu(a: torch.Tensor, w_blocks: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a . gate^T) * (a . up^T) in one tensor-core product; w_blocks [2I, K] holds
    blocks of 16 gate rows followed by their 16 up rows (interleave_gate_up)."""
    from . import gemm_select
    gemm_select.gemm_silu(a, w_blocks, out)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K], [I, K] -> [2I, K]: 16 gate rows, their 16 up rows, the next 16 gate rows, ... (I % 16 == 0)."""
    I, K = gate.shape
    return torch.stack([gate.view(I // 16, 16, K), up.view(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()
