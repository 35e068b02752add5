"""Grouped-query attention over the paged cache.

    q, k, v = h Wq^T, h Wk^T, h Wv^T          one product with the three weights stacked
    q, k    = norm over each head (optional), then the position encoding
    k, v    -> cache pages at this step's slots
    out     = softmax(scale q k^T, causal, optional window) v, then Wo

Formulas: src/model/qwen3.cpp:218-230 and src/backend/cpu/cpu_backend.cpp:261-319. Every
size and constant is a parameter: heads, kv heads, head size, scale, window, eps of the
head norms, which position encoding.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import CacheNeed, Mixer, build_part, register_part, to_compute

from ..ops.gemm_select import NUM_SMS      # the SM count the split and tiling heuristics were tuned for (one B200)

SPLIT_KEYS = 256       # keys per split for sequences that bring one token
MAX_SPLITS = 64        # at most tie_attention_decode_limit(1) = 256
TMA_DECODE_TABLE_ENTRIES = 512     # tie_attention_decode_limit(0) (csrc/attention_decode.cu: kMaxTablePages)


class GQAttention(Mixer):
    launches_only = True

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = int(p.get("window") or 0)
        # 1/sqrt(head_dim) in float32, as the reference computes it (src/model/qwen3.cpp:195)
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(
            np.float32(1.0) / np.sqrt(np.float32(self.head_dim)))
        if self.heads % self.kv_heads:
            raise InvalidArgument(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.dtype = dtype
        self.q_norm = build_part("norm", p["q_norm"], dtype, prefix=self.prefix) if p.get("q_norm") else None
        self.k_norm = build_part("norm", p["k_norm"], dtype, prefix=self.prefix) if p.get("k_norm") else None
        self.position = build_part("position", p["position"], dtype, prefix=self.prefix)
        self.scale *= float(self.position.score_scale())
        self.q_dim, self.kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.w_qkv = self.w_o = None

    # -- weights
    def needs(self):
        n = {self.prefix + "q_proj.weight": TensorNeed((self.q_dim, self.hidden)),
             self.prefix + "k_proj.weight": TensorNeed((self.kv_dim, self.hidden)),
             self.prefix + "v_proj.weight": TensorNeed((self.kv_dim, self.hidden)),
             self.prefix + "o_proj.weight": TensorNeed((self.hidden, self.q_dim))}
        for part in (self.q_norm, self.k_norm, self.position):
            if part is not None:
                n.update(part.needs())
        return n

    def bind(self, get):
        w = [to_compute(get(self.prefix + f"{n}_proj.weight"), self.dtype) for n in "qkv"]
        # One stacked weight, so that one product reads the activations once; the products bound to it keep it in the
        # layout they stream best, and q, k and v alone (layers that read another layer's cache, norms and position
        # encodings that the fused kernel does not know) are row slices of the same memory.
        self.gemm_qkv = ops.bound_gemm(torch.cat(w, dim=0).contiguous(), split_many=False)
        del w
        self.w_qkv = self.gemm_qkv.w
        self.gemm_q = self.gemm_qkv.rows(0, self.q_dim)
        self.gemm_k = self.gemm_qkv.rows(self.q_dim, self.q_dim + self.kv_dim)
        self.gemm_v = self.gemm_qkv.rows(self.q_dim + self.kv_dim, self.q_dim + 2 * self.kv_dim)
        self.w_q, self.w_k, self.w_v = self.gemm_q.w, self.gemm_k.w, self.gemm_v.w
        self.gemm_o = ops.bound_gemm(to_compute(get(self.prefix + "o_proj.weight"), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        self._capacity = None       # (q/k/v product, output product): the most partial sums a step can leave
        for part in (self.q_norm, self.k_norm, self.position):
            if part is not None:
                part.bind(get)

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.kv_heads, self.head_dim, self.window)

    # -- one step
    def forward(self, h, ctx, cache, state):
        T = h.shape[0]
        Hq, Hkv, Dh = self.heads, self.kv_heads, self.head_dim
        g = ctx.groups[cache.group]
        # One kernel does the head norms, the rotation and the cache append when the parts say it may: a norm
        # that is exactly an RMSNorm (`fusable_rms`), an encoding that is a rotation by a frequency table or
        # leaves q and k alone. Anything else is called through its own interface below.
        table = self.position.fused_table()
        fused = (table is not None or self.position.is_identity) and \
            all(n is None or n.fusable_rms for n in (self.q_norm, self.k_norm))
        if fused:
            qw = self.q_norm.weight if self.q_norm is not None else None
            kw = self.k_norm.weight if self.k_norm is not None else None
            q_eps = self.q_norm.eps if self.q_norm is not None else 0.0
            k_eps = self.k_norm.eps if self.k_norm is not None else 0.0
            width = self.q_dim + (2 * self.kv_dim if cache.writes else 0)
            qkv = ctx.ws.rows("attn.qkv", T, self.q_dim + 2 * self.kv_dim, self.dtype)[:, :width]
            if self._capacity is None:
                self._capacity = (ops.partial_capacity(ctx.ws.max_rows, self.gemm_qkv.N, self.gemm_qkv.K, split_many=False),
                                  ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K))
            got = (self.gemm_qkv if cache.writes else self.gemm_q)(
                h, qkv, lambda n: ctx.ws.flat("attn.qkv.partial", n, torch.float32, self._capacity[0]))
            partial = got if isinstance(got, ops.SplitSum) else None
            if ctx.multi_rows == 0 and ops.attention_decode_prep_takes(qkv, Hq, Hkv, Dh, cache.k.shape[2], table):
                # every sequence brings one token: the attention kernel prepares the heads itself
                attn = ctx.ws.rows("attn.out", T, self.q_dim, self.dtype)
                self.attend_single(None, attn, ctx, g, cache, prep=(qkv, qw, kw, q_eps, k_eps, table, partial))
                return self.output(attn, ctx)
            ops.qk_norm_rope_append(qkv, qw, kw, q_eps, k_eps, table, ctx.positions, g.slots, cache.k, cache.v, Hq, Hkv,
                                    Dh, write_kv=cache.writes, partial=partial)
            q = qkv[:, :self.q_dim]
        else:
            # Any other norm or position encoding: separate products and the parts' own kernels.
            q = ctx.ws.rows("attn.q", T, self.q_dim, self.dtype)
            self.gemm_q(h, q)
            if self.q_norm is not None:
                self.q_norm.rows(q.view(T * Hq, Dh), q.view(T * Hq, Dh))
            if not self.position.is_identity:
                self.position.apply(q, ctx.positions, Hq, Dh)
            if cache.writes:
                k = ctx.ws.rows("attn.k", T, self.kv_dim, self.dtype)
                v = ctx.ws.rows("attn.v", T, self.kv_dim, self.dtype)
                self.gemm_k(h, k)
                self.gemm_v(h, v)
                if self.k_norm is not None:
                    self.k_norm.rows(k.view(T * Hkv, Dh), k.view(T * Hkv, Dh))
                if not self.position.is_identity:
                    self.position.apply(k, ctx.positions, Hkv, Dh)
                ops.kv_append(k, v, g.slots, cache.k, cache.v)
        attn = ctx.ws.rows("attn.out", T, self.q_dim, self.dtype)
        self.attend(q, attn, ctx, g, cache)
        return self.output(attn, ctx)

    def output(self, attn, ctx):
        out = ctx.ws.rows("mixer.out", attn.shape[0], self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = (ops.partial_capacity(ctx.ws.max_rows, self.gemm_qkv.N, self.gemm_qkv.K, split_many=False),
                              ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K))
        return self.gemm_o(attn, out, lambda n: ctx.ws.flat("mixer.out.partial", n, torch.float32, self._capacity[1]))

    def attend(self, q, attn, ctx, g, cache):
        """Rows of sequences that bring several tokens come first in a step, then one row per
        sequence that brings one token (ctx.multi_rows, ctx.single_seqs). bfloat16 with a head
        size the tensor-core kernels take runs there, everything else on the CUDA cores."""
        Hq, Hkv, Dh = self.heads, self.kv_heads, self.head_dim
        tc = ops.attention_tc_takes(q, Hq, Hkv, Dh)
        if ctx.multi_rows > 0:
            n = ctx.multi_rows
            if tc:
                tma = ops.attention_decode_tma_takes(q, Hq, Hkv, Dh, cache.k.shape[2])
                fn = ops.attention_prompt_tma if tma else ops.attention_prompt_tc
                if tma and ops.attention_prompt_umma_takes(q, Hq, Hkv, Dh, cache.k.shape[2], ctx.multi_max_queries):
                    fn = ops.attention_prompt_umma
                fn(q, cache.k, cache.v, attn, ctx.query_start, ctx.context_lens, g.block_tables, ctx.multi_seqs,
                   ctx.multi_max_queries, Hq, Hkv, Dh, self.scale, self.window)
            else:
                ops.attention_rows(q[:n], cache.k, cache.v, attn[:n], ctx.seq_of_row[:n], ctx.query_start,
                                   ctx.context_lens, g.block_tables, Hq, Hkv, Dh, self.scale, self.window)
        if ctx.single_count > 0:
            self.attend_single(q, attn, ctx, g, cache, tc)

    def attend_single(self, q, attn, ctx, g, cache, tc=True, prep=None):
        """The sequences that bring one token. With `prep` (the q/k/v product's output, the head norms' weights and
        eps, the rotation's frequencies, the product's partial sums or None) the TMA-fed kernel norms and rotates the
        heads and appends the newest key and value itself; q is not used then."""
        Hq, Hkv, Dh = self.heads, self.kv_heads, self.head_dim
        longest = ctx.single_max_context if self.window <= 0 else min(ctx.single_max_context, self.window)
        page = cache.k.shape[2]
        if prep is not None or (tc and ops.attention_decode_tma_takes(q, Hq, Hkv, Dh, page)):
            lens = ctx.single_contexts if self.window <= 0 else None
            key = ("decode_splits", longest, ctx.single_count, Hkv, page, lens is None)
            memo = getattr(ctx, "memo", None)
            splits = memo.get(key) if memo is not None else None
            if splits is None:
                splits = decode_splits(longest, ctx.single_count, Hkv, page, lens)
                if memo is not None:
                    memo[key] = splits
            split_keys, max_splits = splits
            scratch = ctx.ws.flat("attn.split", ops.attention_split_scratch_floats(ctx.max_seqs, Hq, Dh, MAX_SPLITS),
                                  torch.float32)
            counters = ctx.ws.zeros("attn.counters", ctx.max_seqs * Hkv, torch.int32)
            # the splits of a sequence as one cluster, merged through shared memory: where every CTA of the launch is
            # resident at once (a split without keys keeps its place until its cluster is through)
            cluster = max_splits in ops.CLUSTER_SPLITS and ctx.single_count * Hkv * max_splits <= 2 * NUM_SMS
            if prep is not None:
                qkv, qw, kw, q_eps, k_eps, table, partial = prep
                ops.attention_decode_prep(qkv, qw, kw, q_eps, k_eps, table, ctx.positions, cache.k, cache.v, attn,
                                          ctx.query_start, ctx.context_lens, g.block_tables, Hq, Hkv, Dh, self.scale,
                                          ctx.multi_seqs, ctx.single_count, split_keys, max_splits, scratch, counters,
                                          self.window, append=cache.writes, partial=partial, cluster=cluster)
                return
            ops.attention_decode_tma(q, cache.k, cache.v, attn, ctx.query_start, ctx.context_lens, g.block_tables, Hq,
                                     Hkv, Dh, self.scale, ctx.multi_seqs, ctx.single_count, split_keys, max_splits,
                                     scratch, counters, self.window, cluster=cluster)
            return
        split_keys = SPLIT_KEYS
        while math.ceil(longest / split_keys) > MAX_SPLITS:
            split_keys *= 2
        max_splits = max(1, math.ceil(longest / split_keys))
        scratch = ctx.ws.flat("attn.split", ops.attention_split_scratch_floats(ctx.max_seqs, Hq, Dh, MAX_SPLITS),
                              torch.float32)
        fn = ops.attention_decode_tc if tc else ops.attention_split
        fn(q, cache.k, cache.v, attn, ctx.query_start, ctx.context_lens, g.block_tables, Hq, Hkv, Dh, self.scale,
           ctx.single_seqs, ctx.single_count, split_keys, max_splits, scratch, self.window)


def decode_splits(longest: int, sequences: int, kv_heads: int, page_size: int, contexts=None) -> tuple[int, int]:
    """(keys per split, most splits of a sequence) for the TMA decode kernel: about two CTAs per SM in all
    ((sequence, kv head) pairs times splits), splits of whole 64-key tiles and at least SPLIT_KEYS keys, no
    longer than the page ids the kernel keeps in shared memory allow (TMA_DECODE_TABLE_ENTRIES boxes, one per
    page or per 64 keys of a larger page) and no more than MAX_SPLITS of them. With the sequences' own context
    lengths (steps that are not captured graphs) the split is the shortest that keeps all CTAs resident at
    once, so that a few long sequences among short ones are cut up instead of setting the pace alone."""
    slots = 2 * NUM_SMS
    boxes_per_tile = 64 // min(page_size, 64)
    cap = (TMA_DECODE_TABLE_ENTRIES // boxes_per_tile - 1) * 64
    if contexts:
        split_keys = SPLIT_KEYS
        lens = np.asarray(contexts, dtype=np.int64)
        while split_keys < longest and int((-(-lens // split_keys)).sum()) * kv_heads > slots:
            split_keys += max(64, split_keys // 8 // 64 * 64)
        split_keys = min(split_keys, max(SPLIT_KEYS, -(-longest // 64) * 64))
    else:
        want = max(1, slots // max(1, sequences * kv_heads))
        split_keys = max(SPLIT_KEYS, -(-math.ceil(longest / want) // 64) * 64)
    split_keys = min(split_keys, cap)
    while math.ceil(longest / split_keys) > MAX_SPLITS:
        split_keys += 64
    return split_keys, max(1, math.ceil(longest / split_keys))


register_part("mixer", "gqa_attention", GQAttention, replace=True)
