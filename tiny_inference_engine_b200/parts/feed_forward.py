"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)), silu(g) = g / (1 + exp(-g))
(src/model/qwen3.cpp:235-238, src/backend/cpu/cpu_backend.cpp:195-207). Gate and up are
stacked into one weight so that one product reads h once."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorNeed
from .base import FeedForward, register_part, to_compute


class SwiGLU(FeedForward):
    launches_only = True

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.dtype = dtype
        self.w_gate_up = self.w_down = None

    def needs(self):
        return {self.prefix + "gate_proj.weight": TensorNeed((self.inter, self.hidden)),
                self.prefix + "up_proj.weight": TensorNeed((self.inter, self.hidden)),
                self.prefix + "down_proj.weight": TensorNeed((self.hidden, self.inter))}

    def bind(self, get):
        gate = to_compute(get(self.prefix + "gate_proj.weight"), self.dtype)
        up = to_compute(get(self.prefix + "up_proj.weight"), self.dtype)
        # On the tensor-core path gate and up rows are interleaved in blocks of 16 and SiLU * up
        # happens in the product's epilogue; else they are stacked and a kernel of its own does it.
        self.fused = self.dtype == torch.bfloat16 and self.inter % 16 == 0 and self.hidden % 8 == 0
        self.gate_up = ops.bound_gemm(ops.interleave_gate_up(gate, up) if self.fused else torch.cat([gate, up], dim=0).contiguous(),
                                      silu=self.fused)
        del gate, up
        self.down = ops.bound_gemm(to_compute(get(self.prefix + "down_proj.weight"), self.dtype).contiguous())
        self.w_gate_up, self.w_down = self.gate_up.w, self.down.w      # as the products keep them (in k-blocks when they stream them)
        self._partial_capacity = None

    def forward(self, h, ctx):
        T = h.shape[0]
        act = ctx.ws.rows("ffn.act", T, self.inter, self.dtype)
        if self.fused:
            self.gate_up(h, act)
        else:
            gu = ctx.ws.rows("ffn.gate_up", T, 2 * self.inter, self.dtype)
            self.gate_up(h, gu)
            ops.silu_mul(gu, act)
        out = ctx.ws.rows("ffn.out", T, self.hidden, self.dtype)
        if self._partial_capacity is None:
            self._partial_capacity = ops.partial_capacity(ctx.ws.max_rows, self.down.N, self.down.K)
        return self.down(act, out, lambda n: ctx.ws.flat("ffn.out.partial", n, torch.float32, self._partial_capacity))


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
