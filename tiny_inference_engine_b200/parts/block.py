"""Pre-norm arrangement of a layer: x += mixer(norm(x)); x += ffn(norm(x))
(src/model/qwen3.cpp:214-239). Each residual add is fused with the norm that follows it, so
the feed-forward's output is handed on as a pending delta that the next layer's first norm
(or the final norm) adds."""
from __future__ import annotations

from .base import Block, build_part, register_part


class PreNormBlock(Block):
    def __init__(self, layer_spec, dtype, prefix: str = ""):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, dtype)
        self.mixer = build_part("mixer", layer_spec.mixer, dtype)
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm, dtype)
        self.ffn = build_part("feed_forward", layer_spec.ffn, dtype)
        self.dtype = dtype
        self.parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def needs(self):
        n = {}
        for p in self.parts:
            n.update(p.needs())
        return n

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def forward(self, x, pending, ctx, cache, state):
        h = ctx.ws.rows("block.normed", x.shape[0], x.shape[1], self.dtype)
        self.mixer_norm.add_norm(x, pending, h)
        mixed = self.mixer.forward(h, ctx, cache, state)
        self.ffn_norm.add_norm(x, mixed, h)
        return self.ffn.forward(h, ctx)


register_part("block", "prenorm", PreNormBlock, replace=True)
