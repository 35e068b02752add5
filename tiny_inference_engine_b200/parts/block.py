"""Pre-norm arrangement of a layer: x += mixer(norm(x)); x += ffn(norm(x))
(src/model/qwen3.cpp:214-239). Each residual add is fused with the norm that follows it, so
the feed-forward's output is handed on as a pending delta that the next layer's first norm
(or the final norm) adds."""
from __future__ import annotations

from .base import Block, build_part, register_part


class PreNormBlock(Block):
    launches_only = True

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
        """`pending` and what the parts return may be tensors [T, D] or ops.SplitSum (a split product
        whose partial sums the next add+norm adds up itself)."""
        h = ctx.ws.rows("block.normed", x.shape[0], x.shape[1], self.dtype)
        self.mixer_norm.add_norm(x, as_delta(pending, self.mixer_norm, ctx, "block.delta"), h)
        mixed = self.mixer.forward(h, ctx, cache, state)
        self.ffn_norm.add_norm(x, as_delta(mixed, self.ffn_norm, ctx, "block.delta"), h)
        return self.ffn.forward(h, ctx)


def as_delta(delta, norm, ctx, name):
    """A SplitSum stays one for norms that add the splits themselves (`takes_split_sum`), else it is added up first."""
    from .. import ops
    if isinstance(delta, ops.SplitSum) and not getattr(norm, "takes_split_sum", False):
        return delta.materialize(ctx.ws.rows(name, delta.M, delta.N, ctx.ws_dtype))
    return delta


register_part("block", "prenorm", PreNormBlock, replace=True)
