"""Token embedding and the output table (src/model/qwen3.cpp:75,92-100,213,255-259): x[t] = table[id],
logits = last . W^T in float32, W = the embedding table when the model ties them."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import Embedding, OutputHead, register_part, to_compute


class TokenEmbedding(Embedding):
    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = spec["name"]
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.dtype = dtype
        self.table = None

    def needs(self):
        return {self.name: TensorNeed((self.vocab, self.hidden))}

    def bind(self, get):
        # Kept the way a matrix product streams it best (in k-blocks, for the tensor-core kernels): an output head
        # that shares the table multiplies by this very tensor (`product`), and a row of it is as cheap to gather.
        self.product = ops.bound_gemm(to_compute(get(self.name), self.dtype).contiguous())
        self.table = self.product.w

    def forward(self, tokens, x):
        ops.embed(self.table, tokens, x)


class LMHead(OutputHead):
    def __init__(self, spec, dtype, embedding: TokenEmbedding | None = None, prefix: str = ""):
        self.name = spec["name"]
        self.tied = bool(spec["tied"])
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.dtype = dtype
        self.embedding = embedding
        self.weight = None

    def needs(self):
        # A tied checkpoint may still carry a duplicate output table; it is accepted and ignored.
        return {self.name: TensorNeed((self.vocab, self.hidden), optional=self.tied)}

    def bind(self, get):
        if self.tied:
            if getattr(self.embedding, "product", None) is None:
                raise InvalidArgument("a tied output head needs an embedding part that offers the `product` with its table")
            self.product = self.embedding.product
        else:
            self.product = ops.bound_gemm(to_compute(get(self.name), self.dtype).contiguous())
        self.weight = self.product.w

    def forward(self, last, logits):
        self.product(last, logits)


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("head", "lm_head", LMHead, replace=True)
