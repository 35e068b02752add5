"""Typed configuration of Qwen3 (dense), read from config.json, and its model description.

Keys, defaults and rejections follow the reference's `config_from_hf_json` and
`ModelConfig::validate` (src/model/config.cpp:10-67). No size lives anywhere else.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass

from ..errors import LoadError, UnsupportedError
from .registry import Architecture, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    model_type: str = "qwen3"

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def validate(self) -> None:
        """src/model/config.cpp:10-29."""
        if self.model_type != "qwen3":
            raise UnsupportedError(f"architecture '{self.model_type}' is not supported (supported: qwen3)")
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "max_position_embeddings"):
            value = getattr(self, key)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise LoadError(f"config {key} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise LoadError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                            f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise LoadError(f"head_dim {self.head_dim} must be even for rotary embeddings")
        for key in ("rms_norm_eps", "rope_theta"):
            value = getattr(self, key)
            if not isinstance(value, (int, float)) or isinstance(value, bool) or not math.isfinite(value) or not value > 0:
                raise LoadError(f"config {key} must be a positive number, got {value!r}")

    def to_json(self) -> dict:
        d = asdict(self)
        d["architectures"] = ["Qwen3ForCausalLM"]
        return d


def parse_qwen3_config(j: dict) -> Qwen3Config:
    """src/model/config.cpp:31-67: required keys, defaults of the optional ones, what is rejected."""
    def required(key):
        if key not in j:
            raise LoadError(f"config.json has no '{key}'")
        return j[key]

    model_type = j.get("model_type", "qwen3")
    if model_type != "qwen3":
        raise UnsupportedError(f"architecture '{model_type}' is not supported (supported: qwen3)")
    if j.get("use_sliding_window", False):
        raise UnsupportedError("use_sliding_window=true is not supported; the engine computes full attention for qwen3")
    if j.get("rope_scaling") is not None:
        raise UnsupportedError(f"rope_scaling {j['rope_scaling']!r} is not supported")
    if j.get("attention_bias", False):
        raise UnsupportedError("attention_bias=true is not supported")
    heads = required("num_attention_heads")
    hidden = required("hidden_size")
    head_dim = j.get("head_dim")
    if head_dim is None:
        if not isinstance(heads, int) or not isinstance(hidden, int) or heads <= 0:
            raise LoadError(f"config num_attention_heads must be a positive integer, got {heads!r}")
        head_dim = hidden // heads
    cfg = Qwen3Config(
        vocab_size=required("vocab_size"), hidden_size=hidden, intermediate_size=required("intermediate_size"),
        num_hidden_layers=required("num_hidden_layers"), num_attention_heads=heads,
        num_key_value_heads=j.get("num_key_value_heads", heads), head_dim=head_dim,
        max_position_embeddings=required("max_position_embeddings"), rms_norm_eps=required("rms_norm_eps"),
        rope_theta=j.get("rope_theta", 10000.0), tie_word_embeddings=bool(j.get("tie_word_embeddings", False)),
        model_type=model_type)
    cfg.validate()
    return cfg


def qwen3_spec(c: Qwen3Config) -> ModelSpec:
    """Qwen3 as parts (src/model/qwen3.cpp:75-100 for the names, :214-262 for the order):
    every layer is pre-norm, grouped-query attention with per-head RMSNorm of q and k and
    rotate-half RoPE over the whole head, and a SwiGLU feed-forward; all norms share eps."""
    def norm(name: str, size: int) -> PartSpec:
        return PartSpec("rmsnorm", {"name": name, "size": size, "eps": c.rms_norm_eps})

    layers = []
    for l in range(c.num_hidden_layers):
        p = f"model.layers.{l}."
        mixer = PartSpec("gqa_attention", {
            "prefix": p + "self_attn.", "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
            "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim, "window": 0,
            "scale": None,  # 1/sqrt(head_dim)
            "q_norm": norm("q_norm.weight", c.head_dim), "k_norm": norm("k_norm.weight", c.head_dim),
            "position": PartSpec("rope", {"theta": c.rope_theta, "head_dim": c.head_dim, "rotary_dim": c.head_dim}),
        })
        ffn = PartSpec("swiglu", {"prefix": p + "mlp.", "hidden_size": c.hidden_size,
                                  "intermediate_size": c.intermediate_size})
        layers.append(LayerSpec(prefix=p, block=PartSpec("prenorm"), mixer=mixer,
                                mixer_norm=norm(p + "input_layernorm.weight", c.hidden_size), ffn=ffn,
                                ffn_norm=norm(p + "post_attention_layernorm.weight", c.hidden_size)))
    return ModelSpec(
        architecture="Qwen3ForCausalLM", hidden_size=c.hidden_size, vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"name": "model.embed_tokens.weight", "vocab_size": c.vocab_size,
                                               "hidden_size": c.hidden_size}),
        layers=tuple(layers), run_order=tuple(RunEntry(l) for l in range(c.num_hidden_layers)),
        final_norm=norm("model.norm.weight", c.hidden_size),
        head=PartSpec("lm_head", {"name": "lm_head.weight", "tied": c.tie_word_embeddings,
                                  "tied_to": "model.embed_tokens.weight", "vocab_size": c.vocab_size,
                                  "hidden_size": c.hidden_size}))


register_architecture(Architecture(name="Qwen3ForCausalLM", parse_config=parse_qwen3_config, build_spec=qwen3_spec,
                                   model_types=("qwen3",)), replace=True)
