"""A plain, slow Qwen3 (dense) in numpy: whole sequences, no cache, one function per part.

It is written from the formulas of AnishKamatam/tiny-inference-engine and rests on them;
`tests/golden/` holds outputs of that project's own CPU code for one tiny random model, and
`tests/test_plain.py` checks this file against them. Citations are `path:line` inside that
project. Nothing here imports the engine package: the tests compare the two.

Arithmetic is float64 on float32 inputs, except where the reference's result depends on
float32 rounding (the rotary angle). `storage` names the dtype the engine would store
activations in: with "bfloat16" every value that crosses a part's boundary is rounded to
bfloat16 the way the engine's bfloat16 path does, so that the natural size of bfloat16
noise can be measured on the CPU.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- rounding

def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 -> float32 (src/core/half.h:14-20)."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(a.shape)


def _store(x: np.ndarray, storage: str) -> np.ndarray:
    if storage == "bfloat16":
        return round_bf16(x.astype(np.float32)).astype(np.float64)
    return x


# --------------------------------------------------------------------------- parts

def embed(table: np.ndarray, ids) -> np.ndarray:
    """x[t] = table[ids[t]], no scaling (src/backend/cpu/cpu_backend.cpp:51-76)."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token id outside the vocabulary")
    return table[ids].astype(np.float64)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """(x * 1/sqrt(mean(x^2) + eps)) * w over the last axis (src/backend/cpu/cpu_backend.cpp:141-159)."""
    x = x.astype(np.float64)
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + np.float64(np.float32(eps)))
    return (x * inv) * weight.astype(np.float64)


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = x . W^T with W [out, in], no bias (src/backend/cpu/cpu_backend.cpp:93-139)."""
    return x.astype(np.float64) @ w.astype(np.float64).T


def rope_inv_freq(theta: float, head_dim: int) -> np.ndarray:
    """inv_freq[i] = 1 / theta^(2i / head_dim) in float32 (src/backend/rope.h:9-13)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    expo = (np.float32(2.0) * i) / np.float32(head_dim)
    return (np.float32(1.0) / np.power(np.float32(theta), expo, dtype=np.float32)).astype(np.float32)


def rope_neox(x: np.ndarray, positions, num_heads: int, head_dim: int, theta: float) -> np.ndarray:
    """Rotate-half RoPE over the whole head; angle = float32(pos) * inv_freq in float32
    (src/backend/cpu/cpu_backend.cpp:161-193)."""
    T = x.shape[0]
    half = head_dim // 2
    inv = rope_inv_freq(theta, head_dim)
    pos = np.asarray(positions, dtype=np.int64).astype(np.float32)
    angle = (pos[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)  # [T, half]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    v = x.astype(np.float64).reshape(T, num_heads, head_dim)
    x1, x2 = v[..., :half], v[..., half:]
    out = np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1)
    return out.reshape(T, num_heads * head_dim)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, num_heads: int, num_kv_heads: int,
                     head_dim: int, window: int = 0) -> np.ndarray:
    """Dense restatement of the paged attention: query t sees keys 0..t, q head h reads kv head
    h // (Hq/Hkv), scale 1/sqrt(Dh), softmax in full precision (src/backend/cpu/cpu_backend.cpp:261-319).
    `window` > 0 keeps only the last `window` keys (t-window+1..t); the reference has no window."""
    T = q.shape[0]
    group = num_heads // num_kv_heads
    scale = np.float64(np.float32(1.0) / np.sqrt(np.float32(head_dim)))
    qh = q.astype(np.float64).reshape(T, num_heads, head_dim)
    kh = k.astype(np.float64).reshape(T, num_kv_heads, head_dim)
    vh = v.astype(np.float64).reshape(T, num_kv_heads, head_dim)
    out = np.zeros((T, num_heads, head_dim))
    j = np.arange(T)
    mask = j[None, :] <= j[:, None]
    if window > 0:
        mask &= j[None, :] > (j[:, None] - window)
    for h in range(num_heads):
        kvh = h // group
        scores = scale * (qh[:, h, :] @ kh[:, kvh, :].T)
        scores = np.where(mask, scores, -np.inf)
        scores -= scores.max(axis=-1, keepdims=True)
        p = np.exp(scores)
        out[:, h, :] = (p @ vh[:, kvh, :]) / p.sum(axis=-1, keepdims=True)
    return out.reshape(T, num_heads * head_dim)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """g / (1 + exp(-g)) * u (src/backend/cpu/cpu_backend.cpp:195-207)."""
    g = gate.astype(np.float64)
    return g / (1.0 + np.exp(-g)) * up.astype(np.float64)


# --------------------------------------------------------------------------- blocks

def attention_block(h: np.ndarray, w: dict, p: str, cfg: dict, positions, storage: str = "float32",
                    window: int = 0) -> np.ndarray:
    """q/k/v projections, per-head RMSNorm of q and k before RoPE, RoPE, causal attention,
    output projection (src/model/qwen3.cpp:218-230)."""
    Hq, Hkv, Dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    T = h.shape[0]
    q = _store(linear(h, w[p + "self_attn.q_proj.weight"]), storage)
    k = _store(linear(h, w[p + "self_attn.k_proj.weight"]), storage)
    v = _store(linear(h, w[p + "self_attn.v_proj.weight"]), storage)
    q = rms_norm(q.reshape(T * Hq, Dh), w[p + "self_attn.q_norm.weight"], eps).reshape(T, Hq * Dh)
    k = rms_norm(k.reshape(T * Hkv, Dh), w[p + "self_attn.k_norm.weight"], eps).reshape(T, Hkv * Dh)
    q = _store(rope_neox(q, positions, Hq, Dh, theta), storage)
    k = _store(rope_neox(k, positions, Hkv, Dh, theta), storage)
    a = _store(causal_attention(q, k, v, Hq, Hkv, Dh, window), storage)
    return _store(linear(a, w[p + "self_attn.o_proj.weight"]), storage)


def mlp_block(h: np.ndarray, w: dict, p: str, storage: str = "float32") -> np.ndarray:
    """SwiGLU feed-forward (src/model/qwen3.cpp:235-238)."""
    g = _store(linear(h, w[p + "mlp.gate_proj.weight"]), storage)
    u = _store(linear(h, w[p + "mlp.up_proj.weight"]), storage)
    a = _store(swiglu(g, u), storage)
    return _store(linear(a, w[p + "mlp.down_proj.weight"]), storage)


def decoder_layer(x: np.ndarray, w: dict, layer: int, cfg: dict, positions, storage: str = "float32") -> np.ndarray:
    """Pre-norm: x += Attn(RMS(x)); x += MLP(RMS(x)) (src/model/qwen3.cpp:214-239).
    The residual stream x stays unrounded, as it does in the engine."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = _store(rms_norm(x, w[p + "input_layernorm.weight"], eps), storage)
    x = x + attention_block(h, w, p, cfg, positions, storage)
    h = _store(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), storage)
    return x + mlp_block(h, w, p, storage)


def forward(w: dict, cfg: dict, tokens, storage: str = "float32", hidden_out: list | None = None) -> np.ndarray:
    """Logits [T, V] (float64) of a whole sequence at every position (src/model/qwen3.cpp:212-262)."""
    cfg = normalise_config(cfg)
    if storage == "bfloat16":
        w = {n: (round_bf16(t) if t.ndim == 2 else t) for n, t in w.items()}
    T = len(tokens)
    positions = np.arange(T)
    x = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, positions, storage)
        if hidden_out is not None:
            hidden_out.append(x.copy())
    last = _store(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), storage)
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(last, head)


def normalise_config(cfg: dict) -> dict:
    """Defaults of absent keys as the reference reads config.json (src/model/config.cpp:31-67)."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("tie_word_embeddings", False)
    return c


# --------------------------------------------------------------------------- sampling

def philox4x32(counter, key, rounds: int = 10):
    """Philox4x32-10 (Salmon et al. 2011). The reference draws from std::mt19937_64
    (src/engine/sequence.h:22); the engine uses a counter-based generator instead so that a
    draw depends only on (seed, index of the generated token). This is the published
    algorithm restated for the tests."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k = [int(v) & 0xFFFFFFFF for v in key]
    for _ in range(rounds):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + W0) & 0xFFFFFFFF, (k[1] + W1) & 0xFFFFFFFF]
    return c


def uniform_for(seed: int, index: int) -> float:
    """The engine's uniform in [0, 1) for generated token `index` of a request seeded `seed`:
    the first Philox word, top 24 bits."""
    r = philox4x32([index & 0xFFFFFFFF, index >> 32, 0, 0], [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    return (r[0] >> 8) * (1.0 / (1 << 24))


def sample(logits: np.ndarray, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
           u: float = 0.0) -> int:
    """Greedy (first maximum) at temperature 0, else shift by the maximum, scale by 1/T, keep the
    top_k most likely, then the smallest prefix reaching top_p of the mass, and pick by inverse
    CDF with the uniform `u` (src/sampling/sampler.cpp:18-81). The reference draws
    uniform(0, total) from mt19937_64; here u*total with u given."""
    z = np.asarray(logits, dtype=np.float64)
    if z.size == 0 or np.isnan(z).any():
        raise ValueError("empty or NaN logits")
    best = int(np.argmax(z))
    if z[best] == -np.inf:
        raise ValueError("all logits are -inf")
    inv_t = np.inf if temperature == 0.0 else float(np.float32(1.0) / np.float32(temperature))
    if not np.isfinite(inv_t) or z[best] == np.inf:
        return best
    scaled = (z - z[best]) * inv_t
    order = np.arange(z.size)
    keep = z.size
    if (0 < top_k < z.size) or top_p < 1.0:
        order = np.lexsort((np.arange(z.size), -scaled))  # by value descending, ties by id
        if 0 < top_k < z.size:
            keep = top_k
    weights = np.exp(scaled[order[:keep]] - scaled[order[:keep]].max())
    total = weights.sum()
    if top_p < 1.0:
        cum = np.cumsum(weights)
        keep = int(np.searchsorted(cum, top_p * total, side="left")) + 1
        keep = min(keep, weights.size)
        weights, total = weights[:keep], cum[keep - 1]
    r = u * total
    cum = np.cumsum(weights)
    idx = int(np.searchsorted(cum, r, side="right"))
    return int(order[min(idx, keep - 1)])


def generate(w: dict, cfg: dict, prompt, max_tokens: int, temperature: float = 0.0, top_k: int = 0,
             top_p: float = 1.0, seed: int = 0, storage: str = "float32") -> list[int]:
    """Recompute the whole sequence for every new token (src/engine/engine.cpp:157-181 without a cache)."""
    tokens = list(prompt)
    out = []
    for i in range(max_tokens):
        logits = forward(w, cfg, tokens, storage)[-1]
        t = sample(logits, temperature, top_k, top_p, uniform_for(seed, i))
        tokens.append(t)
        out.append(t)
    return out


# --------------------------------------------------------------------------- random models and files

def tensor_shapes(cfg: dict) -> dict:
    """Names and shapes of a Qwen3 checkpoint (src/model/qwen3.cpp:75-100)."""
    c = normalise_config(cfg)
    D, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    Q, KV, Dh = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"], c["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, D)}
    for l in range(c["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes.update({
            p + "input_layernorm.weight": (D,), p + "self_attn.q_proj.weight": (Q, D),
            p + "self_attn.k_proj.weight": (KV, D), p + "self_attn.v_proj.weight": (KV, D),
            p + "self_attn.o_proj.weight": (D, Q), p + "self_attn.q_norm.weight": (Dh,),
            p + "self_attn.k_norm.weight": (Dh,), p + "post_attention_layernorm.weight": (D,),
            p + "mlp.gate_proj.weight": (I, D), p + "mlp.up_proj.weight": (I, D),
            p + "mlp.down_proj.weight": (D, I)})
    shapes["model.norm.weight"] = (D,)
    if not c["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (V, D)
    return shapes


def random_weights(cfg: dict, seed: int, std: float = 0.02, norm_std: float = 0.01) -> dict:
    """Matrices N(0, std), norm weights 1 + N(0, norm_std), float32."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            out[name] = (1.0 + norm_std * rng.standard_normal(shape)).astype(np.float32)
        else:
            out[name] = (std * rng.standard_normal(shape)).astype(np.float32)
    return out


def write_safetensors(path, tensors: dict) -> None:
    """8-byte little-endian header length, JSON header, raw bytes (src/model/safetensors.cpp:22-85)."""
    header, blobs, offset = {}, [], 0
    for name, t in tensors.items():
        a = np.ascontiguousarray(t)
        if a.dtype == np.float32:
            dt = "F32"
        elif a.dtype == np.uint16:
            dt = "BF16"
        elif a.dtype == np.int32:
            dt = "I32"
        else:
            raise ValueError(f"{name}: dtype {a.dtype}")
        b = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [offset, offset + len(b)]}
        blobs.append(b)
        offset += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return (round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def write_model_dir(path, cfg: dict, weights: dict, bf16: bool = False) -> None:
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    if bf16:
        weights = {n: (to_bf16_bits(t) if t.ndim == 2 else t) for n, t in weights.items()}
    write_safetensors(path / "model.safetensors", weights)


# The two tiny configurations of the tests. They differ in every size and option that the
# architecture has: layers, width, heads and groups, head size, feed-forward width,
# vocabulary, theta, eps, tied or separate output table.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "tie_word_embeddings": True,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 503, "hidden_size": 96, "intermediate_size": 200, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32,
    "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
}
# Tiny-B with four query heads (q width 128), as the benchmark description states it (same head count as tiny-A;
# TINY_B above has eight so that the two differ there as well). The reference's own CPU code ran this one:
# tests/golden/tiny_b4_*.
TINY_B4 = {**TINY_B, "num_attention_heads": 4, "max_position_embeddings": 256}
# A third one for the odd corners: as many KV heads as query heads (the num_key_value_heads key
# is absent), head size 48 (a multiple of 16 that is no power of two, from hidden/heads since
# the head_dim key is absent too), default theta and untied output. So the three cover
# grouped (A, 2 per group), multi-query (B, 8 per group) and plain multi-head attention (C).
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 311, "hidden_size": 144, "intermediate_size": 104, "num_hidden_layers": 1,
    "num_attention_heads": 3,
    "max_position_embeddings": 640, "rms_norm_eps": 3e-6,
}
# A fourth one whose head size (64) is one the tensor-core attention kernels take, so that the
# bfloat16 runs of the tests go through them; a group of 3 query heads per kv head.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 389, "hidden_size": 136, "intermediate_size": 264, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
    "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "tie_word_embeddings": False,
}
# A fifth one wide enough (hidden 1024, head size 128) that decode-sized matrix products are cut
# along k and hand their partial sums to the kernels behind them, as they do at real sizes.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 300, "hidden_size": 1024, "intermediate_size": 1536, "num_hidden_layers": 1,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True,
}
