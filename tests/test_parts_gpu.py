"""Each part of a layer alone against the plain implementation, and parts put together in other
ways than Qwen3 does: a layer named twice, a layer that reads another layer's cache, a window,
a toy mixer with state of its own that the framework has never seen."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import TOL, assert_logits_close, rel_err, sharp_weights

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dtype)


def to_host(result, dtype):
    """What a part returned (a tensor, or the partial sums of a split product) as a float numpy array."""
    from tiny_inference_engine_b200 import ops
    if isinstance(result, ops.SplitSum):
        result = result.materialize(torch.empty(result.M, result.N, device="cuda", dtype=DT[dtype]))
    return result.float().cpu().numpy()


class DictSource:
    """A TensorSource over numpy arrays."""

    def __init__(self, tensors):
        self.t = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in tensors.items()}

    def shapes(self):
        return {k: (tuple(v.shape), v.dtype) for k, v in self.t.items()}

    def get(self, name):
        return self.t[name]


def build(spec, weights, dtype, page=8, pages=64, max_tokens=256, max_seqs=8):
    from tiny_inference_engine_b200 import StepRunner, make_cache
    from tiny_inference_engine_b200.parts import Model
    model = Model(spec, DT[dtype]).load(DictSource(weights))
    cache, states = make_cache(model, page_size=page, num_pages=pages, max_requests=max_seqs)
    return model, cache, StepRunner(model, cache, max_tokens, max_seqs, max_tokens, states=states)


def run_whole(runner, cache, tokens, cuts=None):
    from tiny_inference_engine_b200 import StepEntry
    req = cache.new_request()
    out, pos = [], 0
    for n in (cuts or [len(tokens)]):
        assert cache.reserve(req, pos + n)
        out.append(runner.run([StepEntry(req, tokens[pos:pos + n], pos, list(range(n)))]).float().cpu().numpy())
        pos += n
        cache.advance_window(req, pos)
    cache.release(req)
    return np.concatenate(out)


def qwen_spec(cfg):
    from tiny_inference_engine_b200.config import parse_qwen3_config, qwen3_spec
    return qwen3_spec(parse_qwen3_config(cfg))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_alone(dtype):
    """The mixer of layer 1 of tiny-B on random rows, whole and cut, against the plain attention block."""
    from tiny_inference_engine_b200 import StepEntry
    from tiny_inference_engine_b200.parts import build_part
    cfg = plain.normalise_config(plain.TINY_B)
    w = sharp_weights(cfg, 4)
    if dtype == "bfloat16":
        w = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()}
    spec = qwen_spec(cfg)
    model, cache, runner = build(spec, w, dtype)
    mixer = model.layers[1].mixer
    rng = np.random.default_rng(0)
    T = 50
    h = rng.standard_normal((T, cfg["hidden_size"])).astype(np.float32)
    if dtype == "bfloat16":
        h = plain.round_bf16(h)
    want = plain.attention_block(h, w, "model.layers.1.", cfg, np.arange(T))
    for cuts in ([T], [9, 2, 25, 1, 1, 12]):
        req = cache.new_request()
        got, pos = [], 0
        for n in cuts:
            assert cache.reserve(req, pos + n)
            ctx = runner.prepare([StepEntry(req, [0] * n, pos, [])])
            out = mixer.forward(dev(h[pos:pos + n], DT[dtype]), ctx, cache.layer_cache(1, writes=True), None)
            got.append(to_host(out, dtype))
            pos += n
        cache.release(req)
        assert rel_err(np.concatenate(got), want) < TOL[dtype] * (1 if dtype == "float32" else 0.6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_norm_and_block_alone(dtype):
    from tiny_inference_engine_b200 import StepEntry
    cfg = plain.normalise_config(plain.TINY_C)
    w = plain.random_weights(cfg, 2, std=0.2)
    if dtype == "bfloat16":
        w = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()}
    model, cache, runner = build(qwen_spec(cfg), w, dtype)
    rng = np.random.default_rng(1)
    T, D = 23, cfg["hidden_size"]
    h = rng.standard_normal((T, D)).astype(np.float32)
    h = plain.round_bf16(h) if dtype == "bfloat16" else h
    req = cache.new_request()
    cache.reserve(req, T)
    ctx = runner.prepare([StepEntry(req, [0] * T, 0, [])])
    block = model.layers[0]
    got = to_host(block.ffn.forward(dev(h, DT[dtype]), ctx), dtype)
    assert rel_err(got, plain.mlp_block(h, w, "model.layers.0.")) < TOL[dtype]
    # the norm part: x += delta, h = norm(x)
    x = rng.standard_normal((T, D)).astype(np.float32)
    xd, out = dev(x), torch.empty(T, D, device="cuda", dtype=DT[dtype])
    block.mixer_norm.add_norm(xd, dev(h, DT[dtype]), out)
    want = plain.rms_norm(x.astype(np.float64) + h, w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    assert rel_err(out.float().cpu().numpy(), want) < TOL[dtype]
    # the whole block: the residual stream after it is x + attn + mlp
    xd = dev(x)
    pending = block.forward(xd, None, ctx, cache.layer_cache(0, writes=True), None)
    torch.cuda.synchronize()
    got_x = xd.cpu().numpy().astype(np.float64) + to_host(pending, dtype)
    want_x = plain.decoder_layer(x.astype(np.float64), w, 0, cfg, np.arange(T))
    assert rel_err(got_x, want_x) < TOL[dtype]
    cache.release(req)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_encoding_part_and_the_unfused_path(dtype):
    """A position encoding the fused kernel does not know (no table) takes the separate kernels; same numbers."""
    from tiny_inference_engine_b200.config import LayerSpec, ModelSpec, PartSpec
    from tiny_inference_engine_b200.parts import RotaryEncoding, register_part

    class OpaqueRope(RotaryEncoding):
        def fused_table(self):
            return None

        def apply(self, x, positions, heads, head_dim):
            from tiny_inference_engine_b200 import ops
            ops.rope(x, positions, RotaryEncoding.fused_table(self), heads, head_dim)

    register_part("position", "opaque_rope", OpaqueRope, replace=True)
    cfg = plain.normalise_config(plain.TINY_A)
    w = sharp_weights(cfg, 3)
    base = qwen_spec(cfg)
    layers = []
    for l in base.layers:
        params = dict(l.mixer.params)
        params["position"] = PartSpec("opaque_rope", dict(params["position"].params))
        layers.append(LayerSpec(l.prefix, l.block, PartSpec("gqa_attention", params), l.mixer_norm, l.ffn, l.ffn_norm))
    spec = ModelSpec(**{**base.__dict__, "layers": tuple(layers)})
    toks = np.random.default_rng(2).integers(0, cfg["vocab_size"], 70).tolist()
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    want = plain.forward(wq, cfg, toks)
    model, cache, runner = build(spec, w, dtype, page=16)
    assert_logits_close(run_whole(runner, cache, toks, [33, 2, 35]), want, dtype, "unfused position encoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_names_a_layer_twice_and_shares_a_cache(dtype):
    """Run order [0, 1, 0, 1*] where 1* reads the cache that the first run of layer 1 wrote. The
    plain side recomputes it with whole sequences."""
    from tiny_inference_engine_b200.config import ModelSpec, RunEntry
    cfg = plain.normalise_config(plain.TINY_A)
    w = sharp_weights(cfg, 5)
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    base = qwen_spec(cfg)
    spec = ModelSpec(**{**base.__dict__, "run_order": (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1))})
    toks = np.random.default_rng(3).integers(0, cfg["vocab_size"], 60).tolist()

    # plain: layers 0, 1, 0 as usual; the fourth entry attends with its own q over layer 1's first-run k, v
    T = len(toks)
    pos = np.arange(T)
    x = plain.embed(wq["model.embed_tokens.weight"], toks)
    x = plain.decoder_layer(x, wq, 0, cfg, pos)
    p = "model.layers.1."
    h1 = plain.rms_norm(x, wq[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    Hq, Hkv, Dh, eps, th = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"], cfg["rope_theta"]
    k1 = plain.rope_neox(plain.rms_norm(plain.linear(h1, wq[p + "self_attn.k_proj.weight"]).reshape(T * Hkv, Dh),
                                        wq[p + "self_attn.k_norm.weight"], eps).reshape(T, -1), pos, Hkv, Dh, th)
    v1 = plain.linear(h1, wq[p + "self_attn.v_proj.weight"])
    x = plain.decoder_layer(x, wq, 1, cfg, pos)
    x = plain.decoder_layer(x, wq, 0, cfg, pos)
    h = plain.rms_norm(x, wq[p + "input_layernorm.weight"], eps)
    q = plain.rope_neox(plain.rms_norm(plain.linear(h, wq[p + "self_attn.q_proj.weight"]).reshape(T * Hq, Dh),
                                       wq[p + "self_attn.q_norm.weight"], eps).reshape(T, -1), pos, Hq, Dh, th)
    x = x + plain.linear(plain.causal_attention(q, k1, v1, Hq, Hkv, Dh), wq[p + "self_attn.o_proj.weight"])
    x = x + plain.mlp_block(plain.rms_norm(x, wq[p + "post_attention_layernorm.weight"], eps), wq, p)
    want = plain.linear(plain.rms_norm(x, wq["model.norm.weight"], eps), wq["model.embed_tokens.weight"])

    model, cache, runner = build(spec, w, dtype, page=16)
    assert len(cache.groups) == 1 and cache.groups[0].entries == (0, 1, 2)      # three planes, the fourth entry has none
    assert_logits_close(run_whole(runner, cache, toks, [31, 1, 1, 27]), want, dtype, "run order with a shared cache")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_different_mixers_one_windowed(dtype):
    """Layer 0 keeps all keys, layer 1 a window of 24: two cache groups, pages of the window group
    come back while the request is still running, and the logits match the plain windowed attention."""
    from tiny_inference_engine_b200.config import LayerSpec, ModelSpec, PartSpec
    cfg = plain.normalise_config(plain.TINY_A)
    w = sharp_weights(cfg, 6)
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    base = qwen_spec(cfg)
    l1 = base.layers[1]
    windowed = LayerSpec(l1.prefix, l1.block, PartSpec("gqa_attention", {**l1.mixer.params, "window": 24}), l1.mixer_norm,
                         l1.ffn, l1.ffn_norm)
    spec = ModelSpec(**{**base.__dict__, "layers": (base.layers[0], windowed)})
    toks = np.random.default_rng(4).integers(0, cfg["vocab_size"], 120).tolist()
    T, pos = len(toks), np.arange(len(toks))
    x = plain.embed(wq["model.embed_tokens.weight"], toks)
    x = plain.decoder_layer(x, wq, 0, cfg, pos)
    p = "model.layers.1."
    x = x + plain.attention_block(plain.rms_norm(x, wq[p + "input_layernorm.weight"], cfg["rms_norm_eps"]), wq, p, cfg, pos,
                                  window=24)
    x = x + plain.mlp_block(plain.rms_norm(x, wq[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), wq, p)
    want = plain.linear(plain.rms_norm(x, wq["model.norm.weight"], cfg["rms_norm_eps"]), wq["model.embed_tokens.weight"])

    model, cache, runner = build(spec, w, dtype, page=8, pages=16)
    assert [g.kind for g in cache.groups] == ["full", "window"]
    from tiny_inference_engine_b200 import StepEntry
    req = cache.new_request()
    got, at = [], 0
    for n in [40, 3, 1, 1, 30, 2, 43]:
        assert cache.reserve(req, at + n)
        got.append(runner.run([StepEntry(req, toks[at:at + n], at, list(range(n)))]).float().cpu().numpy())
        at += n
        cache.advance_window(req, at)
    assert cache.num_free(0) == 16 - 15 and cache.num_free(1) >= 16 - 4          # the window group holds at most 4 pages
    cache.release(req)
    assert_logits_close(np.concatenate(got), want, dtype, "windowed layer")


def test_a_toy_mixer_with_state_of_its_own_is_registered_built_and_stepped():
    """A mixer the framework has never seen: a running mean of the rows of a request,
    s_t = s_{t-1} + h_t, out_t = (s_t / (t+1)) W. Its state lives in the engine's state slots; it is
    registered from here, built by the same Model and stepped by the same step function, cut
    anywhere and beside other requests."""
    from tiny_inference_engine_b200 import StepEntry
    from toy_parts import running_mean_model
    spec, w, cfg, plain_forward = running_mean_model()
    D = cfg["hidden_size"]

    model, cache, runner = build(spec, w, "float32", page=8, pages=32)
    assert model.cache_needs()[1] is None and model.state_needs()[1].shape == (D,)
    assert len(cache.groups) == 1 and cache.groups[0].entries == (0,)
    rng = np.random.default_rng(8)
    a, b = rng.integers(0, 256, 40).tolist(), rng.integers(0, 256, 25).tolist()
    ra, rb = cache.new_request(), cache.new_request()
    assert ra.state_slot == rb.state_slot == -1          # a slot is taken by the first reserve, not before
    with pytest.raises(Exception, match="without a state slot"):
        runner.run([StepEntry(ra, a[:1], 0, [0])])
    got_a, got_b, pa, pb = [], [], 0, 0
    for na, nb in [(7, 0), (2, 11), (1, 1), (20, 13), (10, 0)]:
        entries = []
        if na:
            cache.reserve(ra, pa + na)
            entries.append(StepEntry(ra, a[pa:pa + na], pa, list(range(na))))
        if nb:
            cache.reserve(rb, pb + nb)
            entries.append(StepEntry(rb, b[pb:pb + nb], pb, list(range(nb))))
        out = runner.run(entries).float().cpu().numpy()
        got_a.append(out[:na]), got_b.append(out[na:])
        pa, pb = pa + na, pb + nb
    assert ra.state_slot >= 0 and rb.state_slot >= 0 and ra.state_slot != rb.state_slot
    assert_logits_close(np.concatenate(got_a), plain_forward(a), "float32", "toy mixer, request a")
    assert_logits_close(np.concatenate(got_b), plain_forward(b), "float32", "toy mixer, request b")
    # a slot handed out again starts from zero
    cache.release(ra)
    rc = cache.new_request()
    cache.reserve(rc, 40)
    out = runner.run([StepEntry(rc, a, 0, list(range(40)))]).float().cpu().numpy()
    assert_logits_close(out, plain_forward(a), "float32", "toy mixer, slot used again")


def test_a_toy_feed_forward_with_routing_and_another_position_encoding():
    """Two more parts the framework has never seen, registered from here and chosen for one layer only:
    a feed-forward that routes every token to one of three experts (router logits and softmax in
    float32), and a position encoding that is no rotation (it adds a sinusoid of the position to q and
    k), so the attention part takes its unfused path. The other layer stays Qwen3's. Stepped whole, in
    portions and beside another request."""
    import dataclasses

    from tiny_inference_engine_b200 import StepEntry
    from tiny_inference_engine_b200.config import LayerSpec, ModelSpec, PartSpec
    from tiny_inference_engine_b200.parts import FeedForward, PositionEncoding, register_part
    from tiny_inference_engine_b200.weights import TensorNeed

    class TopOneExperts(FeedForward):
        def __init__(self, spec, dtype, prefix=""):
            p = spec.params if hasattr(spec, "params") else spec
            self.prefix, self.d, self.e, self.dtype = p["prefix"], p["hidden_size"], p["experts"], dtype

        def needs(self):
            return {self.prefix + "router.weight": TensorNeed((self.e, self.d)),
                    self.prefix + "experts.weight": TensorNeed((self.e, self.d, self.d))}

        def bind(self, get):
            self.router, self.experts = get(self.prefix + "router.weight").float(), get(self.prefix + "experts.weight").float()

        def forward(self, h, ctx):
            x = h.float()
            probs = torch.softmax(x @ self.router.T, dim=-1)            # a toy: plain torch
            top = probs.argmax(dim=-1)
            out = torch.einsum("td,tod->to", x, self.experts[top]) * probs.gather(1, top[:, None])
            return out.to(h.dtype)

    class AddedSinusoid(PositionEncoding):
        def __init__(self, spec, dtype, prefix=""):
            p = spec.params if hasattr(spec, "params") else spec
            self.amp, self.base = p["amplitude"], p["base"]

        def apply(self, x, positions, heads, head_dim):
            freq = self.base ** (-torch.arange(head_dim, device=x.device, dtype=torch.float32) / head_dim)
            wave = self.amp * torch.sin(positions.float()[:, None] * freq[None, :])
            view = x.unflatten(1, (heads, head_dim))
            view.add_(wave[:, None, :].to(x.dtype))

    register_part("feed_forward", "top_one_experts", TopOneExperts, replace=True)
    register_part("position", "added_sinusoid", AddedSinusoid, replace=True)

    cfg = plain.normalise_config(plain.TINY_B)
    w = plain.random_weights(cfg, 21, std=0.1)
    D, E = cfg["hidden_size"], 3
    Hq, Hkv, Dh, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    rng = np.random.default_rng(5)
    w["model.layers.1.moe.router.weight"] = rng.standard_normal((E, D)).astype(np.float32)
    w["model.layers.1.moe.experts.weight"] = (rng.standard_normal((E, D, D)) * 0.1).astype(np.float32)
    for k in [k for k in w if k.startswith("model.layers.1.mlp.")]:
        del w[k]
    base = qwen_spec(cfg)
    l1 = base.layers[1]
    mixer_params = dict(l1.mixer.params)
    mixer_params["position"] = PartSpec("added_sinusoid", {"amplitude": 0.5, "base": 50.0})
    toy = dataclasses.replace(l1, mixer=PartSpec(l1.mixer.kind, mixer_params),
                              ffn=PartSpec("top_one_experts", {"prefix": "model.layers.1.moe.", "hidden_size": D, "experts": E}))
    spec = ModelSpec(**{**base.__dict__, "layers": (base.layers[0], toy, base.layers[2])})
    margins = []

    def plain_forward(toks):
        T, pos = len(toks), np.arange(len(toks))
        x = plain.embed(w["model.embed_tokens.weight"], toks)
        x = plain.decoder_layer(x, w, 0, cfg, pos)
        p = "model.layers.1."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q, k, v = (plain.linear(h, w[p + f"self_attn.{n}_proj.weight"]) for n in "qkv")
        q = plain.rms_norm(q.reshape(T * Hq, Dh), w[p + "self_attn.q_norm.weight"], eps).reshape(T, Hq, Dh)
        k = plain.rms_norm(k.reshape(T * Hkv, Dh), w[p + "self_attn.k_norm.weight"], eps).reshape(T, Hkv, Dh)
        wave = 0.5 * np.sin(pos[:, None] * 50.0 ** (-np.arange(Dh) / Dh)[None, :])
        q, k = (q + wave[:, None, :]).reshape(T, -1), (k + wave[:, None, :]).reshape(T, -1)
        x = x + plain.linear(plain.causal_attention(q, k, v, Hq, Hkv, Dh), w[p + "self_attn.o_proj.weight"])
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        logits = h @ w[p + "moe.router.weight"].astype(np.float64).T
        probs = np.exp(logits - logits.max(-1, keepdims=True))
        probs /= probs.sum(-1, keepdims=True)
        top = probs.argmax(-1)
        srt = np.sort(logits, -1)
        margins.append((srt[:, -1] - srt[:, -2]).min())
        experts = w[p + "moe.experts.weight"].astype(np.float64)
        x = x + np.einsum("td,tod->to", h, experts[top]) * probs[np.arange(T), top][:, None]
        x = plain.decoder_layer(x, w, 2, cfg, pos)
        return plain.linear(plain.rms_norm(x, w["model.norm.weight"], eps), w["lm_head.weight"])

    model, cache, runner = build(spec, w, "float32", page=8, pages=48)
    toks_a, toks_b = rng.integers(0, cfg["vocab_size"], 45).tolist(), rng.integers(0, cfg["vocab_size"], 30).tolist()
    want_a, want_b = plain_forward(toks_a), plain_forward(toks_b)
    assert min(margins) > 1e-3, "choose other weights: a router decision is too close to call"
    assert_logits_close(run_whole(runner, cache, toks_a), want_a, "float32", "toy parts, whole")
    assert_logits_close(run_whole(runner, cache, toks_a, cuts=[7, 2, 1, 20, 15]), want_a, "float32", "toy parts, in portions")
    ra, rb = cache.new_request(), cache.new_request()
    got_a, got_b, pa, pb = [], [], 0, 0
    for na, nb in [(30, 0), (1, 12), (1, 1), (13, 17)]:
        entries = []
        if na:
            cache.reserve(ra, pa + na)
            entries.append(StepEntry(ra, toks_a[pa:pa + na], pa, list(range(na))))
        if nb:
            cache.reserve(rb, pb + nb)
            entries.append(StepEntry(rb, toks_b[pb:pb + nb], pb, list(range(nb))))
        out = runner.run(entries).float().cpu().numpy()
        # entries are given in this order; rows come back in the order of the entries
        got_a.append(out[:na]), got_b.append(out[na:])
        pa, pb = pa + na, pb + nb
    assert_logits_close(np.concatenate(got_a), want_a, "float32", "toy parts, request a beside b")
    assert_logits_close(np.concatenate(got_b), want_b, "float32", "toy parts, request b beside a")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_embedding_output_head_norm_and_a_rotation_with_a_score_scale(dtype):
    """Four more parts the framework has never seen, registered from here, each chosen by the model description
    alone: an embedding scaled by sqrt(hidden), an output head with a soft cap on the logits, a head norm with
    another formula (x^ * (1 + w), its weight under the usual name: the fused q/k kernel must not stand in for
    it), and a rotation with stretched frequencies that asks for a factor on the attention scores."""
    import dataclasses
    from tiny_inference_engine_b200.config import ModelSpec, PartSpec
    from tiny_inference_engine_b200.parts import (LMHead, Norm, RotaryEncoding, TokenEmbedding, register_part)
    from tiny_inference_engine_b200.weights import TensorNeed
    CAP, STRETCH, FACTOR = 0.5, 4.0, 1.21

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, tokens, x):
            super().forward(tokens, x)
            x.mul_(float(np.sqrt(np.float32(self.hidden))))

    class SoftCapHead(LMHead):
        def forward(self, last, logits):
            super().forward(last, logits)
            logits.copy_(CAP * torch.tanh(logits / CAP))

    class OnePlusNorm(Norm):
        def __init__(self, spec, dtype, prefix=""):
            self.name, self.size, self.eps = prefix + spec["name"], spec["size"], spec["eps"]

        def needs(self):
            return {self.name: TensorNeed((self.size,), "norm")}

        def bind(self, get):
            self.weight = get(self.name).float()

        def rows(self, x, out):
            v = x.float()
            out.copy_((v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps) * (1.0 + self.weight)).to(out.dtype))

    class StretchedRope(RotaryEncoding):
        def __init__(self, spec, dtype, prefix=""):
            super().__init__(spec, dtype, prefix)
            self.inv_freq_host = (self.inv_freq_host / np.float32(STRETCH)).astype(np.float32)

        def score_scale(self):
            return FACTOR

    register_part("embedding", "scaled_embedding", ScaledEmbedding, replace=True)
    register_part("head", "soft_cap_head", SoftCapHead, replace=True)
    register_part("norm", "one_plus_norm", OnePlusNorm, replace=True)
    register_part("position", "stretched_rope", StretchedRope, replace=True)

    cfg = plain.normalise_config(plain.TINY_D)
    w = sharp_weights(cfg, 31)
    base = qwen_spec(cfg)
    l0, l1 = base.layers
    p0 = dict(l0.mixer.params)
    p0["q_norm"] = PartSpec("one_plus_norm", dict(p0["q_norm"].params))
    p1 = dict(l1.mixer.params)
    p1["position"] = PartSpec("stretched_rope", dict(p1["position"].params))
    spec = ModelSpec(**{**base.__dict__, "embedding": PartSpec("scaled_embedding", dict(base.embedding.params)),
                        "head": PartSpec("soft_cap_head", dict(base.head.params)),
                        "layers": (dataclasses.replace(l0, mixer=PartSpec(l0.mixer.kind, p0)),
                                   dataclasses.replace(l1, mixer=PartSpec(l1.mixer.kind, p1)))})
    Hq, Hkv, Dh, eps, theta = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta"))
    ws = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    st = lambda a: plain.round_bf16(a) if dtype == "bfloat16" else a       # what the engine stores between kernels

    def rotate(x, pos, heads, stretch):
        T, half = x.shape[0], Dh // 2
        inv = (plain.rope_inv_freq(theta, Dh) / np.float32(stretch)).astype(np.float32)
        ang = (pos.astype(np.float32)[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)
        c, s_ = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        v = x.reshape(T, heads, Dh)
        return np.concatenate([v[..., :half] * c - v[..., half:] * s_, v[..., half:] * c + v[..., :half] * s_], -1).reshape(T, -1)

    def layer(x, i, pos, one_plus, stretch, factor):
        p, T = f"model.layers.{i}.", x.shape[0]
        h = st(plain.rms_norm(x, ws[p + "input_layernorm.weight"], eps))
        q, k, v = (st(plain.linear(h, ws[p + f"self_attn.{n}_proj.weight"])) for n in "qkv")
        qw = ws[p + "self_attn.q_norm.weight"]
        if one_plus:
            qr = q.reshape(T * Hq, Dh).astype(np.float64)
            q = st(qr / np.sqrt((qr ** 2).mean(-1, keepdims=True) + eps) * (1.0 + qw.astype(np.float64))).reshape(T, -1)
        else:
            q = plain.rms_norm(q.reshape(T * Hq, Dh), qw, eps).reshape(T, -1)
        k = plain.rms_norm(k.reshape(T * Hkv, Dh), ws[p + "self_attn.k_norm.weight"], eps).reshape(T, -1)
        q, k = st(rotate(q, pos, Hq, stretch)), st(rotate(k, pos, Hkv, stretch))
        a = st(plain.causal_attention(q * factor, k, v, Hq, Hkv, Dh))      # a factor on every score
        x = x + st(plain.linear(a, ws[p + "self_attn.o_proj.weight"]))
        h = st(plain.rms_norm(x, ws[p + "post_attention_layernorm.weight"], eps))
        return x + plain.mlp_block(h, ws, p, dtype)

    def plain_forward(toks):
        pos = np.arange(len(toks))
        x = plain.embed(ws["model.embed_tokens.weight"], toks) * np.float64(np.sqrt(np.float32(cfg["hidden_size"])))
        x = layer(x, 0, pos, True, 1.0, 1.0)
        x = layer(x, 1, pos, False, STRETCH, FACTOR)
        logits = plain.linear(st(plain.rms_norm(x, ws["model.norm.weight"], eps)), ws["lm_head.weight"])
        return CAP * np.tanh(logits / CAP)

    model, cache, runner = build(spec, w, dtype, page=16, pages=32)
    assert type(model.embedding).__name__ == "ScaledEmbedding" and type(model.head).__name__ == "SoftCapHead"
    assert not model.layers[0].mixer.q_norm.fusable_rms and model.layers[0].mixer.k_norm.fusable_rms
    toks = np.random.default_rng(4).integers(0, cfg["vocab_size"], 90).tolist()
    want = plain_forward(toks)
    assert np.abs(want).max() > 0.5 * CAP                       # the cap bites
    assert_logits_close(run_whole(runner, cache, toks), want, dtype, "toy embedding, head, norm, rotation: whole")
    assert_logits_close(run_whole(runner, cache, toks, cuts=[50, 2, 1, 1, 36]), want, dtype, "the same in portions")


@pytest.mark.timeout(600)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_as_wide_as_the_large_model_against_the_plain_implementation(dtype):
    """One layer with Qwen3-8B's widths (hidden 4096, 32/8 heads of 128, intermediate 12288; a small vocabulary),
    in 32-bit (CUDA-core kernels) and in bfloat16: a 512-token portion (matrix products on pairs of SMs, prompt attention on tcgen05), then portions of
    two requests together, a portion beside a decoded token, and decoded tokens of both (split products whose
    partial sums feed the norm kernels, TMA decode attention). Every logit row against the plain implementation
    with the same storage."""
    from tiny_inference_engine_b200 import StepEntry
    cfg = plain.normalise_config({"vocab_size": 1000, "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 1,
                                  "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                                  "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
                                  "tie_word_embeddings": False})
    w = plain.random_weights(cfg, 3)
    w["model.layers.0.self_attn.q_norm.weight"] *= 3.0            # scores a few units apart: attention is not flat
    model, cache, runner = build(qwen_spec(cfg), w, dtype, page=16, pages=96, max_tokens=512, max_seqs=4)
    rng = np.random.default_rng(9)
    a, b = rng.integers(0, 1000, 640).tolist(), rng.integers(0, 1000, 420).tolist()
    want_a, want_b = plain.forward(w, cfg, a, storage=dtype), plain.forward(w, cfg, b, storage=dtype)
    ra, rb = cache.new_request(), cache.new_request()
    got = {"a": [], "b": []}

    def step(parts):
        entries = []
        for name, req, toks, start, n, want in parts:
            assert cache.reserve(req, start + n)
            entries.append(StepEntry(req, toks[start:start + n], start, want))
        out = runner.run(entries).float().cpu().numpy()
        row = 0
        for name, req, toks, start, n, want in parts:
            for k in want:
                got[name].append((start + k, out[row]))
                row += 1
        assert row == out.shape[0]

    step([("a", ra, a, 0, 512, [0, 1, 255, 300, 510, 511])])
    step([("a", ra, a, 512, 100, [0, 50, 99]), ("b", rb, b, 0, 180, [0, 100, 179])])          # 280 tokens
    step([("a", ra, a, 612, 1, [0]), ("b", rb, b, 180, 220, [0, 219])])                        # a decodes beside a portion
    pa, pb = 613, 400
    for _ in range(12):                                                                          # both decode
        step([("a", ra, a, pa, 1, [0]), ("b", rb, b, pb, 1, [0])])
        pa, pb = pa + 1, pb + 1
    from tiny_inference_engine_b200.ops import gemm_select
    torch.cuda.synchronize()
    gemm_select.check_status()
    for name, want in (("a", want_a), ("b", want_b)):
        pos = [p for p, _ in got[name]]
        assert_logits_close(np.stack([g for _, g in got[name]]), want[pos], dtype, f"wide layer, request {name}")


@pytest.mark.parametrize("graphs", [False, True])
def test_tokens_taken_from_the_step_before_on_the_device(tiny_models, graphs):
    """A step whose entries name a `device_row` takes their first token from the ids that the step before it
    sampled, wherever the entry stands in the step and whatever else the step holds: its logits are those of the
    same step fed the same ids from the host."""
    from tiny_inference_engine_b200 import SamplingParams, StepEntry, StepRunner, load_model, make_cache
    cfg, page, w, d = tiny_models["tiny_d"]
    model = load_model(d, "bfloat16")
    rng = np.random.default_rng(9)
    V = cfg["vocab_size"]
    prompts = [rng.integers(0, V, n).tolist() for n in (40, 23, 31)]
    portion = rng.integers(0, V, 17).tolist()
    out = {}
    for on_device in (False, True):
        cache, states = make_cache(model, page_size=page, num_pages=40, max_requests=8)
        runner = StepRunner(model, cache, 128, 8, 64, states=states, use_graphs=graphs)
        reqs = [cache.new_request() for _ in range(4)]
        for r in reqs:
            assert cache.reserve(r, 64)
        greedy = [(SamplingParams(), 0)] * 3
        _, ids = runner.run([StepEntry(r, p, 0, [len(p) - 1]) for r, p in zip(reqs, prompts)], greedy)
        first = ids.tolist()
        # the three requests decode in another order, beside a prompt portion of a fourth (no graph), or alone (a graph)
        order = [2, 0, 1]
        entries = [StepEntry(reqs[i], [0 if on_device else first[i]], len(prompts[i]), [0], i if on_device else None) for i in order]
        if not graphs:
            entries.insert(1, StepEntry(reqs[3], portion, 0, []))
        logits, ids = runner.run(entries, greedy)
        out[on_device] = (logits.float().cpu().numpy().copy(), ids.tolist())
        torch.cuda.synchronize()
        runner.check()
    assert np.array_equal(out[True][0], out[False][0]) and out[True][1] == out[False][1]
