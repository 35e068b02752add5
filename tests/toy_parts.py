"""Toy parts that the framework has never seen, shared by the tests that register them: they are defined here,
under tests/, and no file of the package knows them. Each comes with its plain restatement over whole sequences."""
import numpy as np
import torch

import plain_qwen3 as plain


def running_mean_mixer():
    """A mixer with state of its own: a running mean of the rows of a request,
    s_t = s_{t-1} + h_t, out_t = (s_t / (t+1)) W. Its state lives in the engine's state slots."""
    from tiny_inference_engine_b200.parts import Mixer, StateNeed
    from tiny_inference_engine_b200.weights import TensorNeed

    class RunningMean(Mixer):
        def __init__(self, spec, dtype, prefix=""):
            self.name, self.d, self.dtype = spec["name"], spec["hidden_size"], dtype

        def needs(self):
            return {self.name: TensorNeed((self.d, self.d))}

        def bind(self, get):
            self.w = get(self.name).float()

        def state_need(self):
            return StateNeed((self.d,), torch.float32)

        def forward(self, h, ctx, cache, state):
            out = torch.empty_like(h)
            qs = ctx.host.query_start
            for s in range(ctx.S):                 # a toy: plain torch, one request at a time
                slot = int(ctx.host.state_slots[s])
                rows = h[qs[s]:qs[s + 1]].float()
                sums = state[slot] + torch.cumsum(rows, 0)
                state[slot] = sums[-1]
                counts = torch.arange(ctx.host.starts[s] + 1, ctx.host.starts[s] + 1 + rows.shape[0], device=h.device)
                out[qs[s]:qs[s + 1]] = ((sums / counts[:, None]) @ self.w.T).to(h.dtype)
            return out

    return RunningMean


def running_mean_mixer_on_device():
    """The same mixer for steps in which every request brings one token, written with device tensors of the step
    only, so that it can say `graph_safe` and decode steps of its model are captured as CUDA graphs. Sequences that
    pad a captured batch have state slot -1: they add nothing to any slot."""
    base = running_mean_mixer()

    class RunningMeanOnDevice(base):
        graph_safe = True

        def forward(self, h, ctx, cache, state):
            if ctx.multi_rows > 0:
                return super().forward(h, ctx, cache, state)
            S = ctx.S
            slots = ctx.state_slots[:S]
            live = slots >= 0
            at = slots.clamp(min=0).long()
            state.index_add_(0, at, h.float() * live[:, None])
            counts = (ctx.positions[:S] + 1).float()
            return ((state[at] / counts[:, None]) @ self.w.T).to(h.dtype)

    return RunningMeanOnDevice


def running_mean_model(seed=7, on_device=False):
    """tiny-A with its second layer's attention replaced by the running mean: (spec, weights, config, plain forward)."""
    from tiny_inference_engine_b200.config import LayerSpec, ModelSpec, PartSpec, parse_qwen3_config, qwen3_spec
    from tiny_inference_engine_b200.parts import register_part
    register_part("mixer", "running_mean", running_mean_mixer_on_device() if on_device else running_mean_mixer(), replace=True)
    cfg = plain.normalise_config(plain.TINY_A)
    w = plain.random_weights(cfg, seed, std=0.1)
    D = cfg["hidden_size"]
    w["model.layers.1.toy.weight"] = (np.random.default_rng(0).standard_normal((D, D)) * 0.1).astype(np.float32)
    for k in [k for k in w if k.startswith("model.layers.1.self_attn")]:
        del w[k]
    base = qwen3_spec(parse_qwen3_config(cfg))
    l1 = base.layers[1]
    toy = LayerSpec(l1.prefix, l1.block, PartSpec("running_mean", {"name": "model.layers.1.toy.weight", "hidden_size": D}),
                    l1.mixer_norm, l1.ffn, l1.ffn_norm)
    spec = ModelSpec(**{**base.__dict__, "layers": (base.layers[0], toy)})

    def plain_forward(toks):
        pos = np.arange(len(toks))
        x = plain.embed(w["model.embed_tokens.weight"], toks)
        x = plain.decoder_layer(x, w, 0, cfg, pos)
        p = "model.layers.1."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + (np.cumsum(h, 0) / (pos + 1)[:, None]) @ w[p + "toy.weight"].astype(np.float64).T
        x = x + plain.mlp_block(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), w, p)
        return plain.linear(plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])

    return spec, w, cfg, plain_forward
