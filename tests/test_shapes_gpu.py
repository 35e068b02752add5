"""Sizes drawn at random from everything a configuration allows: head sizes in steps of 16 (and 256), any number of
heads and of heads per group, widths, feed-forward widths and vocabularies that are no power of two (odd ones too,
which the tensor-core kernels refuse and the general kernels take), page sizes that are no power of two, tied and
separate output tables. Each drawn model runs a prompt whole, in portions beside another request, and decoded token
by token, in both dtypes, against the plain implementation: a kernel either takes a size or hands it on; it never
returns something else."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import assert_logits_close, sharp_weights

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = np.random.default_rng(1000 + seed)
    head_dim = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 256]))
    kv_heads = int(rng.choice([1, 2, 3, 5]))
    group = int(rng.choice([1, 2, 3, 4, 7, 8, 16] if head_dim <= 128 else [1, 2]))
    hidden = int(rng.choice([40, 72, 99, 136, 250, 264, 520]))
    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
        "vocab_size": int(rng.choice([97, 256, 389, 1000, 1537])), "hidden_size": hidden,
        "intermediate_size": int(rng.choice([48, 100, 131, 264, 528])), "num_hidden_layers": int(rng.choice([1, 2, 3])),
        "num_attention_heads": kv_heads * group, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "max_position_embeddings": 512, "rms_norm_eps": float(rng.choice([1e-6, 1e-5, 3e-4])),
        "rope_theta": float(rng.choice([1e4, 5e5, 1e6])), "tie_word_embeddings": bool(rng.integers(0, 2)),
    }
    page = int(rng.choice([4, 8, 12, 16, 24, 32, 64]))
    return cfg, page


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_a_drawn_configuration_matches_the_plain_implementation(tmp_path, seed, dtype):
    from tiny_inference_engine_b200 import StepEntry, StepRunner, load_model, make_cache
    cfg, page = draw(seed)
    w = sharp_weights(cfg, seed)
    plain.write_model_dir(tmp_path, cfg, w)
    rng = np.random.default_rng(seed)
    V = cfg["vocab_size"]
    a, b = rng.integers(0, V, 150).tolist(), rng.integers(0, V, 41).tolist()
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    want_a, want_b = plain.forward(wq, cfg, a), plain.forward(wq, cfg, b)
    what = f"seed {seed}: {cfg['num_attention_heads']}/{cfg['num_key_value_heads']} heads of {cfg['head_dim']}, hidden " \
           f"{cfg['hidden_size']}, page {page}"

    model = load_model(tmp_path, dtype)
    pages = -(-150 // page) + -(-41 // page) + 2
    cache, states = make_cache(model, page_size=page, num_pages=pages, max_requests=4)
    runner = StepRunner(model, cache, 160, 4, 200, states=states)

    def logits(entries):
        return runner.run(entries).float().cpu().numpy().copy()

    # whole
    ra = cache.new_request()
    assert cache.reserve(ra, 150)
    assert_logits_close(logits([StepEntry(ra, a, 0, list(range(150)))]), want_a, dtype, what + ", whole")
    cache.release(ra)
    # portions of one request beside portions and decoded tokens of another, on the pages just given back
    ra, rb = cache.new_request(), cache.new_request()
    assert cache.reserve(ra, 150) and cache.reserve(rb, 41)
    got_a, got_b = [], []
    got_a.append(logits([StepEntry(ra, a[:67], 0, list(range(67)))]))
    out = logits([StepEntry(ra, a[67:69], 67, [0, 1]), StepEntry(rb, b[:30], 0, list(range(30)))])
    got_a.append(out[:2]); got_b.append(out[2:])
    out = logits([StepEntry(rb, b[30:31], 30, [0]), StepEntry(ra, a[69:130], 69, list(range(61)))])
    got_b.append(out[:1]); got_a.append(out[1:])
    for i in range(10):                                             # both decode; the first steps are captured graphs
        out = logits([StepEntry(ra, a[130 + i:131 + i], 130 + i, [0]), StepEntry(rb, b[31 + i:32 + i], 31 + i, [0])])
        got_a.append(out[:1]); got_b.append(out[1:])
    out = logits([StepEntry(ra, a[140:], 140, list(range(10)))])
    got_a.append(out)
    torch.cuda.synchronize()
    runner.check()
    assert_logits_close(np.concatenate(got_a), want_a, dtype, what + ", in portions and decoded")
    assert_logits_close(np.concatenate(got_b), want_b, dtype, what + ", beside it")
