"""The plain implementation against the reference's own CPU code (tests/golden) and against itself."""
from pathlib import Path

import numpy as np
import pytest

import plain_qwen3 as plain

GOLDEN = Path(__file__).resolve().parent / "golden"


# model of tests/golden -> (configuration, seed of its weights)
MODELS = {"tiny_a": (plain.TINY_A, 0), "tiny_b4": (plain.TINY_B4, 1)}


def golden_requests(name):
    """[(tokens to generate, prompt)] of a golden workload."""
    out = []
    for line in (GOLDEN / f"{name}_requests.txt").read_text().splitlines():
        f = [int(x) for x in line.split()]
        out.append((f[0], f[1:]))
    return out


def golden_tokens(name, small=False):
    lines = (GOLDEN / f"{name}_greedy{'_small' if small else ''}.txt").read_text().splitlines()
    return [[int(x) for x in l.split()] for l in lines if not l.startswith("#")]


@pytest.mark.parametrize("name", list(MODELS))
def test_logits_and_hidden_states_match_the_reference(name):
    cfg, seed = MODELS[name]
    w = plain.random_weights(cfg, seed)
    for i, (_, ids) in enumerate(golden_requests(name)):
        hidden = []
        logits = plain.forward(w, cfg, ids, hidden_out=hidden)
        ref = np.fromfile(GOLDEN / f"{name}_logits_{i}.f32", dtype="<f4").reshape(len(ids), -1)
        ref_h = np.fromfile(GOLDEN / f"{name}_hidden_{i}.f32", dtype="<f4").reshape(cfg["num_hidden_layers"], len(ids), -1)
        assert ref.shape[1] == cfg["vocab_size"] and ref_h.shape[2] == cfg["hidden_size"]
        assert np.abs(logits - ref).max() <= 2e-6 * np.abs(ref).max()
        assert np.abs(np.stack(hidden) - ref_h).max() <= 2e-6 * np.abs(ref_h).max()
        assert (logits.argmax(-1) == ref.argmax(-1)).all()


@pytest.mark.parametrize("name", list(MODELS))
def test_greedy_tokens_match_the_reference_engine(name):
    cfg, seed = MODELS[name]
    w = plain.random_weights(cfg, seed)
    for (n_new, ids), ref in zip(golden_requests(name), golden_tokens(name)):
        assert plain.generate(w, cfg, ids, n_new) == ref


def test_the_reference_engine_generates_the_same_tokens_when_it_preempts():
    """tiny-B's workload from a pool of so few pages that the reference's scheduler preempts a request
    (tests/engine/test_engine_batching.cpp:58-75): the tokens are those of the roomy run."""
    header = (GOLDEN / "tiny_b4_greedy_small.txt").read_text().splitlines()[0]
    assert header.startswith("# preemptions ") and int(header.split()[2]) >= 1
    assert golden_tokens("tiny_b4", small=True) == golden_tokens("tiny_b4")


def test_rope_position_zero_is_identity_and_scores_depend_on_distance_only():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 32)), rng.standard_normal((1, 32))
    assert np.allclose(plain.rope_neox(q, [0], 1, 32, 1e4), q)
    a = plain.rope_neox(q, [7], 1, 32, 1e4) @ plain.rope_neox(k, [3], 1, 32, 1e4).T
    b = plain.rope_neox(q, [104], 1, 32, 1e4) @ plain.rope_neox(k, [100], 1, 32, 1e4).T
    assert abs(a - b) < 1e-4


def test_attention_is_causal_and_grouped():
    rng = np.random.default_rng(1)
    T, Hq, Hkv, Dh = 9, 4, 2, 8
    q, k, v = (rng.standard_normal((T, h * Dh)) for h in (Hq, Hkv, Hkv))
    full = plain.causal_attention(q, k, v, Hq, Hkv, Dh)
    k2, v2 = k.copy(), v.copy()
    k2[5:], v2[5:] = 9.0, -3.0   # the future of rows 0..4
    assert np.allclose(plain.causal_attention(q, k2, v2, Hq, Hkv, Dh)[:5], full[:5])
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.copy()
    v3[:, Dh:] += 1.0
    out = plain.causal_attention(q, k, v3, Hq, Hkv, Dh).reshape(T, Hq, Dh)
    assert np.allclose(out[:, :2], full.reshape(T, Hq, Dh)[:, :2]) and np.allclose(out[:, 2:], full.reshape(T, Hq, Dh)[:, 2:] + 1.0)
    # a window of 3 keeps keys t-2..t
    win = plain.causal_attention(q, k, v, Hq, Hkv, Dh, window=3)
    assert np.allclose(win[:3], full[:3]) and not np.allclose(win[6], full[6])
    assert np.allclose(win[6], plain.causal_attention(q[4:7], k[4:7], v[4:7], Hq, Hkv, Dh)[2])


def test_rms_norm_and_swiglu_formulas():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.rms_norm(x, np.array([1.0, 2.0]), 0.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])
    assert np.allclose(plain.swiglu(np.array([0.0, 1.0]), np.array([5.0, 2.0])), [0.0, 2.0 / (1 + np.exp(-1.0))])


def test_bfloat16_noise_is_small():
    """The size of bfloat16 rounding noise on the tiny models; the bfloat16 tolerance of the GPU
    tests (2e-2) is set from it."""
    for cfg in (plain.TINY_A, plain.TINY_B, plain.TINY_C):
        w = plain.random_weights(cfg, 0)
        toks = np.random.default_rng(1).integers(0, cfg["vocab_size"], 64)
        wb = {n: (plain.round_bf16(t) if t.ndim == 2 else t) for n, t in w.items()}
        a, b = plain.forward(wb, cfg, toks), plain.forward(w, cfg, toks, storage="bfloat16")
        assert np.abs(a - b).max() / np.abs(a).max() < 8e-3


def test_philox_known_answers():
    """Random123's known-answer vectors for philox4x32-10."""
    assert plain.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert plain.philox4x32([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert plain.philox4x32([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]) == \
        [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_sampling_rules():
    z = np.array([0.1, 2.0, 2.0, -1.0])
    assert plain.sample(z) == 1                                  # first maximum
    assert plain.sample(z, temperature=1e-45) == 1               # 1/T not finite: greedy
    assert plain.sample(np.array([0.0, np.inf, np.inf]), temperature=1.0, u=0.99) == 1
    assert plain.sample(z, temperature=1.0, top_k=1, u=0.999) == 1
    counts = np.zeros(4)
    for i in range(4000):
        counts[plain.sample(z, temperature=1.0, u=(i + 0.5) / 4000)] += 1
    p = np.exp(z - z.max()); p /= p.sum()
    assert np.abs(counts / 4000 - p).max() < 2e-3
    # top_p keeps the smallest prefix reaching p of the mass: 2.0, 2.0 hold 0.83
    assert {plain.sample(z, temperature=1.0, top_p=0.8, u=u) for u in np.linspace(0, 0.999, 50)} == {1, 2}
