"""Shared fixtures. Tests marked `gpu` need a B200; everything else runs on the CPU."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import plain_qwen3 as plain  # noqa: E402

# Tolerances, fixed before the kernels were written. float32: what the baseline asks of the
# 32-bit path (max relative error 1e-4 of the row's largest logit, same argmax). bfloat16:
# 2e-2 of the largest logit, about five times the noise that rounding weights and
# activations to bfloat16 gives the plain implementation itself on these models
# (1.6e-3 to 4.4e-3, see tests/test_plain.py::test_bfloat16_noise_is_small).
TOL = {"float32": 1e-4, "bfloat16": 2e-2}

CONFIGS = {"tiny_a": (plain.TINY_A, 16), "tiny_b": (plain.TINY_B, 8), "tiny_c": (plain.TINY_C, 32),
           "tiny_d": (plain.TINY_D, 16), "tiny_e": (plain.TINY_E, 16), "tiny_b4": (plain.TINY_B4, 8)}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def sharp_weights(cfg, seed):
    """Random weights whose attention is not flat: q and k projections 12 times larger, so that a
    key that is skipped, read from a wrong page or masked wrongly moves the logits visibly."""
    w = plain.random_weights(cfg, seed)
    for name in w:
        if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            w[name] = (w[name] * 12.0).astype(np.float32)
    return w


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """name -> (config, page size, float32 weights, model folder) for the tiny configurations."""
    out = {}
    for i, (name, (cfg, page)) in enumerate(CONFIGS.items()):
        w = sharp_weights(cfg, i)
        d = tmp_path_factory.mktemp(name)
        plain.write_model_dir(d, cfg, w)
        out[name] = (cfg, page, w, d)
    return out


def rel_err(a, b):
    """Largest absolute difference of a row, relative to the row's largest reference value; worst row."""
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    a, b = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
    return float((np.abs(a - b).max(axis=-1) / np.abs(b).max(axis=-1)).max())


def assert_logits_close(got, want, dtype, what=""):
    err = rel_err(got, want)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} above {TOL[dtype]:.0e} ({dtype})"
    if dtype == "float32":
        g, w = np.asarray(got), np.asarray(want)
        g, w = g.reshape(-1, g.shape[-1]), w.reshape(-1, w.shape[-1])
        # same argmax wherever the reference's own top two are further apart than the tolerance
        top2 = np.sort(w, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2 * TOL[dtype] * np.abs(w).max(axis=-1)
        assert (g.argmax(-1)[clear] == w.argmax(-1)[clear]).all(), f"{what}: argmax differs"
