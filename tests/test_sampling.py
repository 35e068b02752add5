"""Sampling parameters, the Philox generator and the host sampler (CPU)."""
import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_inference_engine_b200.errors import InvalidArgument
from host_sampler import sample_host
from tiny_inference_engine_b200.sampling import SamplingParams, philox4x32, uniform


def test_params_are_checked():
    SamplingParams().validate()
    for bad in (dict(temperature=-1.0), dict(temperature=float("nan")), dict(temperature=float("inf")), dict(top_k=-1),
                dict(top_p=0.0), dict(top_p=1.5), dict(max_tokens=0), dict(seed=-1)):
        with pytest.raises(InvalidArgument):
            SamplingParams(**bad).validate()
    assert SamplingParams().temperature == 0.0 and SamplingParams().top_k == 0 and SamplingParams().top_p == 1.0
    assert SamplingParams().max_tokens == 256 and SamplingParams().seed == 0


def test_generator_matches_the_published_vectors_and_the_plain_one():
    assert philox4x32((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    for seed, i in ((0, 0), (7, 3), (2 ** 40 + 5, 2 ** 33), (2 ** 64 - 1, 10)):
        assert uniform(seed, i) == plain.uniform_for(seed, i) and 0.0 <= uniform(seed, i) < 1.0


def test_subnormal_temperature_is_greedy_and_device_path_choice():
    assert SamplingParams(temperature=1e-45).inv_temperature() == 0.0
    assert SamplingParams(temperature=0.5).inv_temperature() == 2.0
    assert not SamplingParams(temperature=0.7).filters and not SamplingParams(top_k=5).filters   # greedy takes the maximum
    assert SamplingParams(temperature=0.7, top_k=5).filters and SamplingParams(temperature=0.7, top_p=0.9).filters


def test_host_sampler_follows_the_plain_one():
    rng = np.random.default_rng(0)
    for trial in range(200):
        z = (rng.standard_normal(97) * 3).astype(np.float32)
        p = SamplingParams(temperature=float(rng.choice([0.0, 0.3, 1.0, 2.5])), top_k=int(rng.choice([0, 1, 5, 200])),
                           top_p=float(rng.choice([1.0, 0.9, 0.3])), seed=int(rng.integers(0, 2 ** 62)))
        want = plain.sample(z, p.temperature, p.top_k, p.top_p, plain.uniform_for(p.seed, trial))
        assert sample_host(z, p, trial) == want


def test_errors_and_certain_tokens():
    with pytest.raises(InvalidArgument, match="empty"):
        sample_host(np.array([], dtype=np.float32), SamplingParams(), 0)
    with pytest.raises(InvalidArgument, match="logit 1 is NaN"):
        sample_host(np.array([0.0, np.nan], dtype=np.float32), SamplingParams(), 0)
    with pytest.raises(InvalidArgument, match="-inf"):
        sample_host(np.array([-np.inf, -np.inf], dtype=np.float32), SamplingParams(), 0)
    assert sample_host(np.array([1.0, np.inf, np.inf], dtype=np.float32), SamplingParams(temperature=1.0), 0) == 1
    assert sample_host(np.array([2.0, 5.0, 5.0], dtype=np.float32), SamplingParams(), 0) == 1


def test_frequencies_follow_softmax():
    z = np.array([0.0, 1.0, 2.0, -50.0], dtype=np.float32)
    p = SamplingParams(temperature=0.8, seed=11)
    counts = np.bincount([sample_host(z, p, i) for i in range(6000)], minlength=4)
    want = np.exp(z / 0.8 - (z / 0.8).max())
    want /= want.sum()
    assert np.abs(counts / 6000 - want).max() < 0.02 and counts[3] == 0
