"""Safetensors files, the binding check and the random-weights mode (CPU)."""
import json
import struct

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_inference_engine_b200.config import parse_qwen3_config, qwen3_spec
from tiny_inference_engine_b200.errors import LoadError
from tiny_inference_engine_b200.parts import expected_tensors
from tiny_inference_engine_b200.weights import (RandomSource, SafetensorsFile, SafetensorsSource, TensorNeed, bind_check,
                                                write_random_model, write_safetensors)


def needs_of(cfg):
    return expected_tensors(qwen3_spec(parse_qwen3_config(cfg)))


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    write_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    for name, want in t.items():
        got = f.tensor(name)
        assert got.dtype == want.dtype and tuple(got.shape) == tuple(want.shape) and torch.equal(got, want)


def test_reads_what_the_plain_writer_writes(tmp_path):
    w = plain.random_weights(plain.TINY_A, 3)
    plain.write_model_dir(tmp_path, plain.TINY_A, w, bf16=True)
    src = SafetensorsSource(tmp_path)
    got = src.get("model.layers.1.mlp.up_proj.weight")
    assert got.dtype == torch.bfloat16                      # stored bfloat16 stays bfloat16
    assert np.array_equal(got.float().numpy(), plain.round_bf16(w["model.layers.1.mlp.up_proj.weight"]))
    assert src.get("model.norm.weight").dtype == torch.float32  # stored 32-bit stays 32-bit
    bind_check(needs_of(plain.TINY_A), src)


def _raw(tmp_path, header: bytes, data: bytes = b"", hlen=None):
    p = tmp_path / "model.safetensors"
    p.write_bytes(struct.pack("<Q", len(header) if hlen is None else hlen) + header + data)
    return p


@pytest.mark.parametrize("make,text", [
    (lambda d: (d / "model.safetensors").write_bytes(b""), "empty"),
    (lambda d: (d / "model.safetensors").write_bytes(b"\x01\x02"), "truncated"),
    (lambda d: _raw(d, b"{}", hlen=1000), "past the end"),
    (lambda d: _raw(d, b"{nope"), "invalid JSON"),
    (lambda d: _raw(d, json.dumps({"t": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}).encode(), b"\0" * 8), "unsupported dtype F64"),
    (lambda d: _raw(d, json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}).encode(), b"\0" * 8), "outside"),
    (lambda d: _raw(d, json.dumps({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode(), b"\0" * 8), "needs 12"),
    (lambda d: _raw(d, json.dumps({"t": {"dtype": "F32", "shape": [2 ** 40, 2 ** 40], "data_offsets": [0, 8]}}).encode(), b"\0" * 8), "overflowing"),
    (lambda d: _raw(d, json.dumps({"t": {"dtype": "F32"}}).encode()), "malformed"),
])
def test_corrupt_files_name_the_problem(tmp_path, make, text):
    make(tmp_path)
    with pytest.raises(LoadError, match=text):
        SafetensorsFile(tmp_path / "model.safetensors")


def test_missing_file_and_duplicate_across_shards(tmp_path):
    with pytest.raises(LoadError, match="cannot open"):
        SafetensorsSource(tmp_path)
    write_safetensors(tmp_path / "a.safetensors", {"x": torch.zeros(1)})
    write_safetensors(tmp_path / "b.safetensors", {"x": torch.zeros(1)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "a.safetensors", "y": "b.safetensors"}}))
    with pytest.raises(LoadError, match="duplicate tensor 'x'"):
        SafetensorsSource(tmp_path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = plain.random_weights(plain.TINY_B, 0)
    del w["model.layers.2.self_attn.k_norm.weight"]
    del w["lm_head.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = np.zeros(256, dtype=np.float32)
    w["model.layers.1.mlp.down_proj.weight"] = w["model.layers.1.mlp.down_proj.weight"].T.copy()
    plain.write_model_dir(tmp_path, plain.TINY_B, w)
    with pytest.raises(LoadError) as e:
        bind_check(needs_of(plain.TINY_B), SafetensorsSource(tmp_path), what="Qwen3ForCausalLM")
    msg = str(e.value)
    assert "missing tensors: " in msg and "'model.layers.2.self_attn.k_norm.weight'" in msg and "'lm_head.weight'" in msg
    assert "tensors not used by Qwen3ForCausalLM: 'model.layers.0.self_attn.q_proj.bias'" in msg
    assert "'model.layers.1.mlp.down_proj.weight' has shape [200, 96], expected [96, 200]" in msg


def test_tied_model_accepts_a_duplicate_head_and_untied_needs_one(tmp_path):
    w = plain.random_weights(plain.TINY_A, 0)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].copy()
    plain.write_model_dir(tmp_path, plain.TINY_A, w)
    bind_check(needs_of(plain.TINY_A), SafetensorsSource(tmp_path))
    w["lm_head.weight"] = np.zeros((3, 3), dtype=np.float32)
    plain.write_model_dir(tmp_path, plain.TINY_A, w)
    with pytest.raises(LoadError, match="lm_head.weight' has shape"):
        bind_check(needs_of(plain.TINY_A), SafetensorsSource(tmp_path))


def test_integer_tensor_where_a_matrix_is_expected(tmp_path):
    w = plain.random_weights(plain.TINY_A, 0)
    w["model.norm.weight"] = np.ones(64, dtype=np.int32)
    plain.write_model_dir(tmp_path, plain.TINY_A, w)
    with pytest.raises(LoadError, match="dtype I32"):
        bind_check(needs_of(plain.TINY_A), SafetensorsSource(tmp_path))


def test_random_model_folder(tmp_path):
    d = write_random_model(tmp_path / "m", plain.TINY_B, seed=5, dtype=torch.bfloat16)
    assert json.loads((d / "config.json").read_text())["hidden_size"] == 96
    src = SafetensorsSource(d)
    bind_check(needs_of(plain.TINY_B), src)
    q = src.get("model.layers.0.self_attn.q_proj.weight")
    assert q.dtype == torch.bfloat16 and 0.015 < q.float().std() < 0.025 and abs(q.float().mean()) < 2e-3
    n = src.get("model.layers.0.input_layernorm.weight")
    assert n.dtype == torch.float32 and abs(n.mean() - 1) < 0.01 and 0.003 < n.std() < 0.02
    # the same seed gives the same bytes, another seed does not
    d2 = write_random_model(tmp_path / "m2", plain.TINY_B, seed=5, dtype=torch.bfloat16)
    d3 = write_random_model(tmp_path / "m3", plain.TINY_B, seed=6, dtype=torch.bfloat16)
    assert (d / "model.safetensors").read_bytes() == (d2 / "model.safetensors").read_bytes()
    assert (d / "model.safetensors").read_bytes() != (d3 / "model.safetensors").read_bytes()


def test_random_source_is_per_tensor():
    needs = needs_of(plain.TINY_A)
    a = RandomSource(needs, 1, torch.float32).get("model.layers.1.mlp.up_proj.weight")
    fewer = {k: v for k, v in needs.items() if "layers.0" not in k}
    b = RandomSource(needs, 1, torch.float32).get("model.layers.1.mlp.up_proj.weight")
    assert torch.equal(a, b) and len(fewer) < len(needs)


def test_counter_based_normal_values_are_a_function_of_seed_tensor_and_element():
    """Philox against the scalar generator of the sampling code, any slice equal to the same slice of the whole,
    streams that differ by seed and by tensor, and the statistics of a standard normal."""
    from tiny_inference_engine_b200.sampling import philox4x32
    from tiny_inference_engine_b200.weights.counter_random import _philox4x32_10, standard_normal
    c = torch.tensor([0, 1, 2 ** 33 + 5, 12345678901], dtype=torch.int64)
    words = _philox4x32_10(c, 0xDEADBEEF, 0x12345678)
    for i, ci in enumerate(c.tolist()):
        assert tuple(int(x[i]) for x in words) == tuple(philox4x32((ci & 0xFFFFFFFF, ci >> 32, 0, 0), (0xDEADBEEF, 0x12345678)))
    z = standard_normal(3, 7, 0, 400_000)
    for start, count in [(0, 1), (1, 6), (1001, 5000), (399_997, 3)]:
        assert torch.equal(standard_normal(3, 7, start, count), z[start:start + count])
    assert not torch.equal(standard_normal(4, 7, 0, 64), z[:64]) and not torch.equal(standard_normal(3, 8, 0, 64), z[:64])
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1) < 5e-3 and abs((z.abs() > 2).double().mean() - 0.0455) < 2e-3
    assert abs((z ** 3).mean()) < 0.02 and abs((z ** 4).mean() - 3) < 0.05 and z.abs().max() < 6.5
    lag = (z[:-1] * z[1:]).mean()                 # neighbours come from one Philox call: still uncorrelated
    assert abs(lag) < 5e-3


@pytest.mark.gpu
def test_random_weights_drawn_on_the_gpu_are_those_of_the_written_folder(tmp_path):
    """`--random-weights` (drawn on the device) and `tie make-random` (drawn on the CPU, written to a folder) name the
    same model by configuration and seed: every tensor bit for bit, in both dtypes."""
    for dtype in (torch.bfloat16, torch.float32):
        d = write_random_model(tmp_path / str(dtype), plain.TINY_D, seed=9, dtype=dtype)
        folder = SafetensorsSource(d)
        on_gpu = RandomSource(needs_of(plain.TINY_D), 9, dtype, device="cuda")
        for name in folder.shapes():
            a, b = folder.get(name), on_gpu.get(name).cpu()
            assert a.dtype == b.dtype and torch.equal(a, b), name
    big = RandomSource({"w": TensorNeed((5000, 4099))}, 2, torch.bfloat16, device="cuda").get("w")   # more than one piece
    assert torch.equal(big.cpu()[-3:], RandomSource({"w": TensorNeed((5000, 4099))}, 2, torch.bfloat16).get("w")[-3:])
