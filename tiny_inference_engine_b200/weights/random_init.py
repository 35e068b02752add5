"""The random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.registry import resolve_architecture
from .loader import RandomSource
from .safetensors import write_safetensors


def write_random_model(model_dir, config_json: dict, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       norm_std: float = 0.01, device: str = "cpu") -> Path:
    """Writes `model_dir/config.json` and `model_dir/model.safetensors` for the architecture that
    `config_json` names; matrices N(0, std) in `dtype`, norm weights 1 + N(0, norm_std) in float32. The values
    are those that `--random-weights` draws for the same configuration and seed, on whichever `device` they
    are drawn here (a large model is drawn far faster on the GPU)."""
    from ..parts.model import expected_tensors
    arch = resolve_architecture(config_json)
    spec = arch.build_spec(arch.parse_config(config_json))
    spec.validate()
    source = RandomSource(expected_tensors(spec), seed, dtype, std, norm_std, device=device)
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps(config_json, indent=1))
    write_safetensors(d / "model.safetensors", {n: source.get(n).cpu() for n in sorted(source.needs)})
    return d
