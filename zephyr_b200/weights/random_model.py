"""The random-weights mode: write a model folder from a configuration and a seed.

The reference has no such mode (it loads checkpoints only).  Distributions:
projection matrices N(0, 0.02), embedding N(0, 0.02), norm scales
1 + N(0, 0.01); each tensor is seeded by the model seed and its own name.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .loader import RandomWeights
from .safetensors_io import save_safetensors


def write_random_model(config, seed: int, out_dir: str | Path, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration with
    ``to_dict()`` and ``to_model_spec()``) into ``out_dir`` and return the folder."""
    from ..parts import expected_weights

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    spec = config.to_model_spec()
    store = RandomWeights(expected_weights(spec), seed, dtype=dtype, device="cpu")
    tensors = {name: store.read(name) for name in store.names()}
    (out / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n", encoding="utf-8")
    save_safetensors(out / "model.safetensors", tensors,
                     metadata={"format": "pt", "seed": str(seed), "generator": "zephyr_b200.random"})
    return out
