"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor the model's parts declare is drawn in checkpoint-name order from one
``torch.Generator(seed)``: matrices, embeddings and biases N(0, std), gains 1 + N(0, std).
Values are drawn in float32 and stored in ``dtype``.
"""
from __future__ import annotations

import json
import os

import torch

from dispec_b200.weights.loader import build_model
from dispec_b200.weights.safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(config, seed: int, std: float, dtype: str = "bfloat16",
                   overrides: dict | None = None) -> dict:
    """name -> tensor.  ``overrides``: name -> std for single tensors (a wider output matrix
    keeps argmax away from near-ties in tests)."""
    model = build_model(config)
    g = torch.Generator().manual_seed(seed)
    store = _STORE[dtype]
    out = {}
    for name, spec in model.tensor_requirements().items():
        s = (overrides or {}).get(name, std)
        if spec.dtype == "int32":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        if spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32)
        else:
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32) * s
            if spec.init == "one_plus_normal":
                t = t + 1.0
        out[name] = t.to(torch.float32 if spec.dtype == "float32" else store)
    return out


def write_random_model(config, folder: str, seed: int, std: float = 0.02, dtype: str = "bfloat16",
                       overrides: dict | None = None) -> str:
    os.makedirs(folder, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(config, seed, std, dtype, overrides),
                      metadata={"format": "pt", "seed": seed, "std": std})
    return folder
