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


class RandomSource:
    """A tensor source that draws each tensor when it is asked for (same values as
    ``random_tensors``: one generator, checkpoint-name order), so that a large model reaches
    the device without a file in between."""

    def __init__(self, config, seed: int, std: float, dtype: str = "bfloat16",
                 overrides: dict | None = None):
        self._req = build_model(config).tensor_requirements()
        self._gen = torch.Generator().manual_seed(seed)
        self._std, self._store, self._overrides = std, _STORE[dtype], overrides or {}
        self._order = list(self._req)
        self._next = 0

    def names(self):
        return list(self._req)

    def shape(self, name):
        return tuple(self._req[name].shape)

    def dtype(self, name):
        spec = self._req[name]
        return torch.int32 if spec.dtype == "int32" else (torch.float32 if spec.dtype == "float32" else self._store)

    def get(self, name):
        if self._order[self._next] != name:
            raise RuntimeError("RandomSource hands tensors out once, in checkpoint-name order")
        self._next += 1
        spec = self._req[name]
        if spec.dtype == "int32":
            return torch.zeros(spec.shape, dtype=torch.int32)
        if spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32)
        else:
            t = torch.randn(spec.shape, generator=self._gen, dtype=torch.float32) * self._overrides.get(name, self._std)
            if spec.init == "one_plus_normal":
                t = t + 1.0
        return t.to(self.dtype(name))


def load_random_model(config, seed: int, std: float = 0.02, dtype="bfloat16", device="cuda:0",
                      overrides: dict | None = None):
    """A model with random weights on the device, equal to writing the folder with
    ``write_random_model`` (stored as bfloat16) and loading it."""
    from dispec_b200.weights.loader import load_into
    model = build_model(config)
    return load_into(model, RandomSource(config, seed, std, "bfloat16", overrides), dtype, device,
                     where="random weights")


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
