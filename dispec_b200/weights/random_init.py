"""Random-weights mode: a model folder (config.json, model.safetensors) or a model on the
device from a configuration and a seed.

Every value is a function of (seed, the tensor's ordinal among the checkpoint names in sorted
order, the element's index) and of nothing else (``counter_rng``): matrices, embeddings and
biases N(0, std), gains 1 + N(0, std), drawn in float32 and rounded once to the storage type.
The device kernel ``dsp_fill_normal`` and the numpy function ``counter_rng.normal`` give the same
bits, so a large model is filled on the device in place (no host copy of its weights exists)
while a test oracle recomputes any tensor of it on the CPU.
"""
from __future__ import annotations

import json
import os

import torch

from dispec_b200.weights import counter_rng
from dispec_b200.weights.loader import build_model
from dispec_b200.weights.safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def tensor_ordinals(names) -> dict:
    """name -> ordinal: the place of the name among the checkpoint's names in sorted order."""
    return {name: i for i, name in enumerate(sorted(names))}


def _mean_std(spec, name: str, std: float, overrides: dict) -> tuple[float, float]:
    return (1.0 if spec.init == "one_plus_normal" else 0.0), overrides.get(name, std)


class RandomSource:
    """A tensor source that computes each tensor when it is asked for, on the CPU (numpy) or,
    with ``device`` a CUDA device, by the fill kernel straight into device memory.  Tensors can
    be asked for in any order, any number of times."""

    def __init__(self, config, seed: int, std: float, dtype: str = "bfloat16",
                 overrides: dict | None = None, device=None):
        self._req = build_model(config).tensor_requirements()
        self._ordinal = tensor_ordinals(self._req)
        self._seed, self._std, self._store = int(seed), std, _STORE[dtype]
        self._overrides = overrides or {}
        self._device = torch.device(device) if device is not None else None
        if self._device is not None and self._device.type != "cuda":
            self._device = None

    def names(self):
        return list(self._req)

    def shape(self, name):
        return tuple(self._req[name].shape)

    def dtype(self, name):
        spec = self._req[name]
        return torch.int32 if spec.dtype == "int32" else (torch.float32 if spec.dtype == "float32" else self._store)

    def get(self, name):
        spec = self._req[name]
        store = self.dtype(name)
        if spec.dtype == "int32":
            return torch.zeros(spec.shape, dtype=torch.int32, device=self._device)
        if spec.init == "zeros":
            return torch.zeros(spec.shape, dtype=store, device=self._device)
        mean, std = _mean_std(spec, name, self._std, self._overrides)
        if self._device is not None and store in (torch.bfloat16, torch.float32):
            from dispec_b200.ops.elementwise import fill_normal
            out = torch.empty(spec.shape, dtype=store, device=self._device)
            return fill_normal(out, self._seed, self._ordinal[name], std, mean)
        t = torch.from_numpy(counter_rng.normal(self._seed, self._ordinal[name], tuple(spec.shape), std, mean))
        t = t.to(store)
        return t.to(self._device) if self._device is not None else t


def random_tensors(config, seed: int, std: float, dtype: str = "bfloat16",
                   overrides: dict | None = None, device=None) -> dict:
    """name -> tensor on the host.  ``overrides``: name -> std for single tensors (a wider output
    matrix keeps argmax away from near-ties in tests).  ``device``: a CUDA device that fills
    the tensors (same bits, much faster for large models)."""
    src = RandomSource(config, seed, std, dtype, overrides, device)
    return {name: src.get(name).cpu() for name in src.names()}


def load_random_model(config, seed: int, std: float = 0.02, dtype="bfloat16", device="cuda:0",
                      overrides: dict | None = None):
    """A model with random weights on the device, filled there; equal to writing the folder with
    ``write_random_model`` (stored as bfloat16) and loading it."""
    from dispec_b200.weights.loader import load_into
    model = build_model(config)
    src = RandomSource(config, seed, std, "bfloat16", overrides, device)
    return load_into(model, src, dtype, device, where="random weights")


def write_random_model(config, folder: str, seed: int, std: float = 0.02, dtype: str = "bfloat16",
                       overrides: dict | None = None, device=None) -> str:
    os.makedirs(folder, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(config, seed, std, dtype, overrides, device),
                      metadata={"format": "pt", "seed": seed, "std": std,
                                "generator": "philox4x32-10 box-muller, counter = element index, tensor ordinal"})
    return folder
