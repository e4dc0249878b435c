"""Weights by tensor name: checks a source of tensors against what the model's parts
declare, converts and uploads them.

Floating-point tensors a part declares as "model" are kept in the engine's type (bfloat16,
or float32 on the 32-bit path); "float32" tensors stay 32-bit in every mode; integer tables
become int32.  Every disagreement between the source and the model is collected and raised
as one ``WeightError`` that lists missing tensors, unexpected tensors and wrong shapes.
"""
from __future__ import annotations

import torch

from dispec_b200.config.model_config import load_model_config, read_config_json
from dispec_b200.models.model import DecoderModel
from dispec_b200.registry import architecture_entry
from dispec_b200.weights.safetensors_io import CheckpointFolder

_ENGINE_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                  "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


class WeightError(ValueError):
    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_type=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_type = sorted(wrong_type)
        lines = [f"{where}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {tuple(got)}, the model needs {tuple(want)}")
        for name, got, want in self.wrong_type:
            lines.append(f"  wrong type: {name} is {got}, the model needs {want}")
        super().__init__("\n".join(lines))


def engine_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, not {name}")
        return name
    if name not in _ENGINE_DTYPES:
        raise ValueError(f"engine dtype must be bfloat16 or float32, not {name!r}")
    return _ENGINE_DTYPES[name]


def check_source(model: DecoderModel, source, where: str) -> dict:
    """Compares names and shapes; returns the requirements if everything fits."""
    req = model.tensor_requirements()
    have = set(source.names())
    missing = [n for n in req if n not in have]
    unexpected = [n for n in have if n not in req and n not in model.spec.optional_tensors]
    wrong_shape, wrong_type = [], []
    for n, spec in req.items():
        if n not in have:
            continue
        if tuple(source.shape(n)) != tuple(spec.shape):
            wrong_shape.append((n, tuple(source.shape(n)), tuple(spec.shape)))
        is_float = source.dtype(n).is_floating_point
        if spec.dtype == "int32" and is_float:
            wrong_type.append((n, str(source.dtype(n)), "an integer type"))
        if spec.dtype != "int32" and not is_float:
            wrong_type.append((n, str(source.dtype(n)), "a floating-point type"))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_type)
    return req


def load_into(model: DecoderModel, source, dtype, device, where: str = "weights") -> DecoderModel:
    dtype = engine_dtype(dtype)
    if torch.device(device).type != "cuda":
        raise ValueError("the engine runs on a CUDA device only (there is no CPU path)")
    req = check_source(model, source, where)
    tensors = {}
    for name, spec in req.items():
        t = source.get(name)
        if spec.dtype == "model":
            target = dtype
        elif spec.dtype == "float32":
            target = torch.float32
        elif spec.dtype == "int32":
            target = torch.int32
        else:
            raise ValueError(f"tensor {name!r}: unknown storage class {spec.dtype!r}")
        tensors[name] = t.to(device=device, dtype=target).contiguous()
    model.load(tensors, dtype, torch.device(device))
    return model


def build_model(config) -> DecoderModel:
    """Model (without weights) for a configuration object, through the registry."""
    entry = architecture_entry(config.architecture)
    return DecoderModel(entry.builder(config), config)


def load_model(folder: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """A model folder (config.json + safetensors) -> a model on the device.  Same role and
    argument order as the reference's ``load_model(name, dtype, device)``
    (puneethgv/DiSpec dispec/models/loader.py:18-27)."""
    config = load_model_config(read_config_json(folder))
    model = build_model(config)
    return load_into(model, CheckpointFolder(folder), dtype, device, where=folder)
