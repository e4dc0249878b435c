"""Typed model configurations read from an architecture's own config.json keys.

A configuration class is registered per architecture name (``architectures[0]`` of
config.json).  Nothing here carries a size: every number comes from the file, and a key
that is absent is an error that names it, except where the reference engine itself
falls back (``head_dim``, puneethgv/DiSpec dispec/engine/model_runner.py:70).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot be served, with the offending keys named."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations."""

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def flat(self) -> dict:
        """Scalars only, for logs and benchmark records."""
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, (int, float, str, bool)):
                out[f.name] = v
        return out


def _require(d: dict, keys: list[str], where: str) -> None:
    missing = [k for k in keys if k not in d or d[k] is None]
    if missing:
        raise ConfigError(f"{where}: config.json lacks required key(s): {', '.join(missing)}")


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """Qwen2 / Qwen2.5 dense decoder (``Qwen2ForCausalLM``).

    Keys as the reference reads them from the model's config object:
    dispec/engine/model_runner.py:68-72 (heads, kv heads, head_dim and its fallback),
    dispec/kv/paged_cache.py:44-55 (layers), dispec/engine/model_runner.py:79-84
    (``layer_types``), :86-87 (``rope_theta`` sits at the top level or, in newer
    files, under ``rope_parameters``).

    ``layer_windows[i]`` is 0 for a full-attention layer and W > 0 for a layer whose
    query at position p sees only keys b with p - W < b <= p.  The reference refuses
    such layers; this engine serves them through a cache group of their own.
    """

    architecture: ClassVar[str] = "Qwen2ForCausalLM"

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    hidden_act: str
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_windows: tuple[int, ...]
    bos_token_id: int | None = None
    eos_token_id: int | None = None

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        where = cls.architecture
        _require(d, ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "hidden_act",
                     "tie_word_embeddings", "max_position_embeddings"], where)
        heads = int(d["num_attention_heads"])
        kv_heads = int(d["num_key_value_heads"])
        hidden = int(d["hidden_size"])
        layers = int(d["num_hidden_layers"])
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(f"{where}: num_attention_heads={heads} is not a positive multiple of "
                              f"num_key_value_heads={kv_heads}")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{where}: no head_dim given and hidden_size={hidden} is not "
                                  f"divisible by num_attention_heads={heads}")
            head_dim = hidden // heads
        head_dim = int(head_dim)
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"{where}: head_dim={head_dim} must be positive and even for rotary pairs")
        # rope_theta: top level (released Qwen2.5 files) or nested (newer writers)
        rope = d.get("rope_parameters") or {}
        scaling = d.get("rope_scaling")
        rope_type = rope.get("rope_type", "default")
        if scaling:
            rope_type = scaling.get("rope_type", scaling.get("type", rope_type))
        if rope_type != "default":
            raise ConfigError(f"{where}: rotary type {rope_type!r} is not implemented (only 'default')")
        if d.get("rope_theta") is not None:
            theta = float(d["rope_theta"])
        elif rope.get("rope_theta") is not None:
            theta = float(rope["rope_theta"])
        else:
            raise ConfigError(f"{where}: config.json lacks rope_theta (top level or rope_parameters)")
        if d["hidden_act"] != "silu":
            raise ConfigError(f"{where}: hidden_act={d['hidden_act']!r} is not implemented (only 'silu')")
        # which layers slide
        windows = [0] * layers
        layer_types = d.get("layer_types")
        if layer_types is not None:
            if len(layer_types) != layers:
                raise ConfigError(f"{where}: layer_types has {len(layer_types)} entries for {layers} layers")
            for i, t in enumerate(layer_types):
                if t == "sliding_attention":
                    # a file that marks a layer as sliding while it switches windows off contradicts
                    # itself; which of the two wins is not for the engine to guess
                    if d.get("use_sliding_window") is False or d.get("sliding_window") is None:
                        raise ConfigError(f"{where}: layer_types[{i}] is 'sliding_attention' but "
                                          f"use_sliding_window is false or sliding_window is missing")
                    windows[i] = int(d["sliding_window"])
                elif t != "full_attention":
                    raise ConfigError(f"{where}: layer_types[{i}]={t!r} is not implemented")
        elif d.get("use_sliding_window", False):
            _require(d, ["sliding_window", "max_window_layers"], where)
            first = int(d["max_window_layers"])
            windows = [int(d["sliding_window"]) if i >= first else 0 for i in range(layers)]
        if any(w < 0 for w in windows):
            raise ConfigError(f"{where}: sliding_window must be positive")
        return cls(
            vocab_size=int(d["vocab_size"]), hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]), num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            rms_norm_eps=float(d["rms_norm_eps"]), rope_theta=theta, hidden_act=d["hidden_act"],
            tie_word_embeddings=bool(d["tie_word_embeddings"]),
            max_position_embeddings=int(d["max_position_embeddings"]),
            layer_windows=tuple(windows),
            bos_token_id=d.get("bos_token_id"), eos_token_id=d.get("eos_token_id"),
        )

    def to_dict(self) -> dict:
        d: dict[str, Any] = {
            "architectures": [self.architecture], "model_type": "qwen2",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "hidden_act": self.hidden_act, "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "bos_token_id": self.bos_token_id, "eos_token_id": self.eos_token_id,
        }
        if any(self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = max(self.layer_windows)
            d["layer_types"] = ["sliding_attention" if w else "full_attention"
                                for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
        return d


def read_config_json(path: str) -> dict:
    """The dict in ``<folder>/config.json`` (or in the file itself)."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.exists(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path) as f:
        return json.load(f)


def load_model_config(path_or_dict) -> ModelConfig:
    """Choose the configuration class by ``architectures[0]`` through the registry."""
    from dispec_b200.registry import architecture_entry

    d = path_or_dict if isinstance(path_or_dict, dict) else read_config_json(path_or_dict)
    archs = d.get("architectures")
    if not archs:
        raise ConfigError("config.json lacks 'architectures'")
    return architecture_entry(archs[0]).config_class.from_dict(d)
