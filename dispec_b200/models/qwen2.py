"""Qwen2 / Qwen2.5 dense decoder as a ``ModelSpec``.

Tensor names are those of a ``Qwen2ForCausalLM`` checkpoint, which the reference reaches
through ``model.model.embed_tokens / .layers[i].self_attn.{q,k,v,o}_proj / .mlp.{gate,up,down}_proj
/ .input_layernorm / .post_attention_layernorm / .norm`` and ``model.lm_head``
(puneethgv/DiSpec dispec/engine/model_runner.py:62-66,104-118).  Biases on q, k, v only; a
tied head reuses the embedding tensor and the file carries no ``lm_head.weight``.
"""
from __future__ import annotations

from dispec_b200.config.model_config import Qwen2Config
from dispec_b200.models.spec import LayerCall, ModelSpec
from dispec_b200.parts.base import PartSpec
from dispec_b200.registry import register_architecture


def build_qwen2(cfg: Qwen2Config) -> ModelSpec:
    h = cfg.hidden_size
    rotary = PartSpec("position_encoding", "rotary",
                      {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        mixer = PartSpec(
            "mixer", "gqa_attention",
            {"hidden_size": h, "num_heads": cfg.num_attention_heads,
             "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "qkv_bias": True,
             "position_encoding": rotary, "window": cfg.layer_windows[i]},
            {f"{n}_proj.{k}": f"{a}{n}_proj.{k}" for n in "qkv" for k in ("weight", "bias")}
            | {"o_proj.weight": a + "o_proj.weight"})
        ffn = PartSpec(
            "feed_forward", "swiglu", {"hidden_size": h, "intermediate_size": cfg.intermediate_size},
            {f"{n}_proj.weight": f"{p}mlp.{n}_proj.weight" for n in ("gate", "up", "down")})
        norm1 = PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.rms_norm_eps},
                         {"weight": p + "input_layernorm.weight"})
        norm2 = PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.rms_norm_eps},
                         {"weight": p + "post_attention_layernorm.weight"})
        layers.append(PartSpec("block", "pre_norm", {"mixer_norm": norm1, "mixer": mixer,
                                                     "ffn_norm": norm2, "feed_forward": ffn}))
    embedding = PartSpec("embedding", "token_embedding",
                         {"vocab_size": cfg.vocab_size, "hidden_size": h},
                         {"weight": "model.embed_tokens.weight"})
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    head = PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h},
                    {"weight": head_name})
    final_norm = PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.rms_norm_eps},
                          {"weight": "model.norm.weight"})
    return ModelSpec(
        architecture=cfg.architecture, embedding=embedding, layers=layers, final_norm=final_norm,
        head=head, schedule=[LayerCall(i, i, True) for i in range(cfg.num_hidden_layers)],
        optional_tensors=frozenset({"lm_head.weight"}) if cfg.tie_word_embeddings else frozenset(),
        vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings)


register_architecture(Qwen2Config.architecture, Qwen2Config, build_qwen2)
