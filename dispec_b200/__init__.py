"""dispec_b200: a small, whole LLM inference engine for one NVIDIA B200.

Model folder (config.json + safetensors) -> typed configuration -> model assembled from
registered parts -> paged cache + step function -> scheduler -> sampled tokens.
"""
__version__ = "0.1.0"

from dispec_b200.config import EngineConfig, GenConfig, KVConfig, load_model_config  # noqa: E402,F401
from dispec_b200.registry import (architectures, register_architecture,  # noqa: E402,F401
                                  register_part)


def __getattr__(name):
    # heavier pieces load on first use, so that configuration and cache bookkeeping import
    # without touching CUDA
    if name in ("load_model", "build_model", "write_random_model", "load_random_model"):
        import dispec_b200.weights as w
        return getattr(w, name)
    if name in ("LLMEngine", "ContinuousBatchingEngine", "ModelRunner", "SeqEntry", "Scheduler"):
        import dispec_b200.engine as e
        return getattr(e, name)
    if name in ("SamplingParams", "sample"):
        import dispec_b200.sampling as s
        return getattr(s, name)
    raise AttributeError(name)
