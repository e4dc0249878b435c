"""dispec_b200: a small, whole LLM inference engine for one NVIDIA B200.

Model folder (config.json + safetensors) -> typed configuration -> model assembled from
registered parts -> paged cache + step function -> scheduler -> sampled tokens.
"""
__version__ = "0.1.0"
