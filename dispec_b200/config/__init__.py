from dispec_b200.config.engine_config import EngineConfig, GenConfig, KVConfig
from dispec_b200.config.model_config import (ConfigError, ModelConfig, Qwen2Config,
                                             load_model_config, read_config_json)

__all__ = ["EngineConfig", "GenConfig", "KVConfig", "ConfigError", "ModelConfig", "Qwen2Config",
           "load_model_config", "read_config_json"]
