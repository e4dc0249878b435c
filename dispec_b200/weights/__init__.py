from dispec_b200.weights.loader import WeightError, build_model, load_into, load_model
from dispec_b200.weights.random_init import (RandomSource, load_random_model, random_tensors,
                                             write_random_model)
from dispec_b200.weights.safetensors_io import (CheckpointFolder, SafetensorsError, SafetensorsFile,
                                                write_safetensors)

__all__ = ["WeightError", "build_model", "load_into", "load_model", "random_tensors", "RandomSource", "load_random_model",
           "write_random_model", "CheckpointFolder", "SafetensorsError", "SafetensorsFile",
           "write_safetensors"]
