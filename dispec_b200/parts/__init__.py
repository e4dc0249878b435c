"""Built-in parts; importing this package registers them."""
from dispec_b200.parts import attention, block, embedding, norms, rotary, swiglu  # noqa: F401
from dispec_b200.parts.base import (Block, CacheNeed, CacheTensor, FeedForward, Mixer, Norm, Part, PartSpec,
                                    PositionEncoding, StateNeed, TensorSpec)

__all__ = ["Block", "CacheNeed", "CacheTensor", "FeedForward", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "StateNeed", "TensorSpec"]
