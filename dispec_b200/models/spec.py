"""Declarative description of a decoder: parts with their parameters and tensor names, and
the order in which the layers run.

``ModelSpec.schedule`` is data: a list of ``LayerCall``.  A layer may be named twice (its
weights run again, each call with a cache of its own) and a call may read the cache another
call wrote (``cache`` equal to that call's, ``write=False``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from dispec_b200.parts.base import PartSpec


@dataclass(frozen=True)
class LayerCall:
    layer: int  # index into ModelSpec.layers
    cache: int | None = None  # label of the layer cache this call uses (None: the call's own index)
    write: bool = True  # False: read-only use of a cache another call writes


@dataclass
class ModelSpec:
    architecture: str
    embedding: PartSpec
    layers: list[PartSpec]  # block specs
    final_norm: PartSpec
    head: PartSpec
    schedule: list[LayerCall] = field(default_factory=list)
    optional_tensors: frozenset = frozenset()  # checkpoint names that may be present and are ignored
    vocab_size: int = 0
    max_position: int = 0

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [LayerCall(i, i, True) for i in range(len(self.layers))]
