"""Engine, cache and generation settings, with the reference's names and defaults.

``GenConfig``: puneethgv/DiSpec dispec/config.py:31-43.  ``KVConfig``: dispec/config.py:46-51.
``EngineConfig`` gathers what the reference passes as constructor arguments
(dispec/sched/scheduler.py:61-63: num_blocks=2048, max_batch_tokens=2048, chunk_size).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class GenConfig:
    max_new_tokens: int = 256
    temperature: float = 0.0  # <= 0 means greedy
    top_p: float = 1.0
    top_k: int = 0  # 0 means off
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


@dataclass
class KVConfig:
    block_size: int = 16  # tokens per page
    max_blocks: int = 4096  # pages in each pool


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"  # "bfloat16" or "float32" (true 32-bit everywhere)
    kv: KVConfig = field(default_factory=KVConfig)
    num_blocks: int | None = None  # pages per cache group; None: kv.max_blocks
    max_batch_tokens: int = 2048  # token budget of one step
    chunk_size: int | None = None  # largest prompt portion; None: max_batch_tokens
    max_num_seqs: int = 256  # live requests (= state slots)
    max_model_len: int | None = None  # longest request; None: the model's max_position_embeddings
    cuda_graph: bool = True  # replay captured graphs for all-decode steps (bfloat16 only)
    device: str = "cuda:0"

    def pages(self) -> int:
        return self.num_blocks if self.num_blocks is not None else self.kv.max_blocks
