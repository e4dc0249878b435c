"""Single-sequence driver: prefill the whole prompt, sample, decode one token at a time, free
the pages in ``finally`` (puneethgv/DiSpec dispec/engine/engine.py:23-101)."""
from __future__ import annotations

import itertools

from dispec_b200.config.engine_config import KVConfig
from dispec_b200.engine.batch import SeqEntry
from dispec_b200.engine.runner import ModelRunner
from dispec_b200.sampling.sampler import Sampler, SamplingParams, make_rng


class LLMEngine:
    """``LLMEngine(model, kv, num_blocks, cuda_graph).generate(prompt_ids, max_new_tokens, params,
    eos_token_id, generator) -> list[int]``.  The reference's ``prefix_cache``, ``attn_backend``
    and ``fuse`` arguments have no counterpart here."""

    _seq_counter = itertools.count()

    def __init__(self, model, kv: KVConfig | None = None, num_blocks: int | None = None,
                 cuda_graph: bool = False):
        kv = kv or KVConfig()
        self.block_size = kv.block_size
        self.runner = ModelRunner(model, page_size=kv.block_size,
                                  num_pages=kv.max_blocks if num_blocks is None else num_blocks,
                                  max_num_seqs=4, cuda_graph=cuda_graph)
        self.sampler = Sampler(model.device)
        self.last_prefill_tokens = 0

    def generate(self, prompt_ids, max_new_tokens: int, params: SamplingParams | None = None,
                 eos_token_id: int | None = None, generator=None) -> list:
        params = params or SamplingParams()
        rng = make_rng(params, generator)
        prompt = list(prompt_ids)
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        seq_id = ("llm", next(self._seq_counter))
        self.runner.admit(seq_id)
        try:
            self.last_prefill_tokens = len(prompt)
            logits = self.runner.step([SeqEntry(seq_id, prompt, 0, [len(prompt) - 1])])
            next_id = self.sampler.sample(logits, [params], [rng])[0]
            out = [next_id]
            cur = len(prompt)
            while len(out) < max_new_tokens and next_id != eos_token_id:
                logits = self.runner.step([SeqEntry(seq_id, [next_id], cur, [0])])
                next_id = self.sampler.sample(logits, [params], [rng])[0]
                out.append(next_id)
                cur += 1
            return out
        finally:
            self.runner.release(seq_id)
