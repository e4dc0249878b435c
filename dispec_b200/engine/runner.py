"""The step function: runs a batch of (request, its next tokens) from the cache and returns
the logits at the wanted places.

``ModelRunner`` owns the cache manager, the device pools and the state buffers of one model.
``step(entries)`` runs only the tokens it is given, as one flat batch (portions of prompts
beside single decoded tokens), and leaves their keys and values in the pages.  It plays the
role of ``ModelRunner.forward`` + ``ModelRunner.logits`` of the reference (puneethgv/DiSpec
dispec/engine/model_runner.py:188-231) with the bookkeeping its callers do by hand
(dispec/sched/scheduler.py:132-197) moved behind one call.
"""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.cache.manager import CacheManager
from dispec_b200.cache.storage import CacheStorage, StateStorage
from dispec_b200.engine.batch import HostStaging, SeqEntry, StepPlanLayout, build_context
from dispec_b200.ops import library as _library
from dispec_b200.models.model import DecoderModel

# Context lengths for which a captured decode step is laid out (the last class is the engine's
# own maximum): few enough that little is captured, far enough apart that a short context does
# not pay for the key sharing that a long one needs.
GRAPH_CONTEXT_CLASSES = (2048, 8192, 32768, 131072, 524288)


class ModelRunner:
    def __init__(self, model: DecoderModel, page_size: int = 16, num_pages=4096,
                 max_num_seqs: int = 256, poison: bool = False, cuda_graph: bool = False,
                 max_model_len: int | None = None):
        if model.device is None:
            raise ValueError("the model has no weights yet (load it first)")
        self.model = model
        self.dtype = model.dtype
        self.device = model.device
        self.page_size = page_size
        groups = model.cache_groups
        counts = [num_pages] * len(groups) if isinstance(num_pages, int) else list(num_pages)
        self.cache = CacheManager(groups, page_size, counts, max_num_seqs)
        self.storage = CacheStorage(groups, page_size, counts, self.dtype, self.device, poison=poison)
        self.states = StateStorage(model.state_needs, max_num_seqs, self.device)
        self.staging = HostStaging(self.device)
        self.poison = poison  # tests: pages given back are filled with NaN
        self.vocab_size = model.spec.vocab_size
        self.num_steps = 0
        self.cuda_graph = (bool(cuda_graph) and self.dtype == torch.bfloat16
                           and all(getattr(p, "graph_safe", True) for p in model._parts))
        # captured decode steps, one per padded batch size; the page tables of a captured step
        # have room for the longest sequence the pools or the model allow
        # (powers of two, and the largest batch itself so that every batch has a bucket)
        self.graph_buckets = [1 << i for i in range(13) if (1 << i) < max_num_seqs]
        self.graph_buckets.append(max_num_seqs)
        # the longest request: the configuration's max_position_embeddings unless the caller says
        # otherwise (angles are computed from the position, so no table stands in the way of more)
        limit = max_model_len or model.spec.max_position or (1 << 30)
        self.max_model_len = min(limit, self.cache.capacity_tokens())
        # page-table width of a captured step: a full group never holds more pages than its pool has;
        # a window group's table is indexed by logical page (holes behind the window), so its
        # length follows the context, not the pool
        longest = max(1, -(-self.max_model_len // page_size))
        self._graph_pages = [longest if g.window > 0 else max(1, min(c, longest))
                             for g, c in zip(groups, counts)]
        self._graphs: dict = {}

    # ---------------------------------------------------------------- request lifecycle
    def admit(self, req_id, prompt_len: int = 0, max_total_len: int = 0, max_chunk: int = 1) -> None:
        slot = self.cache.admit(req_id, prompt_len, max_total_len, max_chunk)
        if self.states.buffers:
            self.states.reset_slot(slot)

    def release(self, req_id) -> None:
        self._poison(self.cache.free(req_id))

    def _poison(self, released) -> None:
        if self.poison and released:
            for g in range(len(self.cache.groups)):
                self.storage.poison_pages(g, [p for gg, p in released if gg == g])

    # ----------------------------------------------------------------------- the step
    @torch.inference_mode()
    def step(self, entries: list[SeqEntry], feed_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Logits [number of wanted places, vocab] in float32, in the order of ``entries`` and
        of each entry's ``want``.  ``feed_tokens`` (int32, on the device): the tokens sampled in
        the previous step; an entry with ``feed_row`` r takes its single token from row r of it
        on the device, so the host need not have seen that token yet."""
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        seen = set()
        for e in entries:
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if not self.cache.has(e.req_id):
                raise KeyError(f"request {e.req_id!r} was not admitted")
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.req_id!r} brings no tokens")
            stored = self.cache.num_tokens(e.req_id)
            if e.start != stored:
                raise ValueError(f"request {e.req_id!r}: tokens start at position {e.start} but "
                                 f"{stored} tokens are stored")
        if any(e.feed_row >= 0 for e in entries) and feed_tokens is None:
            raise ValueError("an entry is fed from the previous step but feed_tokens is missing")
        for e in entries:  # may raise OutOfPagesError before anything ran
            self.cache.extend(e.req_id, e.start + len(e.tokens))
        if (self.cuda_graph and self.graph_buckets and len(entries) <= self.graph_buckets[-1]
                and all(len(e.tokens) == 1 for e in entries)):
            return self._graph_step(entries, feed_tokens)
        ctx, _ = build_context(entries, self.cache, self.storage, self.states, self.staging,
                               self.dtype, self.device, self.model.attention_tile_tokens,
                               self.vocab_size)
        if ctx.num_fed:
            ops.feed_tokens(ctx.token_ids, ctx.feed_src, feed_tokens)
        x, pending = self.model.forward(ctx)
        n_rows = ctx.logit_rows.shape[0]
        if n_rows:
            logits = self.model.logits(ctx, x, pending, ctx.logit_rows)
        else:
            logits = torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        for e in entries:
            self._poison(self.cache.commit(e.req_id, e.start + len(e.tokens)))
        self.num_steps += 1
        return logits

    # -------------------------------------------------------- captured all-decode steps
    def _context_class(self, entries: list) -> int:
        """The context length a captured step is laid out for: the smallest class that holds the
        step's longest request.  How the keys of a row are shared among CTAs is decided on the
        host from this bound, so a graph serves one class."""
        longest = max(e.start + len(e.tokens) for e in entries)
        for bound in GRAPH_CONTEXT_CLASSES:
            if longest <= bound < self.max_model_len:
                return bound
        return self.max_model_len

    def _capture(self, bucket: int, ctx_bound: int) -> dict:
        """Captures one decode step of ``bucket`` single-token rows, none longer than
        ``ctx_bound``, as a CUDA graph.  Every
        integer input lives in one device buffer of fixed address and layout; a replay copies
        the step's values there first.  Rows beyond the live requests carry position -1 and
        length 0, which the kernels skip."""
        plan = StepPlanLayout([], self.cache, self.model.attention_tile_tokens, self.vocab_size,
                              pad_seqs=bucket, fixed_pages=self._graph_pages)
        buffer = torch.empty(plan.total, dtype=torch.int32, device=self.device)
        self.staging.upload(plan.total, plan.fill, into=buffer)
        ctx = plan.context(buffer, self.storage, self.states, self.dtype, self.device)
        ctx.max_ctx_len = ctx_bound  # choices made on the host must not vary per step
        ctx.graph_capture = True

        def run():
            x, pending = self.model.forward(ctx)
            return self.model.logits(ctx, x, pending, ctx.logit_rows)

        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = _library.LaunchCounter.n
        with torch.cuda.graph(graph):
            logits = run()
        entry = dict(graph=graph, buffer=buffer, total=plan.total, logits=logits,
                     launches=_library.LaunchCounter.n - before)
        self._graphs[(bucket, ctx_bound)] = entry
        return entry

    def _graph_step(self, entries: list, feed_tokens=None) -> torch.Tensor:
        bucket = next(b for b in self.graph_buckets if b >= len(entries))
        ctx_bound = self._context_class(entries)
        g = self._graphs.get((bucket, ctx_bound)) or self._capture(bucket, ctx_bound)
        plan = StepPlanLayout(entries, self.cache, self.model.attention_tile_tokens, self.vocab_size,
                              pad_seqs=bucket, fixed_pages=self._graph_pages)
        assert plan.total == g["total"]
        self.staging.upload(plan.total, plan.fill, into=g["buffer"])
        if plan.num_fed:
            (o_ids, n_ids), (o_src, n_src) = plan.layout["token_ids"], plan.layout["feed_src"]
            ops.feed_tokens(g["buffer"][o_ids:o_ids + n_ids], g["buffer"][o_src:o_src + n_src], feed_tokens)
        g["graph"].replay()
        _library.LaunchCounter.n += g["launches"]
        for e in entries:
            self._poison(self.cache.commit(e.req_id, e.start + len(e.tokens)))
        self.num_steps += 1
        # rows of the padded batch follow the sorted (= given) order of the single-token entries
        wanted = [i for i, e in enumerate(entries) if e.want]
        logits = g["logits"][:len(entries)]
        if len(wanted) != len(entries):
            logits = logits[torch.tensor(wanted, dtype=torch.long, device=self.device)]
        return logits

    def check_device(self, where: str = "step") -> None:
        """Raises if a kernel recorded a bad page or token id (synchronises)."""
        ops.raise_on_device_error(where)
