"""Continuous batching: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

Structure, names and defaults follow puneethgv/DiSpec dispec/sched/scheduler.py: states
(:28-32), ``Request`` (:35-57), per step first one token for every running request, then
prompts in progress, then waiting requests by (-priority, id) (:132-197), admission that
stops at the first request that does not fit (:159-164), a portion that does not finish the
prompt yields no token (:189-197), the end-of-sequence token is kept in the output (:222-232).

Decided here, where the reference raises out of ``step()`` (its ``append_token`` at :137
lets OutOfBlocksError through): when a running request cannot get a page, the newest live
request is preempted by recomputation: its pages are given back, it returns to the head of the
waiting queue with prompt + emitted tokens as its new prompt, and it keeps what it emitted.
A request that could never fit the pool alone is refused in ``add_request``.  Sampling uses
each request's own parameters and generator.

Overlapped steps (not in the reference): the engine launches step n + 1 before it has read the
tokens of step n.  ``Scheduler.launched`` puts a placeholder into the output of every request
the step samples for (so lengths, and finishing by length, are known at once);
``Scheduler.resolve`` fills the placeholders in when the tokens arrive and retires requests
that drew their end-of-sequence token, one step late: such a request has one more step in
flight, whose token is dropped.  A request whose newest token is a placeholder is scheduled
with ``SeqEntry.feed_row``: the step takes the token from the previous step's result on the
device.  Preemption needs the real tokens (the request is recomputed from them), so the
engine resolves the step in flight first whenever pages are short.

``Scheduler`` is pure bookkeeping over a ``CacheManager`` (testable without a GPU);
``ContinuousBatchingEngine`` joins it with the step function and the sampler.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum, auto

import torch

from dispec_b200.cache.manager import CacheManager
from dispec_b200.cache.pages import OutOfPagesError
from dispec_b200.config.engine_config import KVConfig
from dispec_b200.engine.batch import SeqEntry
from dispec_b200.sampling.sampler import SamplingParams, make_rng


PENDING = -1  # placeholder in output_ids for a token that a step in flight will sample


class State(Enum):
    WAITING = auto()
    PREFILLING = auto()
    RUNNING = auto()
    FINISHED = auto()


@dataclass
class Request:
    id: int
    prompt_ids: list
    params: SamplingParams
    max_new_tokens: int
    eos_id: int | None = None
    output_ids: list = field(default_factory=list)
    state: State = State.WAITING
    priority: int = 0  # higher is admitted sooner
    prefill_pos: int = 0  # tokens of the current prompt already stored
    prefilled: bool = False
    num_preemptions: int = 0
    finish_reason: str | None = None
    rng: object = None
    _recompute: list | None = None  # prompt + emitted tokens after a preemption
    _pending_row: int = -1  # row of the newest launched step's tokens that holds output_ids[-1]

    @property
    def feed(self) -> list:
        """Tokens that must be stored before the next token can be sampled."""
        return self._recompute if self._recompute is not None else self.prompt_ids

    @property
    def done(self) -> bool:
        if len(self.output_ids) >= self.max_new_tokens:
            return True
        return bool(self.output_ids) and self.eos_id is not None and self.output_ids[-1] == self.eos_id


@dataclass
class StepPlan:
    entries: list  # SeqEntry, single-token entries first
    sampled: list  # requests that get a token this step, in the order of the logits rows
    num_decode_tokens: int = 0
    num_prefill_tokens: int = 0
    pending_index: dict = field(default_factory=dict)  # request id -> index of its placeholder in output_ids


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int = 2048, chunk_size: int | None = None,
                 max_model_len: int | None = None, on_admit=None, on_free=None):
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.chunk_size = chunk_size or max_batch_tokens
        # the largest portion a step brings: the caller's, the budget, and what the window groups'
        # pools can hold beside the window (so that a request that was admitted once, and comes
        # back after a preemption with a longer prompt, can always be admitted again)
        self.max_portion = min(self.chunk_size, max_batch_tokens, cache.largest_chunk())
        self.max_model_len = max_model_len
        self.waiting: list[Request] = []
        self.prefilling: list[Request] = []
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._ids = itertools.count()
        self._on_admit = on_admit or (lambda req_id, *a: cache.admit(req_id, *a))
        self._on_free = on_free or cache.free
        self.num_steps = 0
        self.num_prefill_tokens = 0
        self.num_decode_tokens = 0
        self.num_preemptions = 0

    # -------------------------------------------------------------------------- requests
    def add_request(self, prompt_ids, max_new_tokens: int, params: SamplingParams | None = None,
                    eos_id: int | None = None, priority: int = 0) -> int:
        prompt = list(prompt_ids)
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        total = len(prompt) + max_new_tokens
        # the last emitted token is never stored, hence total - 1 positions
        if total - 1 > self.cache.capacity_tokens():
            raise ValueError(f"request of {len(prompt)} + {max_new_tokens} tokens can never fit the "
                             f"cache pool of {self.cache.capacity_tokens()} tokens")
        if self.max_model_len is not None and total - 1 > self.max_model_len:
            raise ValueError(f"request of {len(prompt)} + {max_new_tokens} tokens exceeds the longest "
                             f"sequence the engine serves ({self.max_model_len})")
        # admission asks every cache group for pages (the prompt's in a full group, the most the
        # request ever holds at once in a window group): a request whose need exceeds a whole pool
        # would wait forever at the head of the queue
        if self.max_portion < 1:
            raise ValueError("a window group's pool is too small to hold its window and one more token")
        need = self.cache.admission_need(*self._admission_args(len(prompt), max_new_tokens))
        for g, (n, pool) in enumerate(zip(need, self.cache.pools)):
            if n > pool.num_pages:
                raise ValueError(f"request of {len(prompt)} + {max_new_tokens} tokens needs {n} pages of cache "
                                 f"group {g} at once, the pool has {pool.num_pages}")
        params = params or SamplingParams()
        req = Request(next(self._ids), prompt, params, max_new_tokens, eos_id, priority=priority,
                      rng=make_rng(params))
        self.waiting.append(req)
        return req.id

    def _admission_args(self, feed_len: int, remaining_new: int) -> tuple:
        """(prompt length, positions ever stored, largest portion) of a request that enters with
        ``feed_len`` tokens to store and ``remaining_new`` tokens to emit; the last emitted token
        is never stored."""
        return (feed_len, feed_len + remaining_new - 1, max(1, min(self.max_portion, feed_len)))

    def has_work(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running)

    def collect_outputs(self) -> dict:
        return {r.id: r.output_ids for r in self.finished + self.running}

    # ------------------------------------------------------------------------ preemption
    def _preempt(self, req: Request) -> None:
        if PENDING in req.output_ids:
            raise RuntimeError("a request with a token still in flight cannot be preempted "
                               "(resolve the launched step first)")
        self._on_free(req.id)
        if req in self.running:
            self.running.remove(req)
        if req in self.prefilling:
            self.prefilling.remove(req)
        req.state = State.WAITING
        req.prefill_pos = 0
        req.prefilled = False
        req._recompute = list(req.prompt_ids) + list(req.output_ids)
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.append(req)

    def _newest_live(self) -> Request | None:
        live = self.running + self.prefilling
        if not live:
            return None
        return max(live, key=lambda r: (-r.priority, r.id))

    # ------------------------------------------------------------------------- one step
    def schedule(self) -> StepPlan:
        budget = self.max_batch_tokens
        entries: dict[int, SeqEntry] = {}
        sampled: list[Request] = []
        n_dec = n_pre = 0

        # 1) one token for every running request, oldest first
        for req in sorted(self.running, key=lambda r: r.id):
            if budget < 1:
                break
            if req.state != State.RUNNING:
                continue  # preempted a moment ago
            stored = self.cache.num_tokens(req.id)
            placed = True
            while not self.cache.can_extend(req.id, stored + 1):
                victim = self._newest_live()
                if victim is None or victim is req:
                    # the request itself is the newest: it waits, the older ones go on
                    if victim is req:
                        self._preempt(req)
                    placed = False
                    break
                if victim.id in entries:
                    gone = entries.pop(victim.id)
                    budget += len(gone.tokens)
                    n_dec -= 1
                    sampled.remove(victim)
                self._preempt(victim)
            if not placed:
                continue
            self.cache.extend(req.id, stored + 1)
            if req.output_ids[-1] == PENDING:  # sampled by the step in flight: fed on the device
                entries[req.id] = SeqEntry(req.id, [0], stored, [0], feed_row=req._pending_row)
            else:
                entries[req.id] = SeqEntry(req.id, [req.output_ids[-1]], stored, [0])
            sampled.append(req)
            budget -= 1
            n_dec += 1

        # 2) prompts in progress, then waiting requests by priority and age
        self.waiting.sort(key=lambda r: (-r.priority, r.id))
        for req in self.prefilling + self.waiting:
            if budget < 1:
                break
            feed = req.feed
            if req.state == State.WAITING:
                args = self._admission_args(len(feed), req.max_new_tokens - len(req.output_ids))
                if not self.cache.can_admit(*args):
                    break
                self._on_admit(req.id, *args)
                req.state = State.PREFILLING
                self.waiting.remove(req)
                self.prefilling.append(req)
            chunk = min(len(feed) - req.prefill_pos, self.max_portion, budget)
            try:
                self.cache.extend(req.id, req.prefill_pos + chunk)
            except OutOfPagesError:
                break
            finishes = req.prefill_pos + chunk >= len(feed)
            entries[req.id] = SeqEntry(req.id, feed[req.prefill_pos:req.prefill_pos + chunk],
                                       req.prefill_pos, [chunk - 1] if finishes else [])
            req.prefill_pos += chunk
            budget -= chunk
            n_pre += chunk
            if finishes:
                sampled.append(req)
                req.prefilled = True
                req.state = State.RUNNING
                self.prefilling.remove(req)
                self.running.append(req)

        ordered = [e for e in entries.values() if len(e.tokens) == 1] + \
                  [e for e in entries.values() if len(e.tokens) != 1]
        order = {e.req_id: i for i, e in enumerate(ordered)}
        want_rows = [r for r in sampled]
        # logits rows follow the order of the entries
        want_rows.sort(key=lambda r: order[r.id])
        self.num_decode_tokens += n_dec
        self.num_prefill_tokens += n_pre
        return StepPlan(ordered, want_rows, n_dec, n_pre)

    def needs_resolved_tokens(self) -> bool:
        """True when the next ``schedule`` may have to preempt, which needs every emitted token
        on the host: some cache group has fewer free pages than there are running requests."""
        if not self.running:
            return False
        return self.cache.min_free_pages() < len(self.running)

    def launched(self, plan: StepPlan) -> None:
        """The step is on its way.  Every request it samples for gets a placeholder for the
        token; a request that reaches its length with it retires now (its pages may be given
        to steps launched later, which run after this one)."""
        self.num_steps += 1
        for row, req in enumerate(plan.sampled):
            plan.pending_index[req.id] = len(req.output_ids)
            req.output_ids.append(PENDING)
            req._pending_row = row
            if len(req.output_ids) >= req.max_new_tokens:
                req.finish_reason = "length"
                self._retire(req)

    def resolve(self, plan: StepPlan, token_ids: list) -> list[Request]:
        """The tokens of a launched step have arrived: fills the placeholders in and retires
        requests that drew their end-of-sequence token; returns the requests that are complete."""
        done = []
        for req, tid in zip(plan.sampled, token_ids):
            idx = plan.pending_index.get(req.id)
            if idx is None or idx >= len(req.output_ids) or req.output_ids[idx] != PENDING:
                continue  # cut off: the request ended at an earlier token
            req.output_ids[idx] = int(tid)
            if idx == len(req.output_ids) - 1:
                req._pending_row = -1
            if req.eos_id is not None and int(tid) == req.eos_id:
                del req.output_ids[idx + 1:]  # a later step in flight sampled past the end
                req._pending_row = -1
                req.finish_reason = "stop"
                if req.state != State.FINISHED:
                    self._retire(req)
                done.append(req)
            elif req.state == State.FINISHED and idx == len(req.output_ids) - 1:
                done.append(req)
        return done

    def _retire(self, req: Request) -> None:
        req.state = State.FINISHED
        if req in self.running:
            self.running.remove(req)
        self.finished.append(req)
        self._on_free(req.id)

    def process(self, plan: StepPlan, token_ids: list) -> list[Request]:
        """Appends the sampled tokens, retires finished requests; returns those retired
        (``launched`` and ``resolve`` in one, for a caller that waits for every step)."""
        self.launched(plan)
        return self.resolve(plan, token_ids)


class ContinuousBatchingEngine:
    """``ContinuousBatchingEngine(model, kv, num_blocks, max_batch_tokens, chunk_size)`` with
    ``add_request / step / has_work / run_until_done / collect_outputs`` as in the reference
    (dispec/sched/scheduler.py:60-63,85-101,234-244).  ``model`` is a model loaded by
    ``dispec_b200.load_model``; the reference's ``attn_backend`` and ``fuse`` switches have no
    counterpart (there is one attention path, projections are always fused).  ``max_model_len``
    replaces the configuration's ``max_position_embeddings`` as the longest request."""

    def __init__(self, model, kv: KVConfig | None = None, num_blocks: int = 2048,
                 max_batch_tokens: int = 2048, chunk_size: int | None = None, max_num_seqs: int = 256,
                 cuda_graph: bool = True, poison: bool = False, overlap: bool = True,
                 max_model_len: int | None = None):
        from dispec_b200.engine.runner import ModelRunner
        from dispec_b200.sampling.sampler import Sampler

        kv = kv or KVConfig()
        self.block_size = kv.block_size
        self.runner = ModelRunner(model, page_size=kv.block_size, num_pages=num_blocks,
                                  max_num_seqs=max_num_seqs, poison=poison, cuda_graph=cuda_graph,
                                  max_model_len=max_model_len)
        self.sampler = Sampler(model.device)
        self.scheduler = Scheduler(self.runner.cache, max_batch_tokens, chunk_size,
                                   max_model_len=max_model_len or model.spec.max_position or None,
                                   on_admit=self.runner.admit, on_free=self.runner.release)
        # overlap: step n + 1 is scheduled and launched while step n runs; its tokens are read
        # one step late (outputs and the queues lag by one step until has_work / collect_outputs /
        # run_until_done catch up)
        self.overlap = overlap
        self._inflight = None  # (plan, tokens on the device, pinned host copy, event)
        self._host_tokens = [torch.empty(max(max_num_seqs, 1), dtype=torch.int32, pin_memory=True)
                             for _ in range(3)]
        self._turn = 0

    # queues and counters under the reference's names
    waiting = property(lambda self: self.scheduler.waiting)
    prefilling = property(lambda self: self.scheduler.prefilling)
    running = property(lambda self: self.scheduler.running)
    finished = property(lambda self: self.scheduler.finished)
    num_steps = property(lambda self: self.scheduler.num_steps)
    num_prefill_tokens = property(lambda self: self.scheduler.num_prefill_tokens)
    num_decode_tokens = property(lambda self: self.scheduler.num_decode_tokens)
    num_preemptions = property(lambda self: self.scheduler.num_preemptions)

    def add_request(self, prompt_ids, max_new_tokens: int, params: SamplingParams | None = None,
                    eos_id: int | None = None, priority: int = 0) -> int:
        return self.scheduler.add_request(prompt_ids, max_new_tokens, params, eos_id, priority)

    def step(self) -> None:
        sched = self.scheduler
        if self._inflight is not None and (not self.overlap or sched.needs_resolved_tokens()):
            self.flush()
        plan = sched.schedule()
        if not plan.entries:
            had_inflight = self._inflight is not None
            self.flush()
            if not had_inflight and sched.has_work():
                # nothing ran, nothing was in flight, and requests remain: no later step can differ
                raise RuntimeError(
                    f"the scheduler is stuck: {len(sched.waiting)} waiting, {len(sched.prefilling)} in "
                    f"prefill, {len(sched.running)} running, and no step can be scheduled "
                    f"(free pages per group: {[p.available for p in sched.cache.pools]})")
            return
        feed = self._inflight[1] if self._inflight is not None else None
        logits = self.runner.step(plan.entries, feed_tokens=feed)
        tokens = self.sampler.sample_device(logits, [r.params for r in plan.sampled],
                                            [r.rng for r in plan.sampled])
        self._turn = (self._turn + 1) % len(self._host_tokens)
        if tokens.shape[0] > self._host_tokens[self._turn].shape[0]:
            self._host_tokens[self._turn] = torch.empty(tokens.shape[0], dtype=torch.int32, pin_memory=True)
        host = self._host_tokens[self._turn][:tokens.shape[0]]
        host.copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        sched.launched(plan)
        previous, self._inflight = self._inflight, (plan, tokens, host, event)
        if previous is not None:
            self._resolve(previous)
        if not self.overlap:
            self.flush()

    def _resolve(self, launched) -> None:
        plan, _, host, event = launched
        event.synchronize()
        self.scheduler.resolve(plan, host.tolist())

    def flush(self) -> None:
        """Reads the tokens of the step in flight, if any: afterwards outputs and queues are current."""
        if self._inflight is not None:
            launched, self._inflight = self._inflight, None
            self._resolve(launched)

    def collect_outputs(self) -> dict:
        self.flush()
        return self.scheduler.collect_outputs()

    def has_work(self) -> bool:
        self.flush()
        return self.scheduler.has_work()

    def run_until_done(self, max_steps: int = 100_000) -> None:
        """Steps until every request has finished; raises if ``max_steps`` do not suffice."""
        steps = 0
        while (self.scheduler.has_work() or self._inflight is not None) and steps < max_steps:
            self.step()
            steps += 1
        self.flush()
        if self.scheduler.has_work():
            raise RuntimeError(f"{max_steps} steps did not finish the requests")
