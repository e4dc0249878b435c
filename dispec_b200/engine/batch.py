"""The flat batch one step runs, and the context the parts see.

A step is a list of ``SeqEntry``: for each request its next tokens (a portion of a prompt,
or one decoded token) and the places among them whose logits are wanted.  ``build_context``
orders single-token entries first, lays every integer array of the step out in one pinned
host buffer, copies it to the device once, and returns a ``StepContext`` whose fields are
views into that device buffer.  The reference builds the same information as Python lists
and one tensor per array (puneethgv/DiSpec dispec/sched/scheduler.py:120-127,203-208,
dispec/engine/model_runner.py:26-32,202-212) and materialises a slot per context token;
here kernels get the page tables.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch


@dataclass
class SeqEntry:
    req_id: Any
    tokens: list
    start: int  # position of tokens[0]; equals the request's stored length
    want: list = field(default_factory=list)  # indices into tokens
    feed_row: int = -1  # >= 0: the single token is row feed_row of the previous step's sampled tokens


@dataclass
class LayerCacheView:
    tensors: dict  # name -> [num_pages, heads, page_size, width]: what the mixer keeps per token
    page_table: torch.Tensor  # [S, max_pages] int32, -1 where a page was given back
    group: int
    write: bool
    page_size: int
    num_pages: int
    window: int

    @property
    def key_pool(self) -> torch.Tensor:
        return self.tensors["key"]

    @property
    def value_pool(self) -> torch.Tensor:
        return self.tensors["value"]


@dataclass
class LayerStateView:
    buffer: torch.Tensor  # [max_num_seqs, *shape]
    slots: torch.Tensor  # [S] int32: state slot of each sequence of the batch


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepContext:
    """Everything a part may read about the current step."""

    def __init__(self):
        self.dtype = None
        self.device = None
        self.num_tokens = 0
        self.num_seqs = 0
        self.num_decode_seqs = 0  # single-token sequences, placed first
        self.token_ids = self.positions = self.seq_of_token = None  # [T] int32
        self.q_start = None  # [S + 1] int32: first flat row of each sequence
        self.ctx_len = None  # [S] int32: stored length after this step
        self.state_slot = None  # [S] int32
        self.logit_rows = None  # [n] int32
        self.feed_src = None  # [S] int32: row of the previous step's tokens that feeds a single token, or -1
        self.logit_rows_are_all = False  # the wanted rows are 0..T-1 in order
        self.page_tables: list = []  # per cache group [S, max_pages] int32
        self.host_q_len: list = []
        self.host_q_start: list = []
        self.host_state_slot: list = []
        self.host_ctx_len: list = []
        self.max_ctx_len = 0
        self.attention_tiles: dict = {}  # tokens per tile -> (tile_seq, tile_tok0, n_tiles) device int32
        self.storage = None
        self.states = None
        self.cache_groups = None
        self.page_size = 0
        self.decode_splits = 0  # fixed number of key splits for single-token rows (0: chosen per step)
        self.decode_outer = 0  # fixed number of key ranges per single-token row beyond the cluster (0: chosen)
        self.num_fed = 0  # single tokens whose value comes from the previous step on the device
        self.graph_capture = False  # host-side choices must not depend on the step's values
        self.scratch: dict = {}

    def cache_view(self, placement, write: bool) -> LayerCacheView:
        g = placement.group
        tensors = self.storage.layer_tensors(g, placement.slot)
        num_pages = next(iter(tensors.values())).shape[0]
        return LayerCacheView(tensors, self.page_tables[g], g, write, self.page_size, num_pages,
                              self.cache_groups[g].window)

    def state_view(self, index: int) -> LayerStateView:
        return LayerStateView(self.states.buffers[index], self.state_slot)


class HostStaging:
    """Two pinned host buffers used in turn, and the device buffer they are copied to."""

    def __init__(self, device, capacity: int = 1 << 16):
        self.device = device
        self.capacity = 0
        self._host = []
        self._events = []
        self._dev = None
        self._turn = 0
        self.last_bytes = 0  # bytes of the latest host-to-device copy
        self._grow(capacity)

    def _grow(self, n: int) -> None:
        cap = max(n, self.capacity * 2)
        self._host = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [None, None]
        self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.capacity = cap

    def upload(self, n: int, fill, into: torch.Tensor | None = None) -> torch.Tensor:
        """``fill(numpy int32 array of length n)`` writes the step's integers; returns the
        device copy (valid until the next upload).  ``into``: a device buffer of fixed address
        to copy to instead (a captured graph reads it)."""
        if n > self.capacity:
            self._grow(n)
        self._turn ^= 1
        ev = self._events[self._turn]
        if ev is not None:
            ev.synchronize()
        host = self._host[self._turn]
        fill(host.numpy()[:n])
        dev = self._dev[:n] if into is None else into[:n]
        dev.copy_(host[:n], non_blocking=True)
        self.last_bytes = 4 * n
        ev = torch.cuda.Event()
        ev.record()
        self._events[self._turn] = ev
        return dev


def order_entries(entries: list) -> list:
    """Indices of the entries with single-token ones first (stable)."""
    dec = [i for i, e in enumerate(entries) if len(e.tokens) == 1]
    rest = [i for i, e in enumerate(entries) if len(e.tokens) != 1]
    return dec + rest


def plan_layout(T: int, S: int, n_rows: int, pages_per_group: list, tiles: dict) -> tuple[dict, int]:
    """Offsets of every array inside the step's integer buffer."""
    off = 0
    layout = {}

    def put(name, n):
        nonlocal off
        layout[name] = (off, n)
        off += _align4(max(n, 1))

    put("token_ids", T)
    put("positions", T)
    put("seq_of_token", T)
    put("q_start", S + 1)
    put("ctx_len", S)
    put("state_slot", S)
    put("logit_rows", n_rows)
    put("feed_src", S)
    for g, mp in enumerate(pages_per_group):
        put(f"page_table{g}", S * mp)
    for tpt, nt in tiles.items():
        put(f"tile_seq{tpt}", nt)
        put(f"tile_tok0{tpt}", nt)
    return layout, off


class StepPlanLayout:
    """Sizes, offsets and host-side values of one step's integer arrays."""

    def __init__(self, entries: list, cache, tile_tokens: list, vocab_size: int,
                 pad_seqs: int | None = None, fixed_pages: list | None = None):
        order = order_entries(entries)
        self.sorted_entries = [entries[i] for i in order]
        real = len(self.sorted_entries)
        q_lens = [len(e.tokens) for e in self.sorted_entries]
        ctx_lens = [e.start + len(e.tokens) for e in self.sorted_entries]
        self.num_real_seqs = real
        self.num_decode = sum(1 for q in q_lens if q == 1)
        self.num_fed = 0
        for e in self.sorted_entries:
            if e.feed_row >= 0:
                if len(e.tokens) != 1:
                    raise ValueError(f"request {e.req_id!r}: only a single token can be fed on the device")
                self.num_fed += 1
        if pad_seqs is not None:
            # fixed-shape batch of single tokens: padding rows have position -1 and length 0
            if self.num_decode != real or real > pad_seqs:
                raise ValueError("a padded batch holds single-token entries only, at most pad_seqs")
            q_lens = q_lens + [1] * (pad_seqs - real)
            ctx_lens = ctx_lens + [0] * (pad_seqs - real)
        self.q_lens, self.ctx_lens = q_lens, ctx_lens
        S = len(q_lens)
        self.S, self.T = S, sum(q_lens)
        self.q_start = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(q_lens, out=self.q_start[1:])
        first_row = {id(e): int(self.q_start[s]) for s, e in enumerate(self.sorted_entries)}
        self.rows, self.row_offsets = [], []
        for e in entries:
            self.row_offsets.append(len(self.rows))
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"request {e.req_id!r}: wanted place {w} outside its "
                                     f"{len(e.tokens)} tokens")
                self.rows.append(first_row[id(e)] + w)
        if pad_seqs is not None:
            self.rows = list(range(S))  # every row, real ones first
        self.cache = cache
        self.vocab_size = vocab_size
        ng = len(cache.groups)
        if fixed_pages is not None:
            self.pages_per_group = list(fixed_pages)
        else:
            self.pages_per_group = [
                max([len(cache.block_table(e.req_id, g)) for e in self.sorted_entries] + [1])
                for g in range(ng)]
        self.tile_lists = {}
        for tpt in tile_tokens:
            ts, t0 = [], []
            for s, q in enumerate(q_lens):
                for a in range(0, q, tpt):
                    ts.append(s)
                    t0.append(a)
            self.tile_lists[tpt] = (ts, t0)
        self.layout, self.total = plan_layout(self.T, S, len(self.rows), self.pages_per_group,
                                              {t: len(v[0]) for t, v in self.tile_lists.items()})

    def fill(self, buf: np.ndarray) -> None:
        layout, cache = self.layout, self.cache

        def view(name):
            o, n = layout[name]
            return buf[o:o + n]

        tok, pos, sot = view("token_ids"), view("positions"), view("seq_of_token")
        tok[:] = 0
        pos[:] = -1
        sot[:] = np.repeat(np.arange(self.S), self.q_lens)
        for s, e in enumerate(self.sorted_entries):
            a, b = int(self.q_start[s]), int(self.q_start[s + 1])
            tok[a:b] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:b] = np.arange(e.start, e.start + (b - a))
        if self.T and (int(tok.min()) < 0 or int(tok.max()) >= self.vocab_size):
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        view("q_start")[:] = self.q_start
        view("ctx_len")[:] = self.ctx_lens
        slots = view("state_slot")
        slots[:] = 0
        slots[:self.num_real_seqs] = [cache.state_slot(e.req_id) for e in self.sorted_entries]
        view("logit_rows")[:] = self.rows
        feed = view("feed_src")
        feed[:] = -1
        if self.num_fed:
            # single-token entries come first: the flat row of sequence s is s
            feed[:self.num_real_seqs] = [e.feed_row if len(e.tokens) == 1 else -1 for e in self.sorted_entries]
        for g, mp in enumerate(self.pages_per_group):
            pt = view(f"page_table{g}").reshape(self.S, mp)
            pt[:] = -1
            for s, e in enumerate(self.sorted_entries):
                table = cache.block_table(e.req_id, g)
                if len(table) > mp:
                    raise ValueError(f"request {e.req_id!r} holds {len(table)} pages, the batch has "
                                     f"room for {mp}")
                pt[s, :len(table)] = table
        for tpt, (ts, t0) in self.tile_lists.items():
            view(f"tile_seq{tpt}")[:] = ts
            view(f"tile_tok0{tpt}")[:] = t0

    def context(self, dev: torch.Tensor, storage, states, dtype, device) -> "StepContext":
        layout = self.layout

        def dview(name):
            o, n = layout[name]
            return dev[o:o + n]

        ctx = StepContext()
        ctx.dtype, ctx.device = dtype, device
        ctx.num_tokens, ctx.num_seqs = self.T, self.S
        ctx.num_decode_seqs = self.S if len(self.q_lens) > self.num_real_seqs else self.num_decode
        ctx.token_ids, ctx.positions = dview("token_ids"), dview("positions")
        ctx.seq_of_token = dview("seq_of_token")
        ctx.q_start, ctx.ctx_len, ctx.state_slot = dview("q_start"), dview("ctx_len"), dview("state_slot")
        ctx.logit_rows = dview("logit_rows")
        ctx.feed_src = dview("feed_src")
        ctx.logit_rows_are_all = self.rows == list(range(self.T))
        ctx.page_tables = [dview(f"page_table{g}").view(self.S, mp)
                           for g, mp in enumerate(self.pages_per_group)]
        ctx.host_q_len, ctx.host_ctx_len = self.q_lens, self.ctx_lens
        ctx.host_q_start = [int(v) for v in self.q_start]
        ctx.host_state_slot = [self.cache.state_slot(e.req_id) for e in self.sorted_entries]
        ctx.max_ctx_len = max(self.ctx_lens) if self.ctx_lens else 0
        for tpt, (ts, _) in self.tile_lists.items():
            ctx.attention_tiles[tpt] = (dview(f"tile_seq{tpt}"), dview(f"tile_tok0{tpt}"), len(ts))
        ctx.storage, ctx.states = storage, states
        ctx.cache_groups, ctx.page_size = self.cache.groups, self.cache.page_size
        return ctx


def build_context(entries: list, cache, storage, states, staging: HostStaging, dtype, device,
                  tile_tokens: list, vocab_size: int) -> tuple[StepContext, list]:
    """Returns the context and, for each original entry, the index of its first wanted row in
    the logits the step returns (logit rows follow the original order of entries and wants)."""
    plan = StepPlanLayout(entries, cache, tile_tokens, vocab_size)
    dev = staging.upload(plan.total, plan.fill)
    ctx = plan.context(dev, storage, states, dtype, device)
    ctx.num_fed = plan.num_fed
    return ctx, plan.row_offsets
