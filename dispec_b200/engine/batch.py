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


@dataclass
class LayerCacheView:
    key_pool: torch.Tensor  # [num_pages, KVH, page_size, D]
    value_pool: torch.Tensor
    page_table: torch.Tensor  # [S, max_pages] int32, -1 where a page was given back
    group: int
    write: bool
    page_size: int
    num_pages: int
    window: int


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
        self.graph_capture = False  # host-side choices must not depend on the step's values
        self.scratch: dict = {}

    def cache_view(self, placement, write: bool) -> LayerCacheView:
        g = placement.group
        pool = self.storage.pools[g]
        return LayerCacheView(pool[placement.slot, 0], pool[placement.slot, 1], self.page_tables[g],
                              g, write, self.page_size, pool.shape[2], self.cache_groups[g].window)

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
        self._grow(capacity)

    def _grow(self, n: int) -> None:
        cap = max(n, self.capacity * 2)
        self._host = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [None, None]
        self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.capacity = cap

    def upload(self, n: int, fill) -> torch.Tensor:
        """``fill(numpy int32 array of length n)`` writes the step's integers; returns the
        device copy (valid until the next upload)."""
        if n > self.capacity:
            self._grow(n)
        self._turn ^= 1
        ev = self._events[self._turn]
        if ev is not None:
            ev.synchronize()
        host = self._host[self._turn]
        fill(host.numpy()[:n])
        dev = self._dev[:n]
        dev.copy_(host[:n], non_blocking=True)
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
    for g, mp in enumerate(pages_per_group):
        put(f"page_table{g}", S * mp)
    for tpt, nt in tiles.items():
        put(f"tile_seq{tpt}", nt)
        put(f"tile_tok0{tpt}", nt)
    return layout, off


def build_context(entries: list, cache, storage, states, staging: HostStaging, dtype, device,
                  tile_tokens: list, vocab_size: int) -> tuple[StepContext, list]:
    """Returns the context and, for each original entry, the index of its first wanted row in
    the logits the step returns (logit rows follow the original order of entries and wants)."""
    order = order_entries(entries)
    sorted_entries = [entries[i] for i in order]
    S = len(sorted_entries)
    q_lens = [len(e.tokens) for e in sorted_entries]
    T = sum(q_lens)
    ctx_lens = [e.start + len(e.tokens) for e in sorted_entries]
    n_decode = sum(1 for q in q_lens if q == 1)
    q_start = np.zeros(S + 1, dtype=np.int64)
    np.cumsum(q_lens, out=q_start[1:])

    # logit rows in the original order of the entries
    first_row = {}
    for s, e in enumerate(sorted_entries):
        first_row[id(e)] = int(q_start[s])
    rows = []
    row_offsets = []
    for e in entries:
        row_offsets.append(len(rows))
        for w in e.want:
            if not 0 <= w < len(e.tokens):
                raise ValueError(f"request {e.req_id!r}: wanted place {w} outside its {len(e.tokens)} tokens")
            rows.append(first_row[id(e)] + w)

    ng = len(cache.groups)
    pages_per_group = []
    for g in range(ng):
        mp = max(len(cache.block_table(e.req_id, g)) for e in sorted_entries)
        pages_per_group.append(max(mp, 1))
    tiles = {}
    tile_lists = {}
    for tpt in tile_tokens:
        ts, t0 = [], []
        for s, q in enumerate(q_lens):
            for a in range(0, q, tpt):
                ts.append(s)
                t0.append(a)
        tile_lists[tpt] = (ts, t0)
        tiles[tpt] = len(ts)
    layout, total = plan_layout(T, S, len(rows), pages_per_group, tiles)

    def fill(buf: np.ndarray) -> None:
        def view(name):
            o, n = layout[name]
            return buf[o:o + n]

        tok = view("token_ids")
        pos = view("positions")
        sot = view("seq_of_token")
        for s, e in enumerate(sorted_entries):
            a, b = int(q_start[s]), int(q_start[s + 1])
            tok[a:b] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:b] = np.arange(e.start, e.start + (b - a))
            sot[a:b] = s
        if T and (int(tok.min()) < 0 or int(tok.max()) >= vocab_size):
            raise ValueError(f"token id outside [0, {vocab_size})")
        view("q_start")[:] = q_start
        view("ctx_len")[:] = ctx_lens
        view("state_slot")[:] = [cache.state_slot(e.req_id) for e in sorted_entries]
        view("logit_rows")[:] = rows
        for g in range(ng):
            mp = pages_per_group[g]
            pt = view(f"page_table{g}").reshape(S, mp)
            pt[:] = -1
            for s, e in enumerate(sorted_entries):
                table = cache.block_table(e.req_id, g)
                pt[s, :len(table)] = table
        for tpt, (ts, t0) in tile_lists.items():
            view(f"tile_seq{tpt}")[:] = ts
            view(f"tile_tok0{tpt}")[:] = t0

    dev = staging.upload(total, fill)

    def dview(name):
        o, n = layout[name]
        return dev[o:o + n]

    ctx = StepContext()
    ctx.dtype, ctx.device = dtype, device
    ctx.num_tokens, ctx.num_seqs, ctx.num_decode_seqs = T, S, n_decode
    ctx.token_ids, ctx.positions, ctx.seq_of_token = dview("token_ids"), dview("positions"), dview("seq_of_token")
    ctx.q_start, ctx.ctx_len, ctx.state_slot = dview("q_start"), dview("ctx_len"), dview("state_slot")
    ctx.logit_rows = dview("logit_rows")
    ctx.page_tables = [dview(f"page_table{g}").view(S, pages_per_group[g]) for g in range(ng)]
    ctx.host_q_len, ctx.host_ctx_len = q_lens, ctx_lens
    ctx.host_q_start = [int(v) for v in q_start]
    ctx.host_state_slot = [cache.state_slot(e.req_id) for e in sorted_entries]
    ctx.max_ctx_len = max(ctx_lens) if ctx_lens else 0
    for tpt in tile_tokens:
        ctx.attention_tiles[tpt] = (dview(f"tile_seq{tpt}"), dview(f"tile_tok0{tpt}"), tiles[tpt])
    ctx.storage, ctx.states = storage, states
    ctx.cache_groups, ctx.page_size = cache.groups, cache.page_size
    return ctx, row_offsets
