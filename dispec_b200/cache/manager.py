"""The cache manager: pages per group of layers, a block table per request and group, and
slots for fixed-size per-request state.  Pure bookkeeping, no tensors.

Layers whose mixers need the same kind of cache form a group with a page pool of its own:
full attention keeps every page of a live request; a window group gives a page back as soon
as every position in it lies more than ``window`` behind the request's stored length, and
hands it out again.  Block tables are indexed by logical page (position // page_size);
a page given back leaves -1 behind, which the kernels never index.

Reference: puneethgv/DiSpec dispec/kv/block_manager.py (one group, tables at :22-31, allocate
:66-86, append_token :98-106, free :143-152).  Differences: several groups, window release,
reservations made at admission (a request admitted by the scheduler can always finish its
prompt), state slots.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from dispec_b200.cache.pages import OutOfPagesError, PagePool


class OutOfSlotsError(RuntimeError):
    """Every per-request state slot is taken."""


@dataclass(frozen=True)
class CacheTensor:
    """One named tensor a mixer keeps per token: ``num_heads`` rows of ``width`` elements."""
    name: str
    num_heads: int
    width: int


def key_value_tensors(num_kv_heads: int, head_dim: int) -> tuple:
    """The two tensors of ordinary attention: a key and a value of equal shape."""
    return (CacheTensor("key", num_kv_heads, head_dim), CacheTensor("value", num_kv_heads, head_dim))


@dataclass(frozen=True)
class CacheGroupSpec:
    """One group of layer caches with identical needs: the tensors every token leaves in a
    layer cache (each with its own heads and width), the window, and how many layer caches."""
    tensors: tuple  # of CacheTensor
    window: int = 0  # 0: all tokens stay
    num_slots: int = 1  # layer caches in the group

    @classmethod
    def key_value(cls, num_kv_heads: int, head_dim: int, window: int = 0, num_slots: int = 1):
        return cls(key_value_tensors(num_kv_heads, head_dim), window, num_slots)

    def page_elements(self, page_size: int) -> int:
        """Elements of one page across the group's layer caches and tensors."""
        return self.num_slots * page_size * sum(t.num_heads * t.width for t in self.tensors)


@dataclass
class _Request:
    state_slot: int
    num_tokens: int = 0  # tokens whose keys/values are stored
    tables: list[list[int]] = field(default_factory=list)  # per group, logical page -> page id | -1
    first_live: list[int] = field(default_factory=list)  # per group, first logical page still held
    reserved: list[int] = field(default_factory=list)  # per group, pages still promised
    renew: list[bool] = field(default_factory=list)  # per group: a released page renews the promise


class CacheManager:
    def __init__(self, groups: list[CacheGroupSpec], page_size: int, num_pages, max_num_seqs: int):
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.groups = list(groups)
        self.page_size = page_size
        counts = [num_pages] * len(groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(groups):
            raise ValueError("one page count per cache group is needed")
        self.pools = [PagePool(n) for n in counts]
        self.max_num_seqs = max_num_seqs
        self._free_slots = list(range(max_num_seqs - 1, -1, -1))
        self._requests: dict = {}

    # ------------------------------------------------------------------ introspection
    def pages_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def has(self, req_id) -> bool:
        return req_id in self._requests

    def live_requests(self) -> list:
        return list(self._requests)

    def num_tokens(self, req_id) -> int:
        return self._requests[req_id].num_tokens

    def state_slot(self, req_id) -> int:
        return self._requests[req_id].state_slot

    def block_table(self, req_id, group: int = 0) -> list[int]:
        return self._requests[req_id].tables[group]

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def num_available_pages(self, group: int = 0) -> int:
        return self.pools[group].available

    def min_free_pages(self) -> int:
        """Pages no request holds or has reserved, in the group that has the fewest."""
        return min(pool.available for pool in self.pools)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def capacity_tokens(self) -> int:
        """Longest single request the pools can ever hold."""
        cap = None
        for spec, pool in zip(self.groups, self.pools):
            if spec.window == 0:
                c = pool.num_pages * self.page_size
                cap = c if cap is None else min(cap, c)
        return cap if cap is not None else 1 << 62

    def window_quota(self, group: int, max_total_len: int, max_chunk: int) -> int:
        """Most pages a request ever holds at once in a window group: a step of ``max_chunk``
        tokens needs the window - 1 positions before it and its own, which touch at most one page
        more than they fill; never more than the pages of the ``max_total_len`` positions the
        request ever stores."""
        w = self.groups[group].window
        bound = (w - 1 + max(1, max_chunk) + self.page_size - 1) // self.page_size + 1
        return min(bound, self.pages_for(max_total_len))

    def largest_chunk(self) -> int:
        """The largest portion of a prompt that one step may bring so that every window group's
        quota (``window_quota``) still fits its pool; unbounded without window groups."""
        cap = 1 << 62
        for spec, pool in zip(self.groups, self.pools):
            if spec.window > 0:
                cap = min(cap, (pool.num_pages - 1) * self.page_size - spec.window + 1)
        return cap

    # ---------------------------------------------------------------------- lifecycle
    def admission_need(self, prompt_len: int, max_total_len: int, max_chunk: int) -> list[int]:
        need = []
        for g, spec in enumerate(self.groups):
            if spec.window == 0:
                need.append(self.pages_for(prompt_len))
            else:
                need.append(self.window_quota(g, max_total_len, max_chunk))
        return need

    def can_admit(self, prompt_len: int, max_total_len: int, max_chunk: int) -> bool:
        if not self._free_slots:
            return False
        need = self.admission_need(prompt_len, max_total_len, max_chunk)
        return all(pool.available >= n for pool, n in zip(self.pools, need))

    def admit(self, req_id, prompt_len: int = 0, max_total_len: int = 0, max_chunk: int = 1) -> int:
        """Registers a request, takes a state slot and reserves the pages its prompt needs
        (prompt_len == 0: no promise, pages are taken as they come).  Returns the state slot."""
        if req_id in self._requests:
            raise ValueError(f"request {req_id!r} is already live")
        if not self._free_slots:
            raise OutOfSlotsError(f"all {self.max_num_seqs} request slots are taken")
        need = ([0] * len(self.groups) if prompt_len <= 0
                else self.admission_need(prompt_len, max(max_total_len, prompt_len), max_chunk))
        for pool, n in zip(self.pools, need):
            if pool.available < n:
                raise OutOfPagesError(f"admission needs {n} pages, {pool.available} available")
        for pool, n in zip(self.pools, need):
            pool.reserve(n)
        slot = self._free_slots.pop()
        ng = len(self.groups)
        self._requests[req_id] = _Request(
            state_slot=slot, tables=[[] for _ in range(ng)], first_live=[0] * ng, reserved=need,
            renew=[spec.window > 0 and prompt_len > 0 for spec in self.groups])
        return slot

    def pages_missing(self, req_id, new_total: int) -> list[int]:
        r = self._requests[req_id]
        want = self.pages_for(new_total)
        return [max(0, want - len(t)) for t in r.tables]

    def can_extend(self, req_id, new_total: int) -> bool:
        r = self._requests[req_id]
        for g, miss in enumerate(self.pages_missing(req_id, new_total)):
            if miss > r.reserved[g] + self.pools[g].available:
                return False
        return True

    def extend(self, req_id, new_total: int) -> None:
        """Makes room for positions up to new_total - 1 in every group, or takes nothing and
        raises OutOfPagesError."""
        if not self.can_extend(req_id, new_total):
            raise OutOfPagesError(f"request {req_id!r} cannot grow to {new_total} tokens")
        r = self._requests[req_id]
        for g, miss in enumerate(self.pages_missing(req_id, new_total)):
            for _ in range(miss):
                if r.reserved[g] > 0:
                    r.reserved[g] -= 1
                    page = self.pools[g].alloc(from_reservation=True)
                else:
                    page = self.pools[g].alloc()
                r.tables[g].append(page)

    def commit(self, req_id, num_tokens: int) -> list[tuple[int, int]]:
        """Records that ``num_tokens`` tokens are stored and gives back the pages every window
        has passed.  Returns the (group, page) pairs given back."""
        r = self._requests[req_id]
        if num_tokens < r.num_tokens:
            raise ValueError("stored length cannot shrink")
        for g, t in enumerate(r.tables):
            if num_tokens > len(t) * self.page_size:
                raise RuntimeError(f"request {req_id!r}: {num_tokens} tokens exceed its pages in group {g}")
        r.num_tokens = num_tokens
        released = []
        for g, spec in enumerate(self.groups):
            if spec.window <= 0:
                continue
            # the next query sits at position >= num_tokens and sees keys >= num_tokens - window + 1
            first_needed = max(0, num_tokens - spec.window + 1)
            keep_from = first_needed // self.page_size
            table = r.tables[g]
            while r.first_live[g] < min(keep_from, len(table)):
                j = r.first_live[g]
                page = table[j]
                table[j] = -1
                self.pools[g].release(page)
                if r.renew[g]:
                    self.pools[g].reserve(1)
                    r.reserved[g] += 1
                released.append((g, page))
                r.first_live[g] += 1
        return released

    def free(self, req_id) -> list[tuple[int, int]]:
        """Ends a request: every page, promise and its state slot go back."""
        r = self._requests.pop(req_id, None)
        if r is None:
            return []
        released = []
        for g, table in enumerate(r.tables):
            for page in table:
                if page >= 0:
                    self.pools[g].release(page)
                    released.append((g, page))
            if r.reserved[g]:
                self.pools[g].unreserve(r.reserved[g])
        self._free_slots.append(r.state_slot)
        return released

    # --------------------------------------------------------------------- invariants
    def check(self) -> None:
        """No page lost, held twice or free while held; promises add up; slots unique."""
        for g, pool in enumerate(self.pools):
            held = []
            promised = 0
            for r in self._requests.values():
                held += [p for p in r.tables[g] if p >= 0]
                promised += r.reserved[g]
            assert len(held) == len(set(held)), f"group {g}: a page is held twice"
            free = set(pool._free)
            assert len(free) == len(pool._free), f"group {g}: a page is on the free list twice"
            assert not (free & set(held)), f"group {g}: a held page is on the free list"
            assert len(free) + len(held) == pool.num_pages, f"group {g}: a page is lost"
            assert promised == pool.reserved, f"group {g}: promises {promised} != {pool.reserved}"
            assert pool.reserved <= len(free), f"group {g}: more promised than free"
            for p in held:
                assert pool.ref_count(p) == 1
        slots = [r.state_slot for r in self._requests.values()]
        assert len(slots) == len(set(slots)) and not (set(slots) & set(self._free_slots))
        assert len(slots) + len(self._free_slots) == self.max_num_seqs
