"""The cache manager: memory for what requests keep between steps.

Two kinds of memory, both sized once at start:

* **Pages** for mixers that keep keys and values per position.  Entries of the
  model's order with the same retention rule form a *group* (all keys; the
  last ``window`` keys).  A group has a pool of page ids of its own and every
  request has one block table per group; a page id addresses the same page in
  the key and value tensors of every entry of the group
  (``[n_pages, kv_heads, page_size, head_dim]`` each).  Pages are taken as a
  request grows, given back when it ends, and in a windowed group also as
  soon as the window has passed them; the ids are then reused by whoever asks
  next.
* **Slots** for per-request state of fixed size (a short convolution's last
  inputs, a recurrent state).  One slot holds the state of every entry that
  needs some, as byte ranges of one row; a slot is zeroed when a request
  takes it.

The manager is plain host code apart from the tensors it allocates, so its
bookkeeping runs (and is tested) without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parts.base import PagedKV, SlotState
from .pools import IdPool, PoolError


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


@dataclass
class PagedKVView:
    """What a mixer sees of its paged cache during one step."""
    k_pages: torch.Tensor
    v_pages: torch.Tensor
    block_table: torch.Tensor          # int32 [requests in the step, max_blocks]
    page_size: int
    writable: bool
    window: Optional[int]


@dataclass
class SlotView:
    state: torch.Tensor                # [n_slots, *shape]; the slot axis is strided
    slot_ids: torch.Tensor             # int32 [requests in the step]
    host_slot_ids: list


@dataclass
class _Group:
    window: Optional[int]
    pool: IdPool
    entries: list = field(default_factory=list)     # (entry index, need index)


@dataclass
class RequestCache:
    """What one live request holds."""
    request_id: object
    slot: Optional[int]
    block_tables: list                 # per group: list of page ids, -1 where a page was given back
    length: int = 0                    # positions written so far


class CacheManager:
    GUARD_BYTE = 0x5A

    def __init__(self, entry_needs, n_pages, page_size: int, n_slots: int, dtype: torch.dtype, device,
                 max_context: int, guard: bool = False):
        """entry_needs: for each entry of the model's order, (list of needs,
        entry whose cache it reads instead or None).  n_pages: an int (for
        every group) or a dict from window (None = all keys) to a count.
        ``guard``: one page before and after every page tensor, one slot row
        before and after the slots and 16 bytes behind every slot are filled
        with a pattern that ``check`` looks at: a kernel that writes outside
        the page or slot it was given is then found where it happened."""
        if page_size <= 0:
            raise ValueError(f"page_size {page_size}")
        self.page_size, self.n_slots, self.dtype = page_size, n_slots, dtype
        self.device = torch.device(device)
        self.max_context = max_context
        self.max_blocks = -(-max_context // page_size)
        self.entry_needs = entry_needs
        self.guard = bool(guard)
        self._guards: list[torch.Tensor] = []
        self.groups: list[_Group] = []
        self._group_of: dict[tuple[int, int], int] = {}
        self._pages: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
        self._slot_ranges: dict[tuple[int, int], tuple[int, int, SlotState]] = {}
        slot_bytes = 0
        by_window: dict[Optional[int], int] = {}
        for e, (needs, reads) in enumerate(entry_needs):
            if reads is not None:
                continue
            for k, need in enumerate(needs):
                if isinstance(need, PagedKV):
                    if need.window not in by_window:
                        count = n_pages[need.window] if isinstance(n_pages, dict) else n_pages
                        by_window[need.window] = len(self.groups)
                        self.groups.append(_Group(need.window, IdPool(count, "page")))
                    g = by_window[need.window]
                    self.groups[g].entries.append((e, k))
                    self._group_of[(e, k)] = g
                    shape = (self.groups[g].pool.size, need.kv_heads, page_size)
                    self._pages[(e, k)] = (self._page_tensor(shape + (need.head_dim,), dtype),
                                           self._page_tensor(shape + (need.value_dim,), dtype))
                elif isinstance(need, SlotState):
                    nbytes = int(torch.tensor([], dtype=need.dtype).element_size())
                    for s in need.shape:
                        nbytes *= int(s)
                    start = -(-slot_bytes // 16) * 16
                    self._slot_ranges[(e, k)] = (start, nbytes, need)
                    slot_bytes = start + nbytes
                else:
                    raise TypeError(f"entry {e} asks for a cache of unknown kind {need!r}")
        self.slot_bytes = -(-slot_bytes // 16) * 16
        self.slots = IdPool(n_slots if self.slot_bytes else 0, "slot")
        self._slot_mem = None
        if self.slot_bytes and not self.guard:
            self._slot_mem = torch.zeros((n_slots, self.slot_bytes), dtype=torch.uint8, device=self.device)
        elif self.slot_bytes:
            whole = torch.full((n_slots + 2, self.slot_bytes + 16), self.GUARD_BYTE, dtype=torch.uint8, device=self.device)
            self._slot_mem = whole[1:-1, :self.slot_bytes]
            self._slot_mem.zero_()
            self._guards += [whole[0], whole[-1], whole[1:-1, self.slot_bytes:]]
        self._slot_views: dict[tuple[int, int], torch.Tensor] = {}
        for key, (start, nbytes, need) in self._slot_ranges.items():
            flat = self._slot_mem[:, start:start + nbytes].view(need.dtype)
            self._slot_views[key] = flat.unflatten(1, tuple(need.shape))
        self.live: dict[object, RequestCache] = {}

    def _page_tensor(self, shape, dtype) -> torch.Tensor:
        """A zeroed page tensor; with guards, the inner pages of a tensor that is two pages longer."""
        if not self.guard:
            return torch.zeros(shape, dtype=dtype, device=self.device)
        whole = torch.zeros((shape[0] + 2,) + tuple(shape[1:]), dtype=dtype, device=self.device)
        for edge in (whole[0], whole[-1]):
            edge.view(torch.uint8).fill_(self.GUARD_BYTE)
            self._guards.append(edge.view(torch.uint8))
        return whole[1:-1]

    def check_guards(self) -> None:
        """Raise if anything wrote into the guard pages, guard slots or the bytes behind a slot."""
        for i, g in enumerate(self._guards):
            if not bool((g == self.GUARD_BYTE).all()):
                bad = int((g != self.GUARD_BYTE).sum())
                raise PoolError(f"guard region {i} of the cache was written to ({bad} bytes changed): a kernel wrote "
                                "outside the page or slot it was given")

    # -- sizes ---------------------------------------------------------------
    def kv_bytes_per_token(self) -> int:
        total = 0
        for (e, k), (kp, vp) in self._pages.items():
            total += kp.shape[1] * (kp.shape[3] + vp.shape[3]) * kp.element_size()
        return total

    def pages_needed(self, length: int) -> int:
        return -(-length // self.page_size)

    def free_pages(self) -> list[int]:
        return [g.pool.n_free for g in self.groups]

    # -- request life --------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise PoolError(f"request {request_id!r} is already live")
        slot = None
        if self.slot_bytes:
            slot = self.slots.take()
            if slot is None:
                raise OutOfSlots(f"all {self.n_slots} state slots are in use")
            self._slot_mem[slot].zero_()
        rc = RequestCache(request_id, slot, [[] for _ in self.groups])
        self.live[request_id] = rc
        return rc

    def _first_needed_page(self, group: _Group, start_pos: int) -> int:
        """Index (in the block table) of the first page a step that starts at
        start_pos can still read."""
        if group.window is None:
            return 0
        return max(0, start_pos - group.window + 1) // self.page_size

    def pages_wanted(self, wants) -> list[int]:
        """Pages each group's pool must still give for ``wants``, a list of
        (request cache, new length), once every request of the list has given
        back the pages its window has passed."""
        need = [0] * len(self.groups)
        for rc, new_length in wants:
            for g, group in enumerate(self.groups):
                table = rc.block_tables[g]
                first = self._first_needed_page(group, rc.length)
                freed = sum(1 for p in table[:first] if p >= 0)
                need[g] += max(self.pages_needed(new_length) - len(table), 0) - freed
        return need

    def can_reserve_all(self, wants) -> bool:
        return all(n <= g.pool.n_free for n, g in zip(self.pages_wanted(wants), self.groups))

    def can_reserve(self, rc: RequestCache, new_length: int) -> bool:
        return self.can_reserve_all([(rc, new_length)])

    def reserve_all(self, wants) -> None:
        """Make room for positions rc.length .. new_length-1 of every (request
        cache, new length) of ``wants`` in every group, all or nothing: first
        EVERY request gives back the pages its window has passed, then the new
        pages are taken, so that one request's returns cover another's needs
        whatever their order.  Takes nothing and raises OutOfPages when a pool
        cannot cover the whole list."""
        for rc, new_length in wants:
            if new_length > self.max_context:
                raise ValueError(f"request {rc.request_id!r} would reach {new_length} positions; "
                                 f"the cache is laid out for {self.max_context}")
        if not self.can_reserve_all(wants):
            raise OutOfPages(f"requests {[rc.request_id for rc, _ in wants]!r} need {self.pages_wanted(wants)} more "
                             f"pages per group; free: {self.free_pages()}")
        for rc, _ in wants:
            for g, group in enumerate(self.groups):
                table = rc.block_tables[g]
                first = self._first_needed_page(group, rc.length)
                for i in range(min(first, len(table))):
                    if table[i] >= 0:
                        group.pool.give_back(table[i])
                        table[i] = -1
        for rc, new_length in wants:
            for g, group in enumerate(self.groups):
                table = rc.block_tables[g]
                while len(table) < self.pages_needed(new_length):
                    table.append(group.pool.take())

    def reserve(self, rc: RequestCache, new_length: int) -> None:
        """``reserve_all`` for one request."""
        self.reserve_all([(rc, new_length)])

    def unreserve(self, rc: RequestCache) -> None:
        """Give back the pages beyond the request's written length: what a
        ``reserve`` took for a step that then did not run.  (Pages a window had
        passed stay given back; no later step reads them.)"""
        keep = self.pages_needed(rc.length)
        for g, group in enumerate(self.groups):
            table = rc.block_tables[g]
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    group.pool.give_back(p)

    def advance(self, rc: RequestCache, new_length: int) -> None:
        """Record that positions up to new_length-1 are written."""
        if new_length < rc.length:
            raise ValueError("a request's cache cannot shrink")
        rc.length = new_length

    def close(self, request_id) -> None:
        """Give back everything the request holds."""
        rc = self.live.pop(request_id, None)
        if rc is None:
            raise PoolError(f"request {request_id!r} is not live (closed twice?)")
        for g, group in enumerate(self.groups):
            for p in rc.block_tables[g]:
                if p >= 0:
                    group.pool.give_back(p)
            rc.block_tables[g] = []
        if rc.slot is not None:
            self.slots.give_back(rc.slot)
            rc.slot = None

    def check(self) -> None:
        """Invariants: no page or slot lost, none held twice."""
        for g, group in enumerate(self.groups):
            group.pool.check()
            held = [p for rc in self.live.values() for p in rc.block_tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise PoolError(f"a page of group {g} is held twice")
            if len(held) != group.pool.n_used:
                raise PoolError(f"group {g}: {group.pool.n_used} pages are out but requests hold {len(held)}")
        self.slots.check()
        held = [rc.slot for rc in self.live.values() if rc.slot is not None]
        if len(held) != len(set(held)) or len(held) != self.slots.n_used:
            raise PoolError("slots held by requests and slots out of the pool differ")
        if self.guard:
            self.check_guards()

    # -- views for one step --------------------------------------------------
    def fill_block_tables(self, rcs: list, out) -> None:
        """Write the block tables of the step's requests into ``out``, an int32
        numpy array [n_groups, len(rcs), max_blocks] (-1 where there is no page)."""
        out[:, :len(rcs), :] = -1
        for g in range(len(self.groups)):
            for r, rc in enumerate(rcs):
                t = rc.block_tables[g]
                if t:
                    out[g, r, :len(t)] = t

    def views(self, block_tables: list, slot_ids: torch.Tensor, host_slot_ids: list) -> list:
        """Per entry of the order, the list of views its mixer gets (one per
        need; an entry that reads another entry's cache gets that entry's
        views, read-only).  block_tables: per group a device int32 tensor
        [requests, max_blocks]."""
        out = []
        for e, (needs, reads) in enumerate(self.entry_needs):
            owner = e if reads is None else reads
            views = []
            for k, need in enumerate(self.entry_needs[owner][0]):
                if isinstance(need, PagedKV):
                    kp, vp = self._pages[(owner, k)]
                    g = self._group_of[(owner, k)]
                    views.append(PagedKVView(kp, vp, block_tables[g], self.page_size, reads is None, need.window))
                else:
                    views.append(SlotView(self._slot_views[(owner, k)], slot_ids, host_slot_ids))
            out.append(views)
        return out
