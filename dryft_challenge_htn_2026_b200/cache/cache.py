"""The cache of a model: a slot per live sequence, and per group of layers either paged keys and
values or a fixed-size state.

Layers (cache entries) whose mixers make the same request share a group; each group has storage
and, for keys/values, a page pool of its own, so a group of windowed layers can give pages back
that a group of full-attention layers must keep. A sequence's length is the same in every group.

Key/value storage of a group: [entries, 2 (k, v), pages, n_kv_heads, PAGE, head_dim]; page p of a
kv head is one contiguous [PAGE, head_dim] tile. State storage: [entries, slots, *shape].
The reference keeps one dense [B, nkv, cap, hd] pair per layer per batch shape
(engine/engine.py:344-347); pages let sequences of any lengths share one allocation.
"""
from dataclasses import dataclass

import torch

from ..csrc.api import PAGE
from .pool import CacheFull, PagePool, SlotTable
from .requests import KVRequest, StateRequest


@dataclass
class KVView:
    group: int            # index into StepContext.tables
    k: torch.Tensor       # [pages, n_kv, PAGE, hd]
    v: torch.Tensor


@dataclass
class StateView:
    group: int
    state: torch.Tensor   # [slots, *shape]; row = the sequence's slot (StepContext.seq_slot)


class KVGroup:
    def __init__(self, index, request, entries, num_pages, device, allocate=True):
        self.index, self.request, self.entries = index, request, list(entries)
        self.pool = PagePool(num_pages)
        self.pages = {}                                   # slot -> list of page ids (-1: given back)
        self.first = {}                                   # slot -> index of the first page not yet given back
        self.store = None
        if allocate:
            self.store = torch.zeros((len(self.entries), 2, num_pages, request.n_kv_heads, PAGE, request.head_dim),
                                     dtype=request.dtype, device=device)

    def view(self, entry):
        e = self.entries.index(entry)
        return KVView(self.index, self.store[e, 0], self.store[e, 1])

    def start(self, slot):
        self.pages[slot] = []
        self.first[slot] = 0

    def ensure(self, slot, length):
        """Pages for positions [0, length) of the slot (those still inside the window)."""
        have = self.pages[slot]
        need = (length + PAGE - 1) // PAGE - len(have)
        if need > 0:
            have.extend(self.pool.alloc(need))

    def trim(self, slot, length):
        """Gives back pages no later token can see: a query at position >= length reads keys
        > length - window - 1 only."""
        w = self.request.window
        if w is None:
            return
        first_needed = length - w + 1
        have = self.pages[slot]
        i = self.first[slot]
        while i < len(have) and i * PAGE + PAGE - 1 < first_needed:
            self.pool.free([have[i]])
            have[i] = -1
            i += 1
        self.first[slot] = i

    def end(self, slot):
        self.pool.free([p for p in self.pages.pop(slot) if p >= 0])
        del self.first[slot]

    def bytes(self):
        return 0 if self.store is None else self.store.numel() * self.store.element_size()


class StateGroup:
    def __init__(self, index, request, entries, max_slots, device, allocate=True):
        self.index, self.request, self.entries = index, request, list(entries)
        self.store = None
        if allocate:
            self.store = torch.zeros((len(self.entries), max_slots, *request.shape), dtype=request.dtype, device=device)

    def view(self, entry):
        return StateView(self.index, self.store[self.entries.index(entry)])

    def start(self, slot):
        if self.store is not None:
            self.store[:, slot].zero_()

    def ensure(self, slot, length):
        pass

    def trim(self, slot, length):
        pass

    def end(self, slot):
        pass

    def bytes(self):
        return 0 if self.store is None else self.store.numel() * self.store.element_size()


class Cache:
    """``entry_requests``: for each cache entry (in order) the list of requests of its mixer."""

    def __init__(self, entry_requests, max_tokens, max_slots, device, allocate=True):
        self.num_pages = max(1, (max_tokens + PAGE - 1) // PAGE)
        self.max_slots = max(1, min(max_slots, self.num_pages))
        self.slots = SlotTable(self.max_slots)
        self.length = {}                                   # slot -> tokens cached
        self.groups = []
        self._views = []                                   # per entry: list of views, in request order
        by_request = {}
        for entry, requests in enumerate(entry_requests):
            for r in requests:
                by_request.setdefault(r, []).append(entry)
        for r, entries in by_request.items():
            if isinstance(r, KVRequest):
                g = KVGroup(len(self.groups), r, entries, self.num_pages, device, allocate)
            elif isinstance(r, StateRequest):
                g = StateGroup(len(self.groups), r, entries, self.max_slots, device, allocate)
            else:
                raise TypeError(f"unknown cache request {r!r}")
            self.groups.append(g)
        if allocate:
            index = {g.request: g for g in self.groups}
            self._views = [[index[r].view(entry) for r in requests] for entry, requests in enumerate(entry_requests)]

    def views(self, entry):
        return self._views[entry]

    # -- life of a sequence ------------------------------------------------------------------
    def begin(self):
        slot = self.slots.acquire()
        self.length[slot] = 0
        for g in self.groups:
            g.start(slot)
        return slot

    def reserve(self, slot, n_new):
        """Room for n_new more tokens of the slot in every group (before the step that writes them)."""
        try:
            for g in self.groups:
                g.ensure(slot, self.length[slot] + n_new)
        except CacheFull:
            raise CacheFull(f"cache full: sequence in slot {slot} cannot grow from {self.length[slot]} by {n_new} "
                            f"tokens ({self.num_pages} pages of {PAGE} tokens in all)") from None

    def commit(self, slot, n_new):
        """After the step: the tokens are in; windowed groups give back what fell out of sight."""
        self.length[slot] += n_new
        for g in self.groups:
            g.trim(slot, self.length[slot])

    def end(self, slot):
        if slot not in self.length:
            raise ValueError(f"slot {slot} ended but not live")
        for g in self.groups:
            g.end(slot)
        del self.length[slot]
        self.slots.release(slot)

    def page_rows(self, group, slots, min_width=1):
        """Page lists of the slots in one group, padded with -1 to a common width."""
        g = self.groups[group]
        if not isinstance(g, KVGroup):
            return [[-1] * min_width for _ in slots]
        rows = [g.pages[s] for s in slots]
        width = max([min_width] + [len(r) for r in rows])
        return [r + [-1] * (width - len(r)) for r in rows]

    def pages_held(self, slot):
        """Per key/value group the length of the slot's page list (pages given back included): it
        changes exactly when a step's page tables have to be written anew."""
        return tuple(len(g.pages[slot]) for g in self.groups if isinstance(g, KVGroup))

    def bytes(self):
        return sum(g.bytes() for g in self.groups)

    def pages_free(self):
        return [g.pool.n_free for g in self.groups if isinstance(g, KVGroup)]
