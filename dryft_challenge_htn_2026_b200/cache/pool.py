"""Host-side bookkeeping of the cache: a pool of pages and a table of sequence slots.

Pure Python, no device: it decides which page and which slot a sequence gets, and checks that
nothing is handed out twice, freed twice or lost."""


class CacheFull(RuntimeError):
    """No free page or slot: more tokens or sequences are live than the cache was sized for."""


class PagePool:
    def __init__(self, num_pages):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # pop() hands out low pages first
        self._used = [False] * num_pages

    @property
    def n_free(self):
        return len(self._free)

    def alloc(self, n):
        if n > len(self._free):
            raise CacheFull(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            assert not self._used[p], f"page {p} handed out twice"
            self._used[p] = True
        return pages

    def free(self, pages):
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._used[p]:
                raise ValueError(f"page {p} freed but not in use")
            self._used[p] = False
            self._free.append(p)


class SlotTable:
    """Slots 0..max_slots-1, one per live sequence; freed slots are reused lowest first."""

    def __init__(self, max_slots):
        self.max_slots = max_slots
        self._free = list(range(max_slots - 1, -1, -1))
        self._live = set()

    @property
    def n_live(self):
        return len(self._live)

    def acquire(self):
        if not self._free:
            raise CacheFull(f"all {self.max_slots} sequence slots are in use")
        s = self._free.pop()
        assert s not in self._live
        self._live.add(s)
        return s

    def release(self, slot):
        if slot not in self._live:
            raise ValueError(f"slot {slot} released but not live")
        self._live.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    def is_live(self, slot):
        return slot in self._live
