"""The cache's bookkeeping and the generation loop's decisions (no GPU)."""
import random

import numpy as np
import pytest
import torch

from dryft_challenge_htn_2026_b200.cache import Cache, CacheFull, KVRequest, PagePool, SlotTable, StateRequest
from dryft_challenge_htn_2026_b200.engine.batch import build_context
from dryft_challenge_htn_2026_b200.engine.generate import BatchTracker, bucket_rows, plan_batches, run_batch
from dryft_challenge_htn_2026_b200.sampling import SamplingParams, request_seed, seed_words

KV = KVRequest(2, 16, None, torch.float32)
KVW = KVRequest(2, 16, 100, torch.float32)
ST = StateRequest((3, 4), torch.float32)


def test_page_pool_never_loses_or_doubles_a_page():
    pool = PagePool(37)
    rng = random.Random(0)
    held = []
    for _ in range(2000):
        if held and rng.random() < 0.5:
            pool.free(held.pop(rng.randrange(len(held))))
        else:
            n = rng.randint(1, 5)
            if n <= pool.n_free:
                held.append(pool.alloc(n))
            else:
                with pytest.raises(CacheFull):
                    pool.alloc(n)
        flat = [p for h in held for p in h]
        assert len(flat) == len(set(flat)) and len(flat) + pool.n_free == 37
    p = pool.alloc(1)
    pool.free(p)
    with pytest.raises(ValueError):
        pool.free(p)                                         # freed twice
    with pytest.raises(ValueError):
        pool.free([99])


def test_slot_table_reuses_freed_slots():
    t = SlotTable(3)
    a, b, c = t.acquire(), t.acquire(), t.acquire()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheFull):
        t.acquire()
    t.release(b)
    with pytest.raises(ValueError):
        t.release(b)                                         # freed twice
    assert t.acquire() == b and t.n_live == 3


def test_cache_groups_lengths_and_window_pages():
    # entries 0 and 2 keep everything, entry 1 slides and also has a state
    cache = Cache([[KV], [KVW, ST], [KV]], max_tokens=64 * 10, max_slots=4, device="cpu")
    assert len(cache.groups) == 3 and cache.groups[0].entries == [0, 2] and cache.groups[1].entries == [1]
    assert cache.groups[0].store.shape == (2, 2, 10, 2, 64, 16) and cache.groups[2].store.shape == (1, 4, 3, 4)
    assert cache.views(0)[0].k.data_ptr() != cache.views(2)[0].k.data_ptr()
    s = cache.begin()
    cache.reserve(s, 200)
    assert cache.length[s] == 0 and len(cache.groups[0].pages[s]) == 4
    cache.commit(s, 200)
    assert cache.length[s] == 200
    assert cache.groups[0].pages[s].count(-1) == 0
    # the window group gave back the page whose last position (63) < 200 - 100 + 1
    assert cache.groups[1].pages[s][0] == -1 and cache.groups[1].pages[s][1] >= 0
    assert cache.pages_free() == [6, 7]
    s2 = cache.begin()
    with pytest.raises(CacheFull):
        cache.reserve(s2, 64 * 7)
    cache.end(s)
    assert cache.pages_free()[1] == 10
    cache.end(s2)
    assert cache.pages_free() == [10, 10] and cache.slots.n_live == 0
    with pytest.raises(ValueError):
        cache.end(s)


def test_state_is_zero_for_a_reused_slot():
    cache = Cache([[ST]], max_tokens=64 * 4, max_slots=2, device="cpu")
    s = cache.begin()
    cache.views(0)[0].state[s] += 5.0
    cache.end(s)
    s2 = cache.begin()
    assert s2 == s and float(cache.views(0)[0].state[s2].abs().sum()) == 0.0


def test_random_sequence_lifecycles_keep_the_books_straight():
    cache = Cache([[KV], [KVW]], max_tokens=64 * 40, max_slots=8, device="cpu", allocate=False)
    rng = random.Random(1)
    live = {}
    for _ in range(3000):
        r = rng.random()
        if r < 0.2 and len(live) < 8:
            live[cache.begin()] = 0
        elif r < 0.3 and live:
            s = rng.choice(list(live))
            cache.end(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.randint(1, 150)
            try:
                cache.reserve(s, n)
            except CacheFull:
                continue
            cache.commit(s, n)
            live[s] += n
        for s, n in live.items():
            assert cache.length[s] == n
        held = [[p for pages in g.pages.values() for p in pages if p >= 0] for g in cache.groups]
        for g, h in zip(cache.groups, held):
            assert len(h) == len(set(h)) and len(h) + g.pool.n_free == 40
        # the full group holds exactly the pages the lengths need (reservations that failed half-way may hold more)
        assert all(len(cache.groups[0].pages[s]) >= (n + 63) // 64 for s, n in live.items())
    for s in list(live):
        cache.end(s)
    assert cache.pages_free() == [40, 40]


def test_build_context_rows_positions_and_tiles():
    cache = Cache([[KV]], max_tokens=64 * 16, max_slots=8, device="cpu")
    a, b, c = cache.begin(), cache.begin(), cache.begin()
    from dryft_challenge_htn_2026_b200.parts.attention import QueryTiles
    narrow, wide = QueryTiles(64), QueryTiles(128)
    ctx = build_context(cache, [(a, [1] * 5, [4]), (b, [2] * 130, [0, 129]), (c, [3], [0])], torch.device("cpu"),
                        plans=[narrow, wide, QueryTiles(64)])       # parts' planning data: built once per key
    assert (ctx.n_tok, ctx.n_seq, ctx.n_want, ctx.is_decode) == (136, 3, 4, False)
    assert ctx.cu_q.tolist() == [0, 5, 135, 136] and ctx.want_rows.tolist() == [4, 5, 134, 135]
    assert ctx.row_pos[:5].tolist() == [0, 1, 2, 3, 4] and ctx.row_pos[5:135].tolist() == list(range(130))
    assert ctx.row_seq[4:6].tolist() == [0, 1] and ctx.seq_pos0.tolist() == [0, 0, 0]
    assert set(ctx.plans) == {narrow.key, wide.key}
    tiles = ctx.plans[narrow.key]
    assert sorted(map(tuple, tiles.tolist())) == [(0, 0), (1, 0), (1, 64), (1, 128), (2, 0)]
    assert tuple(tiles[0].tolist()) == (1, 128)                  # the tile that sees most keys goes first
    assert sorted(map(tuple, ctx.plans[wide.key].tolist())) == [(0, 0), (1, 0), (1, 128), (2, 0)]
    assert ctx.tables[0].shape == (3, 3) and ctx.tables[0][0].tolist()[1:] == [-1, -1]
    for s, n in ((a, 5), (b, 130), (c, 1)):
        cache.commit(s, n)
    ctx = build_context(cache, [(b, [7], [0]), (a, [8], [0])], torch.device("cpu"), pad_to=4, plans=[narrow])
    assert ctx.plans[narrow.key].numel() == 0                    # a decode step has no query tiles
    assert ctx.is_decode and ctx.n_tok == 4 and ctx.n_seq == 4 and ctx.n_want == 2
    assert ctx.row_pos.tolist() == [130, 5, -1, -1] and ctx.tables[0].shape[0] == 4
    assert ctx.max_position == 130
    with pytest.raises(ValueError):
        build_context(cache, [(a, [], [])], torch.device("cpu"))
    with pytest.raises(ValueError):
        build_context(cache, [(a, [1, 2], [2])], torch.device("cpu"))


# ------------------------------------------------------------------------------- generation loop
class FakePending:
    def __init__(self, toks):
        self.toks = toks

    def wait(self):
        return self.toks


class FakeBackend:
    """Sequence i emits script[i][k] as its k-th token; records what the loop asks for."""

    def __init__(self, script):
        self.script, self.log = script, []

    def start(self, prompts, params, seeds):
        self.rows = [(i, 1) for i in range(len(prompts))]      # (sequence, tokens made after this step)
        self.log.append(("start", len(prompts)))
        return FakePending([self.script[i][0] for i, _ in self.rows])

    def decode(self):
        out = [self.script[i][k] for i, k in self.rows]
        self.rows = [(i, k + 1) for i, k in self.rows]
        self.log.append(("decode", [i for i, _ in self.rows]))
        return FakePending(out)

    def repack(self, rows):
        for i, tok, made in rows:
            assert tok == self.script[i][made - 1]
        self.rows = [(i, made) for i, _, made in rows]
        self.log.append(("repack", [i for i, _, _ in rows]))

    def finish(self):
        self.log.append(("finish",))


def test_loop_runs_to_the_token_limit_without_stops():
    script = [[10 + k for k in range(6)], [20 + k for k in range(6)]]
    be = FakeBackend(script)
    rows = list(run_batch(be, [[1], [2, 3]], SamplingParams(4), [0, 0]))
    assert rows == [[10, 20], [11, 21], [12, 22], [13, 23]]
    assert [l[0] for l in be.log] == ["start", "decode", "decode", "decode", "finish"]


def test_loop_stop_tokens_end_sequences_early_and_repack():
    STOP = 99
    script = [[1, 2, 3, 4, 5, STOP, 7, 7], [3, STOP, 7, 7, 7, 7, 7, 7], [4, 5, 6, 7, 8, 9, 10, 11]]
    be = FakeBackend(script)
    rows = list(run_batch(be, [[0]] * 3, SamplingParams(8, stop_token_ids=(STOP,)), [0] * 3))
    outs = [[r[i] for r in rows if r[i] is not None] for i in range(3)]
    assert outs == [[1, 2, 3, 4, 5, STOP], [3, STOP], [4, 5, 6, 7, 8, 9, 10, 11]]
    assert ("repack", [0, 2]) in be.log and ("repack", [2]) in be.log
    assert be.log[-1] == ("finish",) and len(rows) == 8
    # after sequence 1 ended no later step reports a token for it
    first_none = next(k for k, r in enumerate(rows) if r[1] is None)
    assert all(r[1] is None for r in rows[first_none:])


def test_loop_edge_cases():
    be = FakeBackend([[5]])
    assert list(run_batch(be, [[1]], SamplingParams(0), [0])) == [] and be.log == []
    be = FakeBackend([[5, 6]])
    assert list(run_batch(be, [[1]], SamplingParams(1), [0])) == [[5]]
    assert [l[0] for l in be.log] == ["start", "finish"]             # one token: no decode step at all
    be = FakeBackend([[9, 9], [9, 9]])
    assert list(run_batch(be, [[1], [2]], SamplingParams(5, stop_token_ids=(9,)), [0, 0])) == [[9, 9]]
    gen = run_batch(FakeBackend([[1, 2, 3]]), [[1]], SamplingParams(3), [0])
    next(gen)
    gen.close()                                                      # abandoning the generator still finishes


def test_tracker_and_planning():
    t = BatchTracker(2, 3, (7,))
    assert t.accept([0, 1], [1, 7]) == ([1, 7], [1])
    assert t.accept([0, 1], [2, 5]) == ([2, None], [])
    assert t.accept([0, 1], [3, 5]) == ([3, None], [0]) and t.active([0, 1]) == []
    assert [list(r) for r in plan_batches(10, 4)] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]
    assert plan_batches(0, 4) == [] and [bucket_rows(n) for n in (1, 2, 3, 8, 9, 64)] == [1, 2, 4, 8, 16, 64]
    with pytest.raises(ValueError):
        plan_batches(3, 0)


def test_request_seeds_are_distinct_and_fit_two_words():
    seeds = {request_seed(5, i) for i in range(1000)} | {request_seed(6, i) for i in range(1000)}
    assert len(seeds) == 2000
    lo, hi = seed_words(request_seed(5, 3))
    assert -2**31 <= lo < 2**31 and -2**31 <= hi < 2**31
    assert ((lo & 0xFFFFFFFF) | ((hi & 0xFFFFFFFF) << 32)) == request_seed(5, 3)
    with pytest.raises(ValueError):
        SamplingParams(4, temperature=-1.0)


def test_prefill_plan_groups_whole_sequences_and_chunks_long_ones():
    from dryft_challenge_htn_2026_b200.engine.generate import prefill_plan
    plan = lambda lengths: prefill_plan(lengths, 100)
    assert plan([10, 20, 30]) == [[(0, 0, 10), (1, 0, 20), (2, 0, 30)]]
    assert plan([60, 50, 40, 100]) == [[(0, 0, 60)], [(1, 0, 50), (2, 0, 40)], [(3, 0, 100)]]
    assert plan([30, 250, 5]) == [[(0, 0, 30)], [(1, 0, 100)], [(1, 100, 200)], [(1, 200, 250)], [(2, 0, 5)]]
    for lens in ([1], [100, 100], [101, 99, 1, 300], [7] * 40):
        steps = plan(lens)
        covered = {}
        for step in steps:
            assert sum(p1 - p0 for _, p0, p1 in step) <= 100
            assert [i for i, _, _ in step] == sorted(i for i, _, _ in step)
            for i, p0, p1 in step:
                assert p0 == covered.get(i, 0) and p1 > p0       # every sequence front to back without gaps
                covered[i] = p1
        assert [covered[i] for i in range(len(lens))] == lens
