"""The generation loop above the step function.

``run_batch`` makes the decisions for one batch of sequences that start together — which
sequences are still running, when one has ended (stop token or token limit), when the batch is
re-packed without the ended ones — and talks to the device through a small backend interface, so
the decisions can be tested without a GPU. ``GpuBackend`` is that interface on the real model:
ragged prompts in one step, then one token per sequence per step from a decode state whose
buffers stay in place (token ids, positions, page tables), optionally replayed as a CUDA graph,
with the host reading tokens one step behind the device (reference: engine/engine.py:683-732).
"""
from collections import deque

import numpy as np
import torch

from ..csrc import api
from ..csrc.api import PAGE
from ..sampling import Sampler, seed_words
from .batch import StepContext


# ------------------------------------------------------------------------------ host decisions
class BatchTracker:
    """Outputs and end-of-sequence state of one batch."""

    def __init__(self, n, max_new_tokens, stop_token_ids=()):
        self.max_new = max_new_tokens
        self.stops = frozenset(stop_token_ids)
        self.outputs = [[] for _ in range(n)]
        self.finished = [False] * n

    def accept(self, who, tokens):
        """Tokens of one step for sequences ``who``. Returns (row, newly finished): row[i] is the
        token sequence i got this step, None if it had already ended."""
        row = [None] * len(self.outputs)
        newly = []
        for i, t in zip(who, tokens):
            if self.finished[i]:
                continue
            self.outputs[i].append(int(t))
            row[i] = int(t)
            if int(t) in self.stops or len(self.outputs[i]) >= self.max_new:
                self.finished[i] = True
                newly.append(i)
        return row, newly

    def active(self, who):
        return [i for i in who if not self.finished[i]]


def run_batch(backend, prompts, params, seeds):
    """Generator over the steps of one batch: yields, per step, a list with one token per
    sequence (None for sequences that ended earlier). ``backend`` must offer
    ``start(prompts, params, seeds)`` (prefill and first token; returns the pending tokens),
    ``decode()`` (launch one step for the current rows; returns pending tokens),
    ``repack(rows)`` with rows = [(sequence index, last token, tokens generated)], and
    ``finish()``. Pending tokens have ``wait() -> list``. One step is kept in flight while the
    host reads the previous one."""
    n = len(prompts)
    if params.max_new_tokens <= 0 or n == 0:
        return
    tracker = BatchTracker(n, params.max_new_tokens, params.stop_token_ids)
    who = list(range(n))
    try:
        queue = deque([(who, backend.start(prompts, params, seeds))])
        launched, repack = 1, False
        while True:
            while len(queue) < 2 and launched < params.max_new_tokens and not repack and who:
                queue.append((who, backend.decode()))
                launched += 1
            if not queue:
                break
            w, pending = queue.popleft()
            row, newly = tracker.accept(w, pending.wait())
            if any(t is not None for t in row):   # a step launched for sequences that had all ended
                yield row
            repack = repack or bool(newly)
            if repack and not queue:
                who = tracker.active(who)
                repack = False
                if who and launched < params.max_new_tokens:
                    backend.repack([(i, tracker.outputs[i][-1], len(tracker.outputs[i])) for i in who])
    finally:
        backend.finish()


def plan_batches(n_requests, batch_size):
    """Index ranges of consecutive batches covering all requests."""
    if batch_size < 1:
        raise ValueError("batch_size must be at least 1")
    return [range(s, min(n_requests, s + batch_size)) for s in range(0, n_requests, batch_size)]


def prefill_plan(lengths, limit):
    """Steps of a batch's prefill: each a list of (sequence, first token, end token). Whole sequences
    are taken in order while they fit ``limit`` tokens; a longer one is cut into chunks."""
    limit = max(1, limit)
    steps, cur, used = [], [], 0
    for i, n in enumerate(lengths):
        if n > limit:
            if cur:
                steps.append(cur)
                cur, used = [], 0
            steps += [[(i, p0, min(n, p0 + limit))] for p0 in range(0, n, limit)]
            continue
        if used + n > limit:
            steps.append(cur)
            cur, used = [], 0
        cur.append((i, 0, n))
        used += n
    if cur:
        steps.append(cur)
    return steps


def bucket_rows(n):
    """Rows of the decode state for n live sequences: the next power of two (a captured graph has
    a fixed size; padding rows are skipped by the kernels)."""
    b = 1
    while b < n:
        b *= 2
    return b


# ------------------------------------------------------------------------------------ device side
class _Pending:
    def __init__(self, host_row, event, n):
        self.host_row, self.event, self.n = host_row, event, n

    def wait(self):
        self.event.synchronize()
        return self.host_row[:self.n].tolist()


class DecodeState:
    """Device buffers of a decode loop for ``rows`` sequences with page tables ``width`` wide:
    token ids, positions, temperatures, seeds and page tables stay at fixed addresses; each step
    reads them, and the sampler writes the new token and advances the position in place."""

    def __init__(self, runner, rows, width):
        self.runner, self.rows, self.width = runner, rows, width
        dev = runner.device
        ng = len(runner.cache.groups)
        sizes = [rows, rows, rows, rows, rows, 2 * rows] + [rows * width] * ng
        offs = np.cumsum([0] + [(s + 3) // 4 * 4 for s in sizes])
        self.host = torch.zeros(int(offs[-1]), dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(int(offs[-1]), dtype=torch.int32, device=dev)
        cut = lambda buf, i, shape: buf[int(offs[i]):int(offs[i]) + sizes[i]].view(shape)
        names = ["tok", "row_seq", "row_pos", "seq_slot", "temps", "seeds"]
        shapes = [(rows,)] * 5 + [(rows, 2)]
        self.h = {n: cut(self.host, i, s).numpy() for i, (n, s) in enumerate(zip(names, shapes))}
        self.h["tables"] = [cut(self.host, 6 + g, (rows, width)).numpy() for g in range(ng)]
        self.h["temps"] = self.h["temps"].view(np.float32)
        d = {n: cut(self.dev, i, s) for i, (n, s) in enumerate(zip(names, shapes))}
        ctx = StepContext(runner._scratch)
        ctx.n_tok = ctx.n_seq = ctx.n_want = rows
        ctx.is_decode, ctx.max_position = True, 0
        ctx.tok, ctx.row_seq, ctx.row_pos, ctx.seq_slot = d["tok"], d["row_seq"], d["row_pos"], d["seq_slot"]
        ctx.want_rows = torch.arange(rows, dtype=torch.int32, device=dev)
        ctx.tables = [cut(self.dev, 6 + g, (rows, width)) for g in range(ng)]
        # one token a sequence: row i is sequence i, and what it had cached before is its position
        ctx.cu_q = torch.arange(rows + 1, dtype=torch.int32, device=dev)
        ctx.seq_pos0 = ctx.row_pos
        ctx.host = None                       # positions advance on the device: the host does not know them
        self.ctx = ctx
        self.logits = None                    # [rows, vocab] float32 of the last step (a fixed buffer once captured)
        self.filled = None                    # what fill() last wrote: [(slot, pages held)] per row
        self.lengths = None                   # tokens each of those sequences has cached, as the device positions stand
        self.tok_copied = torch.cuda.Event()
        self.temps = d["temps"].view(torch.float32)
        self.seeds = d["seeds"]
        self.sampler = Sampler(runner.vocab_size, rows, dev)
        self.graph = None
        self.ring = torch.zeros((4, rows), dtype=torch.int32, pin_memory=True)
        self.events = [torch.cuda.Event() for _ in range(4)]
        self.turn = 0

    def fill(self, seqs):
        """seqs: list of dict(slot, token, pos, temperature, seed). Unused rows become padding."""
        h, cache = self.h, self.runner.cache
        h["tok"][:] = 0
        h["row_seq"][:] = np.arange(self.rows)
        h["row_pos"][:] = -1
        h["seq_slot"][:] = 0
        h["temps"][:] = 0
        h["seeds"][:] = 0
        for t in h["tables"]:
            t[:] = -1
        for r, s in enumerate(seqs):
            h["tok"][r], h["row_pos"][r], h["seq_slot"][r] = s["token"], s["pos"], s["slot"]
            h["temps"][r] = s["temperature"]
            h["seeds"][r] = seed_words(s["seed"])
            for g, t in enumerate(h["tables"]):
                pages = cache.page_rows(g, [s["slot"]])[0][:self.width]
                t[r, :len(pages)] = pages
        self.dev.copy_(self.host, non_blocking=True)
        self.filled = [(s["slot"], cache.pages_held(s["slot"])) for s in seqs]
        self.lengths = [s["pos"] for s in seqs]

    def set_tokens(self, tokens):
        """Overwrites the token ids of the first len(tokens) rows (a replay that forces its tokens)."""
        n = len(tokens)
        self.tok_copied.synchronize()         # the pinned buffer is free again
        self.h["tok"][:n] = tokens
        self.dev[:n].copy_(self.host[:n], non_blocking=True)     # the token ids are the first array of the buffer
        self.tok_copied.record()

    def body(self, advance=True, out_tok=None):
        self.logits = self.runner.model.forward(self.ctx, self.runner.cache)
        self.sampler(self.logits, self.temps, self.seeds, self.ctx.row_pos, None,
                     self.ctx.tok if out_tok is None else out_tok, advance)

    def capture(self):
        """Two plain runs that leave positions and tokens alone (they compile and size everything,
        and only rewrite cache rows the real step writes again), then the captured one."""
        scratch_tok = torch.empty_like(self.ctx.tok)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.body(advance=False, out_tok=scratch_tok)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.body()
        self.graph = g

    def run(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.body()

    def read(self, n):
        """Starts the copy of the first n token ids to the host; returns the pending result."""
        k = self.turn % 4
        self.turn += 1
        self.ring[k].copy_(self.ctx.tok, non_blocking=True)
        self.events[k].record()
        return _Pending(self.ring[k], self.events[k], n)


class DecodeLoop:
    """One-token steps of a runner's sequences through decode states: token ids, positions and page
    tables at fixed addresses, the step replayed as a CUDA graph (or launched plainly). The states,
    and their graphs, are kept per (rows, table width). Generation decodes through it, and a replay
    of given tokens can (``forced_step``), so the logits of this path can be looked at too."""

    def __init__(self, runner, use_graph=True):
        self.runner, self.use_graph = runner, use_graph
        self.states = {}
        self.generation = runner.model.generation
        self.state = None

    def state_for(self, n_live, max_len):
        """The decode state for ``n_live`` sequences that will grow to at most ``max_len`` tokens."""
        rows = bucket_rows(n_live)
        width = bucket_rows((max_len + PAGE - 1) // PAGE)
        generation = self.runner.model.prepare(max_len)
        if generation != self.generation:     # position tables were rebuilt: graphs captured before are stale
            self.generation = generation
            self.states.clear()
        st = self.states.get((rows, width))
        if st is None:
            st = self.states[(rows, width)] = DecodeState(self.runner, rows, width)
        self.state = st
        return st

    def run(self):
        """Launches one step of the current state; its slots' cached lengths move on by one."""
        st = self.state
        if self.use_graph and st.graph is None:
            st.capture()
        st.run()
        cache = self.runner.cache
        for slot, _ in st.filled:
            cache.commit(slot, 1)
        st.lengths = [n + 1 for n in st.lengths]

    @torch.inference_mode()
    def forced_step(self, entries):
        """One token per sequence, given: entries [(slot, [token], want)]. Returns float32 logits of
        the entries whose ``want`` is not empty, in order. The state is filled anew when the
        sequences or their pages are not the ones it holds; otherwise only the tokens are written
        and the positions are those the last step left on the device."""
        cache = self.runner.cache
        for slot, tokens, _ in entries:
            if len(tokens) != 1:
                raise ValueError("a decode step takes exactly one token per sequence")
            cache.reserve(slot, 1)
        now = [(slot, cache.pages_held(slot)) for slot, _, _ in entries]
        st = self.state
        max_len = max(cache.length[slot] for slot, _, _ in entries) + 1
        if st is None or st.filled != now or st.lengths != [cache.length[slot] for slot, _, _ in entries] \
                or st.width * PAGE < max_len or self.runner.model.prepare(max_len) != self.generation:
            st = self.state_for(len(entries), max_len)
            st.fill([dict(slot=slot, token=tokens[0], pos=cache.length[slot], temperature=0.0, seed=0)
                     for slot, tokens, _ in entries])
        else:
            st.set_tokens([tokens[0] for _, tokens, _ in entries])
        self.run()
        rows = [i for i, (_, _, want) in enumerate(entries) if want]
        return st.logits[rows] if rows else st.logits[:0]


class GpuBackend:
    """``run_batch``'s backend on the real model. One instance serves many batches one after
    another. Prompts go through the step function (``Runner.step``), decoding through the
    runner's ``DecodeLoop``."""

    def __init__(self, runner, use_graph=True, max_prefill_tokens=32768):
        self.runner = runner
        self.loop = DecodeLoop(runner, use_graph)
        self.max_prefill_tokens = max_prefill_tokens   # most prompt tokens one step runs (bounds the activations)
        self.seqs = None

    @property
    def state(self):
        return self.loop.state

    @torch.inference_mode()
    def start(self, prompts, params, seeds):
        r = self.runner
        self.params = params
        slots = []
        try:
            for p in prompts:
                slots.append(r.begin())
                r.cache.reserve(slots[-1], len(p) + params.max_new_tokens)   # every page the sequence will need: the
        except Exception:                                                    # decode state's page tables stay as they are
            for s in slots:
                r.end(s)
            raise
        self.seqs = [dict(slot=s, token=0, pos=len(p), temperature=params.temperature, seed=sd, prompt_len=len(p))
                     for s, p, sd in zip(slots, prompts, seeds)]
        self.max_len = max(len(p) for p in prompts) + params.max_new_tokens
        st = self.loop.state_for(len(prompts), self.max_len)
        st.fill(self.seqs)
        for step in prefill_plan([len(p) for p in prompts], self.max_prefill_tokens):
            # logits only where a prompt ends; the first token of those sequences is sampled at once
            ended = [i for i, _, p1 in step if p1 == len(prompts[i])]
            logits, ctx = r.step([(slots[i], prompts[i][p0:p1], [p1 - p0 - 1] if p1 == len(prompts[i]) else [])
                                  for i, p0, p1 in step], with_context=True, graph=self.loop.use_graph)
            if ended:
                lo, hi = ended[0], ended[-1] + 1          # sequences are taken in order: a contiguous range
                st.sampler(logits, st.temps[lo:hi], st.seeds[lo:hi], ctx.row_pos, ctx.want_rows, st.ctx.tok[lo:hi], False)
        self.live = list(range(len(prompts)))
        return st.read(len(prompts))

    @torch.inference_mode()
    def decode(self):
        self.loop.run()
        return self.loop.state.read(len(self.live))

    @torch.inference_mode()
    def repack(self, rows):
        """rows: [(sequence index, last token, tokens generated so far)] of the sequences that go on."""
        seqs = []
        for i, tok, made in rows:
            s = dict(self.seqs[i])
            s["token"], s["pos"] = tok, s["prompt_len"] + made - 1
            seqs.append(s)
        torch.cuda.current_stream().synchronize()
        for i in set(self.live) - {r[0] for r in rows}:   # ended sequences give their pages back now
            self.runner.end(self.seqs[i]["slot"])
            self.seqs[i]["slot"] = None
        self.live = [r[0] for r in rows]
        self.loop.state_for(len(rows), self.max_len).fill(seqs)

    def finish(self):
        if self.seqs is None:
            return
        torch.cuda.current_stream().synchronize()
        for s in self.seqs:
            if s["slot"] is not None:
                self.runner.end(s["slot"])
        self.seqs = None
        api.gemm_tc_check()                   # the tensor-core kernels' bounded waits (decode steps of many rows)
