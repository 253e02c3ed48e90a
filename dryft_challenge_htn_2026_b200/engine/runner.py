"""The step function: a model, its cache, and ``step`` over a batch of sequences.

``step`` runs exactly the tokens it is given as one batch, from what earlier steps left in the
cache, and returns the logits at the wanted places. Sequences of a step either all start (their
prompts, of any lengths, in one ragged pass) or each continue with the tokens given; nothing is
padded to a common length, and a sequence's result does not depend on the others in the batch.
"""
from collections import OrderedDict

import torch

from ..cache import Cache
from ..csrc import api
from .batch import build_context

GRAPH_MAX_TOKENS = 8192     # steps of more tokens are launched plainly (the reference's bound: engine/engine.py:30)
GRAPH_KEEP = 12             # captured step shapes kept, least recently used dropped first


class _StepGraph:
    def __init__(self):
        self.static = {}        # the step context's device buffer (engine.batch._pack)
        self.graph = None
        self.logits = None


class Runner:
    def __init__(self, model, max_tokens, max_slots=1024):
        """``max_tokens``: tokens all live sequences may hold together, each sequence rounded up
        to whole pages of 64."""
        self.model = model
        self.device = model.rt.device
        self.cache = Cache(model.entry_requests(), max_tokens, max_slots, self.device)
        self._scratch = {}
        self.vocab_size = model.spec.vocab_size
        self._seen = OrderedDict()      # step shapes run so far -> times
        self._graphs = OrderedDict()    # step shape -> _StepGraph
        self._generation = model.generation

    def begin(self):
        """A slot for a new sequence (its length starts at 0)."""
        return self.cache.begin()

    def end(self, slot):
        """Gives the sequence's pages and slot back."""
        self.cache.end(slot)

    def length(self, slot):
        return self.cache.length[slot]

    def _check(self, entries):
        for slot, tokens, _ in entries:
            if not self.cache.slots.is_live(slot):
                raise ValueError(f"slot {slot} is not live")
            if len(tokens) and (min(tokens) < 0 or max(tokens) >= self.vocab_size):
                raise ValueError(f"token id outside [0, {self.vocab_size})")
        if len({e[0] for e in entries}) != len(entries):
            raise ValueError("a slot appears twice in one step")

    def context(self, entries, pad_to=None, static=None):
        self._check(entries)
        ctx = build_context(self.cache, entries, self.device, self._scratch, pad_to, self.model.step_plans, static)
        self.model.prepare(ctx.max_position + 1)     # tables grow here, never inside a step
        return ctx

    def _shape(self, entries):
        """What fixes every launch of a step: the new and the cached length of each sequence, how
        many places are wanted, and how wide the page tables are. Steps of equal shape differ in
        data only (token ids, slots, page ids, which places)."""
        cache = self.cache
        for slot, tokens, _ in entries:
            cache.reserve(slot, len(tokens))
        return (tuple(len(t) for _, t, _ in entries), tuple(cache.length[s] for s, _, _ in entries),
                sum(len(w) for _, _, w in entries),
                tuple(max(len(r) for r in cache.page_rows(g, [s for s, _, _ in entries])) for g in range(len(cache.groups))))

    @torch.inference_mode()
    def step(self, entries, tap=None, with_context=False, graph=False):
        """entries: list of (slot, tokens, want). Returns float32 logits [sum(len(want)), vocab]
        on the device, in the order of the entries and of each ``want``. ``tap``: see
        ``CausalLM.forward``. ``with_context``: also return the step's ``StepContext`` (the
        generation loop samples from the logits with its positions and wanted rows).
        ``graph``: a step shape that comes a second time is captured as a CUDA graph and replayed
        from then on (short steps are bound by the host's launches otherwise; the reference
        captures its prefill per length too: engine/engine.py:505-536). The logits of a replayed
        step live in the graph's memory and are overwritten by the next step of that shape."""
        n_tok = sum(len(t) for _, t, _ in entries)
        if graph and tap is None and n_tok <= GRAPH_MAX_TOKENS and self.device.type == "cuda":
            self._check(entries)
            return self._graph_step(entries, with_context)
        ctx = self.context(entries)
        logits = self.model.forward(ctx, self.cache, tap)
        for slot, tokens, _ in entries:
            self.cache.commit(slot, len(tokens))
        if not ctx.is_decode:
            api.gemm_tc_check()
        return (logits, ctx) if with_context else logits

    def _graph_step(self, entries, with_context):
        shape = self._shape(entries)
        if self.model.prepare(max(p + n for n, p in zip(shape[0], shape[1]))) != self._generation:
            self._generation = self.model.generation
            self._graphs.clear()                      # they hold the addresses of the old tables
        sg = self._graphs.get(shape)
        if sg is None:
            times = self._seen.pop(shape, 0)
            self._seen[shape] = times + 1
            while len(self._seen) > 64:
                self._seen.popitem(last=False)
            if times == 0:                            # the first time plainly: it sizes the kernels' scratch memory
                return self.step(entries, with_context=with_context)
            sg = _StepGraph()
            ctx = self.context(entries, static=sg.static)
            torch.cuda.synchronize()
            sg.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(sg.graph):
                sg.logits = self.model.forward(ctx, self.cache)
            sg.ctx = ctx
            self._graphs[shape] = sg
            while len(self._graphs) > GRAPH_KEEP:
                self._graphs.popitem(last=False)
        else:
            self._graphs.move_to_end(shape)
            sg.ctx = self.context(entries, static=sg.static)   # same shape: the same views, new data
        sg.graph.replay()
        for slot, tokens, _ in entries:
            self.cache.commit(slot, len(tokens))
        if not sg.ctx.is_decode:
            api.gemm_tc_check()
        return (sg.logits, sg.ctx) if with_context else sg.logits
