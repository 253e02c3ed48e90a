"""The step function: a model, its cache, and ``step`` over a batch of sequences.

``step`` runs exactly the tokens it is given as one batch, from what earlier steps left in the
cache, and returns the logits at the wanted places. Sequences of a step either all start (their
prompts, of any lengths, in one ragged pass) or each continue with the tokens given; nothing is
padded to a common length, and a sequence's result does not depend on the others in the batch.
"""
import torch

from ..cache import Cache
from ..csrc import api
from .batch import build_context


class Runner:
    def __init__(self, model, max_tokens, max_slots=1024):
        """``max_tokens``: tokens all live sequences may hold together, each sequence rounded up
        to whole pages of 64."""
        self.model = model
        self.device = model.rt.device
        self.cache = Cache(model.entry_requests(), max_tokens, max_slots, self.device)
        self._scratch = {}
        self.vocab_size = model.spec.vocab_size

    def begin(self):
        """A slot for a new sequence (its length starts at 0)."""
        return self.cache.begin()

    def end(self, slot):
        """Gives the sequence's pages and slot back."""
        self.cache.end(slot)

    def length(self, slot):
        return self.cache.length[slot]

    def context(self, entries, pad_to=None):
        for slot, tokens, _ in entries:
            if not self.cache.slots.is_live(slot):
                raise ValueError(f"slot {slot} is not live")
            if len(tokens) and (min(tokens) < 0 or max(tokens) >= self.vocab_size):
                raise ValueError(f"token id outside [0, {self.vocab_size})")
        if len({e[0] for e in entries}) != len(entries):
            raise ValueError("a slot appears twice in one step")
        return build_context(self.cache, entries, self.device, self._scratch, pad_to, self.model.step_plans)

    @torch.inference_mode()
    def step(self, entries, tap=None, with_context=False):
        """entries: list of (slot, tokens, want). Returns float32 logits [sum(len(want)), vocab]
        on the device, in the order of the entries and of each ``want``. ``tap``: see
        ``CausalLM.forward``. ``with_context``: also return the step's ``StepContext`` (the
        generation loop samples from the logits with its positions and wanted rows)."""
        ctx = self.context(entries)
        logits = self.model.forward(ctx, self.cache, tap)
        for slot, tokens, _ in entries:
            self.cache.commit(slot, len(tokens))
        if not ctx.is_decode:
            api.gemm_tc_check()
        return (logits, ctx) if with_context else logits
