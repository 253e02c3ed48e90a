"""Keeps HBM busy between the weight-streaming kernels of a decode step.

A decode step alternates kernels that stream a weight matrix at memory speed with short kernels
that wait on latency (norms, rotary + cache write, merges). Each product kernel is told which
matrix the step uses next and asks the memory system to bring (the head of) it into L2
(``cp.async.bulk.prefetch.L2``) while it runs itself, so HBM keeps streaming through the short
kernels and the next product starts on warm lines. The matrices are visited in the order the
model uses them; nothing is launched for this and no stream is forked.

Measured on B200 (Qwen3-4B sizes, batch 8): the step gets 8 to 30 % slower with 16 to 100 MB of
lookahead, so the model leaves it off (``CausalLM.prefetch``)."""


class WeightPrefetcher:
    def __init__(self, weights, max_bytes=48 << 20):
        """``weights``: the matrices of one step in the order they are used. ``max_bytes``: how
        much of the next matrix is asked for (L2 holds 126 MB, and the running product's own
        matrix should stay in it)."""
        self.order = list(weights)
        self.index = {w.data_ptr(): i for i, w in enumerate(self.order)}
        self.max_bytes = max_bytes

    def next_after(self, w):
        """The piece of the next matrix to prefetch during the product with ``w`` (or None)."""
        i = self.index.get(w.data_ptr())
        if i is None or i + 1 >= len(self.order):
            return None
        nxt = self.order[i + 1]
        n = min(nxt.numel() * nxt.element_size(), self.max_bytes) // nxt.element_size()
        return nxt.view(-1)[:n]
