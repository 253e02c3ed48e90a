"""Keeps HBM busy between the weight-streaming kernels of a decode step.

A decode step alternates kernels that stream a weight matrix at memory speed with short kernels
that wait on latency (norms, rotary + cache write, attention over a short context, merges). While
a short one runs, a side stream asks the memory system to bring the next weight matrix into L2
(``cp.async.bulk.prefetch.L2``), so the product that follows reads it from L2. The matrices are
visited in the order the model uses them; inside a captured graph the side stream is a parallel
branch that starts when the product before it has finished."""
import torch

from ..csrc import api


class WeightPrefetcher:
    def __init__(self, weights, max_bytes=64 << 20):
        """``weights``: the matrices of one step in the order they are used."""
        self.order = list(weights)
        self.index = {w.data_ptr(): i for i, w in enumerate(self.order)}
        self.max_bytes = max_bytes
        self.side = torch.cuda.Stream()
        self.used = False

    def after(self, w):
        """Called right after the product with ``w`` was launched on the current stream."""
        i = self.index.get(w.data_ptr())
        if i is None or i + 1 >= len(self.order):
            return
        nxt = self.order[i + 1]
        n = min(nxt.numel() * nxt.element_size(), self.max_bytes) // nxt.element_size()
        self.side.wait_stream(torch.cuda.current_stream())
        api.l2_prefetch(nxt.view(-1)[:n], stream=self.side)
        self.used = True

    def join(self):
        """The side branch ends here (a captured graph needs every branch joined)."""
        if self.used:
            torch.cuda.current_stream().wait_stream(self.side)
            self.used = False
