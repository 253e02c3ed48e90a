"""A causal language model put together from a ``ModelSpec``: embedding, blocks run in schedule
order, final norm, output head. ``forward`` runs one step over the token rows a ``StepContext``
describes and returns float32 logits at the wanted rows (reference: engine/engine.py:459-503).
"""
import torch

from ..csrc import api
from ..parts import ParamDecl, Runtime, build_part
from ..parts.block import add_norm
from ..parts.linear import STORE_F32, linear
from ..parts.norm import RMSNorm


class CausalLM:
    def __init__(self, spec, dtype=torch.bfloat16, device="cuda"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be torch.float32 or torch.bfloat16, not {dtype}")
        self.spec = spec
        self.rt = Runtime(torch.device(device), dtype)
        self.blocks = [build_part(ls, self.rt) for ls in spec.layers]
        self.final_norm = build_part(spec.final_norm, self.rt)
        n_entries = max(e.cache for e in spec.schedule) + 1
        owners = {}
        for e in spec.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.blocks)}")
            if e.writes:
                if e.cache in owners:
                    raise ValueError(f"cache entry {e.cache} is written by two schedule entries")
                owners[e.cache] = e.layer
        for e in spec.schedule:
            if e.cache not in owners:
                raise ValueError(f"cache entry {e.cache} is read but never written")
            if self.blocks[e.layer].cache_requests() != self.blocks[owners[e.cache]].cache_requests():
                raise ValueError(f"layer {e.layer} cannot use cache entry {e.cache}: its owner stores something else")
        self._entry_requests = [self.blocks[owners[c]].cache_requests() for c in range(n_entries)]
        self.embed = self.head = None
        self.tied = None
        # index arrays the parts' kernels want built for every step (engine.batch.build_context), once per key
        self.step_plans = list({p.key: p for b in self.blocks for p in b.step_plans()}.values())
        self.prepared = 0        # positions the parts' tables reach
        self.generation = 0      # counts the times they were rebuilt: captured graphs hold the old tables' addresses

    # -- parameters --------------------------------------------------------------------------
    def param_decls(self, tied):
        """Checkpoint name -> ParamDecl for the whole model."""
        s = self.spec
        out = {s.embed_name: ParamDecl(s.embed_name, (s.vocab_size, s.hidden_size), "matrix")}
        for ls, blk in zip(s.layers, self.blocks):
            for p in blk.param_decls():
                out[ls.prefix + p.name] = p
        for p in self.final_norm.param_decls():
            out[s.final_norm_prefix + p.name] = p
        if not tied:
            out[s.head_name] = ParamDecl(s.head_name, (s.vocab_size, s.hidden_size), "matrix")
        return out

    def bind(self, tensors, tied):
        s = self.spec
        self.tied = tied
        self.embed = tensors.pop(s.embed_name).contiguous()
        self.head = self.embed if tied else tensors.pop(s.head_name).contiguous()
        for ls, blk in zip(s.layers, self.blocks):
            n = len(ls.prefix)
            blk.bind({k[n:]: tensors.pop(k) for k in [k for k in tensors if k.startswith(ls.prefix)]})
        n = len(s.final_norm_prefix)
        self.final_norm.bind({k[n:]: tensors.pop(k) for k in [k for k in tensors if k.startswith(s.final_norm_prefix)]})

    def entry_requests(self):
        return self._entry_requests

    def prepare(self, max_positions):
        """Makes the parts' tables (rotation angles) reach ``max_positions``; they grow by doubling.
        Returns ``generation``, which changes whenever they were rebuilt."""
        if max_positions > self.prepared:
            self.prepared = max(max_positions, 2 * self.prepared, 256)
            for b in self.blocks:
                b.prepare(self.prepared)
            self.generation += 1
        return self.generation

    def weight_bytes_per_step(self):
        """Bytes of weights a decode step reads: what every part says it streams once a step, for
        every run of a layer in the schedule, and the head (the embedding is read by row only, so it
        counts only where it is also the head)."""
        total = self.head.numel() * self.head.element_size()
        for e in self.spec.schedule:
            total += sum(w.numel() * w.element_size() for w in self.blocks[e.layer].step_weights())
        return total

    # -- one step ----------------------------------------------------------------------------
    def forward(self, ctx, cache, tap=None):
        """``tap(k, h)``: called after the k-th schedule entry with the residual stream as it then
        stands (that entry's feed-forward output added in): for dumps that look for the layer where
        two runs part ways. It costs a launch and a copy per entry, so it is for debugging only."""
        s, rt = self.spec, self.rt
        h = torch.empty((ctx.n_tok, s.hidden_size), dtype=torch.float32, device=rt.device)
        a = torch.empty((ctx.n_tok, s.hidden_size), dtype=rt.dtype, device=rt.device)
        first = self.blocks[s.schedule[0].layer]
        fused = isinstance(first.norm_in, RMSNorm)       # the embedding kernel computes RMSNorm and nothing else
        api.embed_rmsnorm(ctx.tok, self.embed, first.norm_in.weight if fused else None,
                          first.norm_in.spec.eps if fused else 0.0, h, a)
        pending = None
        for i, e in enumerate(s.schedule):
            pending = self.blocks[e.layer].forward(ctx, h, pending, cache.views(e.cache), e.writes,
                                                   a if (i == 0 and fused) else None)
            if tap is not None:
                tap(i, h + (pending.ws.sum(0) if isinstance(pending, api.Partial) else pending.to(torch.float32)))
        if ctx.n_want == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=rt.device)
        an = add_norm(self.final_norm, h, pending, rt.dtype, rows=ctx.want_rows)
        return linear(an, self.head, STORE_F32)
