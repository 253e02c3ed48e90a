"""The description of one step that every part reads: which token rows it holds, which sequence
and position each belongs to, where the sequences' pages are, and whose logits are wanted.

All arrays are int32 on the device, uploaded in one copy from pinned host memory (or, for a
captured decode loop, kept in place and advanced by the kernels).
"""
import numpy as np
import torch


class StepContext:
    """Fields:

    n_tok, n_seq, n_want     counts of token rows, sequences, wanted logit rows
    is_decode                every sequence brings exactly one token
    max_position             largest position of any row
    tok [n_tok]              token ids
    row_seq [n_tok]          index (0..n_seq-1) of each row's sequence within this step
    row_pos [n_tok]          position of each row in its sequence; -1 marks a padding row
    cu_q [n_seq+1]           first row of each sequence
    seq_slot [n_seq]         cache slot of each sequence (row index into per-sequence state)
    seq_pos0 [n_seq]         tokens the sequence had cached before this step
    want_rows [n_want]       rows whose logits are returned, in request order
    tables[g] [n_seq, P_g]   page ids of each sequence in cache group g
    plans[key]               what the parts' ``StepPlan`` objects built for this step (e.g. the
                             attention kernels' query tiles), on the device
    host                     dict of the same arrays as numpy, for parts that plan on the host; None
                             in a captured decode loop, whose positions advance on the device
    """

    def __init__(self, scratch_store=None):
        self._scratch = scratch_store if scratch_store is not None else {}
        self.plans = {}
        self.host = None

    def scratch(self, key, make):
        """A buffer (or tuple of buffers) that lives as long as the runner and is reused by every
        step with the same key; kernels' scratch memory comes from here."""
        if key not in self._scratch:
            self._scratch[key] = make()
        return self._scratch[key]


def _pack(arrays, device, static=None):
    """One pinned int32 buffer, one copy, views per array (each 16-byte aligned). ``static``: a dict
    that keeps the device buffer between calls, so that steps of the same shape find their arrays
    at the same addresses (a captured graph reads them there)."""
    offs, total = [], 0
    for a in arrays:
        offs.append(total)
        total += (a.size + 3) // 4 * 4
    host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=device.type == "cuda")
    hn = host.numpy()
    for a, o in zip(arrays, offs):
        hn[o:o + a.size] = a.reshape(-1)
    if static is None:
        dev = host.to(device, non_blocking=True)
    else:
        if "dev" not in static:
            static["dev"] = torch.empty(host.numel(), dtype=torch.int32, device=device)
        dev = static["dev"]
        if dev.numel() != host.numel():
            raise ValueError("a step context of another shape than the one its static buffer was made for")
        dev.copy_(host, non_blocking=True)
        static["host"] = host                  # pinned memory must outlive the copy
    return [dev[o:o + a.size].view(a.shape) for a, o in zip(arrays, offs)]


def build_context(cache, entries, device, scratch_store=None, pad_to=None, plans=(), static=None):
    """``entries``: list of (slot, tokens, want) with ``want`` positions among these tokens.
    Reserves cache room for the new tokens. ``pad_to``: for decode steps, pad the batch with rows
    of position -1 up to this many rows (a captured graph has a fixed size). ``plans``: the
    ``StepPlan`` objects of the model's parts; each is built once and uploaded with the rest.
    ``static``: see ``_pack``."""
    n_seq = len(entries)
    lens = np.array([len(e[1]) for e in entries], dtype=np.int64)
    if n_seq == 0 or (lens < 1).any():
        raise ValueError("a step needs at least one sequence and at least one token per sequence")
    pos0 = np.array([cache.length[e[0]] for e in entries], dtype=np.int64)
    for (slot, tokens, _), n in zip(entries, lens):
        cache.reserve(slot, int(n))
    cu = np.zeros(n_seq + 1, dtype=np.int64)
    np.cumsum(lens, out=cu[1:])
    n_tok = int(cu[-1])
    tok = np.concatenate([np.asarray(e[1], dtype=np.int64) for e in entries])
    row_seq = np.repeat(np.arange(n_seq), lens)
    row_pos = np.arange(n_tok) - np.repeat(cu[:-1] - pos0, lens)
    want = []
    for i, (_, tokens, w) in enumerate(entries):
        for j in w:
            if not 0 <= j < lens[i]:
                raise ValueError(f"wanted position {j} is outside the {lens[i]} tokens of entry {i}")
            want.append(cu[i] + j)
    is_decode = bool((lens == 1).all())
    rows = n_tok
    if pad_to is not None and is_decode and pad_to > n_tok:
        pad = pad_to - n_tok
        tok = np.concatenate([tok, np.zeros(pad, np.int64)])
        row_seq = np.concatenate([row_seq, np.zeros(pad, np.int64)])
        row_pos = np.concatenate([row_pos, -np.ones(pad, np.int64)])
        rows = pad_to
    slots = [e[0] for e in entries]
    tables = []
    for g in range(len(cache.groups)):
        t = np.array(cache.page_rows(g, slots), dtype=np.int32)
        if rows > n_seq and is_decode:   # padding rows index the table by row: give them rows of -1
            t = np.concatenate([t, -np.ones((rows - n_seq, t.shape[1]), np.int32)])
        tables.append(t)
    i32 = lambda a: np.ascontiguousarray(a, dtype=np.int32)
    by_key = {}
    for p in plans:
        if p.key not in by_key:
            by_key[p.key] = i32(p.build(lens, pos0, is_decode))
    fixed = [i32(tok), i32(row_seq), i32(row_pos), i32(cu), i32(slots), i32(pos0), i32(want)]
    dev = _pack(fixed + tables + list(by_key.values()), device, static)
    ctx = StepContext(scratch_store)
    ctx.n_tok, ctx.n_seq, ctx.n_want, ctx.is_decode = rows, n_seq, len(want), is_decode
    ctx.max_position = int((pos0 + lens).max()) - 1
    ctx.tok, ctx.row_seq, ctx.row_pos, ctx.cu_q, ctx.seq_slot, ctx.seq_pos0, ctx.want_rows = dev[:7]
    ctx.tables = dev[7:7 + len(tables)]
    ctx.plans = dict(zip(by_key, dev[7 + len(tables):]))
    ctx.host = dict(lens=lens, pos0=pos0, cu_q=cu, slots=slots, row_seq=row_seq, row_pos=row_pos)
    if is_decode:
        ctx.n_seq = rows  # the decode kernels run one sequence per row, padding rows included
    return ctx
