"""Choosing the next token: greedy (the reference's only rule, engine/engine.py:503) and
temperature sampling with a seed per sequence.

The draw is the Gumbel-max rule on the GPU (``csrc/sampling.cu``): one pass over the logits, no
normalisation, and a sequence's draws depend only on its own seed and positions, so a request
samples the same tokens alone or in any batch."""
from dataclasses import dataclass, field
from typing import Tuple

import torch

from ..csrc import api

MASK64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 is greedy. ``seed`` seeds the whole call; request i draws from the stream
    ``request_seed(seed, i)``. Generation of a sequence ends after ``max_new_tokens`` tokens or
    with the first token that is in ``stop_token_ids`` (which is still returned)."""
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    stop_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")


def request_seed(seed, index):
    """64-bit seed of the index-th request of a call."""
    return ((int(seed) & MASK64) * 0x9E3779B97F4A7C15 + (int(index) + 1) * 0xD1B54A32D192ED03) & MASK64


def seed_words(seed64):
    """(low, high) 32-bit words as signed int32 values (the kernels read them as unsigned)."""
    def signed(x):
        return x - (1 << 32) if x >= (1 << 31) else x
    return signed(seed64 & 0xFFFFFFFF), signed((seed64 >> 32) & 0xFFFFFFFF)


class Sampler:
    """Owns the sampler kernel's scratch memory for up to ``max_rows`` rows of ``vocab`` logits."""

    def __init__(self, vocab, max_rows, device):
        self.vocab, self.max_rows = vocab, max_rows
        n = max_rows * api.sample_chunks(vocab)
        self.ws_val = torch.empty(n, dtype=torch.float32, device=device)
        self.ws_idx = torch.empty(n, dtype=torch.int32, device=device)

    def __call__(self, logits, temperature, seeds, pos, rows, out_tok, advance=False):
        """logits [n, vocab] float32; temperature [n] float32; seeds [n, 2] int32; ``pos`` int32
        positions looked up through ``rows`` (None: row i is position i); out_tok [n] int32."""
        if logits.shape[0] > self.max_rows:
            raise ValueError(f"sampler sized for {self.max_rows} rows, got {logits.shape[0]}")
        api.sample(logits, temperature, seeds, pos, rows, self.ws_val, self.ws_idx, out_tok, advance)
        return out_tok
