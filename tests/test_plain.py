"""The plain implementation against the reference engine's own CPU outputs (tests/golden)."""
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from golden.make_golden import GOLDEN_CONFIGS, N_GREEDY, golden_tokens, golden_weights

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name", sorted(GOLDEN_CONFIGS))
def test_plain_matches_reference_engine(name):
    cfg = GOLDEN_CONFIGS[name]
    g = np.load(os.path.join(HERE, "golden", f"{name}.npz"))
    seed = int(g["seed"])
    t = golden_weights(cfg, seed)
    toks = golden_tokens(cfg, seed)
    logits = plain.forward(cfg, t, toks)
    ref = torch.from_numpy(g["logits"])
    assert logits.shape == ref.shape
    # every prefix of the reference equals the matching row of one whole-sequence forward
    assert (logits - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
    assert plain.greedy(cfg, t, toks, N_GREEDY) == g["greedy"].tolist()


def test_plain_float64_agrees_with_float32():
    cfg = GOLDEN_CONFIGS["g2"]
    t = golden_weights(cfg, 3)
    toks = golden_tokens(cfg, 3)
    a = plain.forward(cfg, t, toks)
    b = plain.forward(cfg, {k: v.double() for k, v in t.items()}, toks)
    assert (a.double() - b).abs().max().item() < 1e-4


def test_window_and_schedule_options():
    cfg = dict(GOLDEN_CONFIGS["g1"], use_sliding_window=True, sliding_window=4, max_window_layers=1)
    t = golden_weights(cfg, 5)
    toks = golden_tokens(cfg, 5)
    full = plain.forward(GOLDEN_CONFIGS["g1"], t, toks)
    win = plain.forward(cfg, t, toks)
    # the first `window` positions see the same keys with and without the window
    assert torch.allclose(full[:4], win[:4], atol=1e-6)
    assert not torch.allclose(full[8:], win[8:], atol=1e-4)
    assert plain.layer_windows(cfg) == [None, 4]
    twice = plain.forward(GOLDEN_CONFIGS["g1"], t, toks, schedule=[(0, 0, True), (1, 1, True), (1, 2, True)])
    assert not torch.allclose(full, twice, atol=1e-4)
    shared = plain.forward(GOLDEN_CONFIGS["g1"], t, toks, schedule=[(0, 0, True), (1, 0, False)])
    assert not torch.allclose(full, shared, atol=1e-4)


def test_hash_is_uniform_enough():
    u = np.array([plain.hash_u32(7, 9, 3, i) for i in range(20000)], dtype=np.float64) / 2**32
    assert abs(u.mean() - 0.5) < 0.01 and abs(u.var() - 1 / 12) < 0.005
    assert len({plain.hash_u32(7, 9, p, 5) for p in range(1000)}) > 990
