"""bin/trace_run against the plain implementation: the same requests replayed whole, with the last
32 tokens one by one, and in batches of unequal lengths whose shorter requests end earlier, one
batch after another so that slots and pages are used again — in float32 and in bfloat16."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, make_folder, random_tokens, run_trace, tolerance

pytestmark = pytest.mark.gpu

# request lengths per configuration: a single token, a page boundary (64, 65), several pages
LENGTHS = {"A": [40, 33, 64, 100, 65, 37], "B": [33, 64, 47, 130, 38, 90], "C": [35, 129, 64, 80, 200, 41],
           "D": [300, 34, 129, 64, 260, 161], "E": [400, 140, 33, 151, 290, 64], "F": [70, 33, 210, 64, 129, 47]}
TAIL = 32


def build_steps(seqs, whole=True):
    """Steps for trace_run and, per step, which (request, position) each wanted row is."""
    steps, meaning = [], {}

    def add(entries, end=()):
        k = len(steps)
        steps.append({"step": k, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w, _ in entries], "end": list(end)})
        meaning[k] = [(r, p0 + j) for _, _, w, (r, p0) in entries for j in w]

    # 1. each request alone and whole, logits everywhere
    for r, s in enumerate(seqs if whole else []):
        add([(f"w{r}", s, list(range(len(s))), (r, 0))], end=[f"w{r}"])
    # 2. all but the last 32 tokens in one step (logits at its end), then one token a step
    for r, s in enumerate(seqs):
        n = len(s) - TAIL
        add([(f"t{r}", s[:n], [n - 1], (r, 0))])
        for p in range(n, len(s)):
            add([(f"t{r}", [s[p]], [0], (r, p))], end=[f"t{r}"] if p == len(s) - 1 else [])
    # 3. batches of three requests of unequal lengths: prompts (all but 32 tokens) in one step,
    #    then one token each; a request leaves the batch when its tokens run out; the second batch
    #    starts when the first has ended, on the slots and pages it gave back
    for b0 in range(0, len(seqs), 3):
        group = list(range(b0, min(b0 + 3, len(seqs))))
        cut = {r: max(1, len(seqs[r]) - TAIL - 7 * (r % 3)) for r in group}    # unequal numbers of decode steps too
        add([(f"b{r}", seqs[r][:cut[r]], [0, cut[r] - 1], (r, 0)) for r in group])
        for k in range(max(len(seqs[r]) - cut[r] for r in group)):
            live = [r for r in group if cut[r] + k < len(seqs[r])]
            add([(f"b{r}", [seqs[r][cut[r] + k]], [0], (r, cut[r] + k)) for r in live],
                end=[f"b{r}" for r in live if cut[r] + k == len(seqs[r]) - 1])
    return steps, meaning


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_replay_matches_plain_however_the_tokens_are_cut(tmp_path, name, dtype):
    folder = make_folder(tmp_path, name, seed=5)
    cfg, t = plain.read_model(folder)
    seqs = [random_tokens(TINY[name]["vocab_size"], n, 100 + i) for i, n in enumerate(LENGTHS[name])]
    ref = [plain.forward(cfg, t, s) for s in seqs]
    steps, meaning = build_steps(seqs)
    # the most tokens live at once: the largest batch of three, each rounded up to pages of 64
    most = max(sum((len(seqs[r]) + 63) // 64 * 64 for r in range(b0, min(b0 + 3, len(seqs)))) for b0 in range(0, len(seqs), 3))
    out = run_trace(folder, dtype, str(tmp_path / f"out_{name}_{dtype}"), most, steps)
    worst, worst_at = 0.0, None
    seen = {}
    for k, rows in meaning.items():
        got = torch.from_numpy(out[k])
        assert got.shape[0] == len(rows) and torch.isfinite(got).all()
        for row, (r, p) in zip(got, rows):
            err = float((row - ref[r][p]).abs().max())
            if err > worst:
                worst, worst_at = err, (k, r, p)
            seen.setdefault((r, p), []).append(row)
    tol = tolerance(dtype, torch.cat(ref))
    assert worst <= tol, f"{name} {dtype}: |engine - plain| = {worst} at (step, request, position) {worst_at}, allowed {tol}"
    # the same position reached three ways: the ways agree with each other at least as closely
    spread = max(float((torch.stack(v) - v[0]).abs().max()) for v in seen.values() if len(v) > 1)
    assert spread <= tol
    assert all((r, len(s) - 1) in seen and len(seen[(r, len(s) - 1)]) == 3 for r, s in enumerate(seqs))


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_replay_through_the_decode_state_that_generation_uses(tmp_path, name, dtype, graph):
    """The one-token steps of the same schedules (last 32 tokens one by one; batches of unequal lengths
    whose shorter requests end earlier, a second batch on the slots the first gave back) run through
    the generation loop's decode state: positions advanced on the device, padded power-of-two rows,
    page tables rewritten when a page or the set of requests changes, plainly launched and as a
    CUDA graph. The logits, not only the tokens, agree with the plain implementation."""
    folder = make_folder(tmp_path, name, seed=6)
    cfg, t = plain.read_model(folder)
    seqs = [random_tokens(TINY[name]["vocab_size"], n, 200 + i) for i, n in enumerate(LENGTHS[name])]
    ref = [plain.forward(cfg, t, s) for s in seqs]
    steps, meaning = build_steps(seqs, whole=False)
    most = max(sum((len(seqs[r]) + 63) // 64 * 64 for r in range(b0, min(b0 + 3, len(seqs)))) for b0 in range(0, len(seqs), 3))
    out = run_trace(folder, dtype, str(tmp_path / "out"), most, steps, ["--decode-state"] + (["--graph"] if graph else []))
    tol = tolerance(dtype, torch.cat(ref))
    worst, worst_at, seen = 0.0, None, {}
    for k, rows in meaning.items():
        got = torch.from_numpy(out[k])
        assert got.shape[0] == len(rows) and torch.isfinite(got).all()
        for row, (r, p) in zip(got, rows):
            err = float((row - ref[r][p]).abs().max())
            if err > worst:
                worst, worst_at = err, (k, r, p)
            seen.setdefault((r, p), []).append(row)
    assert worst <= tol, f"{name} {dtype}: |engine - plain| = {worst} at (step, request, position) {worst_at}, allowed {tol}"
    assert all(len(seen[(r, len(s) - 1)]) == 2 for r, s in enumerate(seqs))


def test_layer_dumps_find_the_layer_where_two_replays_part_ways(tmp_path):
    """--dump-layers writes the residual stream after every layer; tests/layer_diff.py compares two
    dumps (here: the same model with one weight of layer 1 changed) and the dump with the plain
    implementation's layers."""
    import json
    import os
    import subprocess
    import sys

    from safetensors.torch import load_file, save_file

    from helpers import ROOT
    a = make_folder(tmp_path, "B", seed=3)
    b = str(tmp_path / "changed")
    os.makedirs(b)
    json.dump(json.load(open(os.path.join(a, "config.json"))), open(os.path.join(b, "config.json"), "w"))
    w = load_file(os.path.join(a, "model.safetensors"))
    w["model.layers.1.mlp.down_proj.weight"] = w["model.layers.1.mlp.down_proj.weight"] * 1.5
    save_file(w, os.path.join(b, "model.safetensors"))
    tokens = random_tokens(TINY["B"]["vocab_size"], 70, 9)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tokens, "want": [0, 33, 69]}], "end": ["x"]}]
    for folder, out in ((a, "da"), (b, "db")):
        run_trace(folder, "float32", str(tmp_path / out), 128, steps, ["--dump-layers"])
    script = os.path.join(ROOT, "tests", "layer_diff.py")
    r = subprocess.run([sys.executable, script, str(tmp_path / "da"), str(tmp_path / "db"), "--step", "0", "--hidden",
                        str(TINY["B"]["hidden_size"])], capture_output=True, text=True)
    assert r.returncode == 1 and "first difference after layer 1" in r.stdout, r.stdout + r.stderr
    r = subprocess.run([sys.executable, script, str(tmp_path / "da"), "--plain", a, "--step", "0", "--hidden",
                        str(TINY["B"]["hidden_size"]), "--trace", json.dumps(steps[0])], capture_output=True, text=True)
    assert r.returncode == 0 and "no difference" in r.stdout, r.stdout + r.stderr
