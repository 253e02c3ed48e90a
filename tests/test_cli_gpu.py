"""The command line, run as a user runs it: generation with random weights of a tiny configuration,
its printed tokens against the plain implementation's greedy tokens, its JSON records, and its check
reporting a weight that is not finite (the fault is planted in a host copy of the weights; the
reference plants its NaN on the host too: tests/test_selftest_fallback.py:27-43)."""
import json
import os
import subprocess
import sys

import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_qwen3 as plain
from dryft_challenge_htn_2026_b200.cli import random_prompts
from helpers import ROOT, TINY, make_folder, tiny_config

pytestmark = pytest.mark.gpu


def run_cli(*args):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run([sys.executable, "-m", "dryft_challenge_htn_2026_b200.cli", *args], capture_output=True, text=True,
                          env=env, cwd=str(ROOT), timeout=900)


def test_cli_generates_prints_tokens_and_checks_itself(tmp_path):
    cfg_path = str(tmp_path / "config.json")
    tiny_config("B").save(str(tmp_path))
    model_dir = str(tmp_path / "model")
    r = run_cli("--random-weights", cfg_path, "--save-model", model_dir, "--seed", "3", "--dtype", "float32",
                "--shapes", "2,20,6", "--samples", "1", "--print-tokens")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "B2 20->6:" in r.stdout and "correctness: worst gap" in r.stdout and "geomean" in r.stdout
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens 2,20,6 seq ")]
    assert len(lines) == 2
    pcfg, t = plain.read_model(model_dir)
    prompts = random_prompts(2, 20, 1, TINY["B"]["vocab_size"], False)    # the first timed sample's prompts
    for i, line in enumerate(lines):
        emitted = [int(x) for x in line.split(":")[1].split()]
        want = plain.greedy(pcfg, t, prompts[i], 6)
        if emitted != want:                                               # a near-tie may flip: then the gap is rounding-small
            logits = plain.forward(pcfg, t, prompts[i] + emitted[:-1])[len(prompts[i]) - 1:]
            gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
            assert gap < 1e-4, (emitted, want)
    # bfloat16, ragged, two shapes, JSON records
    r = run_cli("--model", model_dir, "--shapes", "3,40,5", "1,70,3", "--samples", "2", "--ragged", "--json", "--check-all")
    assert r.returncode == 0, r.stdout + r.stderr
    records = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [x["shape"] for x in records] == ["3,40,5", "1,70,3"]
    assert all(x["tok_s"] > 0 and x["ttft_ms"] > 0 and x["worst_gap"] <= 2.0 for x in records)


def test_cli_check_reports_a_weight_that_is_not_finite(tmp_path):
    folder = make_folder(tmp_path, "A", seed=1)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    w["model.layers.1.mlp.down_proj.weight"][3, 5] = float("nan")
    save_file(w, path)
    r = run_cli("--model", folder, "--shapes", "2,12,4", "--samples", "1")
    assert r.returncode == 1, r.stdout + r.stderr
    assert "CHECK FAILED" in r.stdout and "not finite" in r.stdout
    r = run_cli("--model", folder, "--shapes", "2,12,4", "--samples", "1", "--no-check")
    assert r.returncode == 0                                              # unchecked, it runs through
