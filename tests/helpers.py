"""Tiny configurations and model folders for the tests (random weights, temporary folders)."""
import os
import subprocess
import sys

import numpy as np
import torch

import dryft_challenge_htn_2026_b200 as dk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three configurations that differ in every size and option. A and B are the two tiny models of
# the benchmark description; C adds what they leave out: a sliding window on the later layers, a
# group of 3 query heads per kv head, an odd head count, a vocabulary that is no multiple of 16.
TINY = {
    "A": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
              max_position_embeddings=128),
    "B": dict(vocab_size=384, hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
              max_position_embeddings=256),
    "C": dict(vocab_size=300, hidden_size=72, intermediate_size=104, num_hidden_layers=4, num_attention_heads=3,
              num_key_value_heads=1, head_dim=48, rms_norm_eps=3e-6, rope_theta=500000.0, tie_word_embeddings=True,
              max_position_embeddings=512, use_sliding_window=True, sliding_window=37, max_window_layers=2),
    # head size 64: the size the tcgen05 attention kernel is built for besides 128
    "D": dict(vocab_size=320, hidden_size=128, intermediate_size=192, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=100000.0, tie_word_embeddings=False,
              max_position_embeddings=512),
    # head size 128 with a window on the upper layers: the tcgen05 attention's window path inside a model
    "E": dict(vocab_size=264, hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, head_dim=128, rms_norm_eps=2e-6, rope_theta=20000.0, tie_word_embeddings=True,
              max_position_embeddings=1024, use_sliding_window=True, sliding_window=150, max_window_layers=1),
    # what the others leave out in one model: head size 48 with a group of 3, an untied head and a window from the
    # second layer on
    "F": dict(vocab_size=272, hidden_size=80, intermediate_size=112, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=2, head_dim=48, rms_norm_eps=1e-5, rope_theta=300000.0, tie_word_embeddings=False,
              max_position_embeddings=512, use_sliding_window=True, sliding_window=45, max_window_layers=1),
}


def tiny_config(name):
    return dk.Qwen3Config.from_dict(dict(TINY[name], architectures=["Qwen3ForCausalLM"]))


def make_folder(tmp_path, name, seed=0, dtype=torch.float32, std=0.08):
    """Writes the tiny model ``name`` with the library's random-weights mode; float32 on disk so
    that the plain implementation and both engine dtypes start from the same numbers."""
    folder = os.path.join(str(tmp_path), f"tiny{name}_{seed}")
    dk.write_random_model(tiny_config(name), folder, seed=seed, dtype=dtype, matrix_std=std)
    return folder


def random_tokens(vocab, n, seed):
    return np.random.RandomState(seed).randint(0, vocab, n).tolist()


def tolerance(dtype, ref):
    """Largest allowed |engine - plain| for logits: float32 differs by summation order only;
    bfloat16 rounds weights, activations and cache to 8 bits of mantissa."""
    scale = max(1.0, float(ref.abs().max()))
    return (2e-4 if dtype == "float32" else 6e-2) * scale


def run_trace(folder, dtype, out_dir, max_tokens, steps, extra=()):
    """Runs bin/trace_run on ``steps`` (list of dicts); returns {step: float32 array [wanted, vocab]}."""
    import json

    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-4000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], proc.stdout[-2000:]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        if n:
            out[s["step"]] = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(n, vocab)
    return out
