#!/usr/bin/env python3
"""Finds the first layer where two replays, or a replay and the plain implementation, part ways.

    python tests/layer_diff.py DUMP_A DUMP_B --step K --hidden H [--tol T]
    python tests/layer_diff.py DUMP_A --plain MODEL_DIR --trace '<the step's JSON line>' --step K --hidden H

``DUMP_*`` are output folders of ``bin/trace_run --dump-layers``: ``<step>.h<k>.f32`` holds the
residual stream after the k-th layer of the schedule at the step's wanted places. Prints, per
layer, the largest difference relative to the layer's largest value, and the first layer where it
exceeds the tolerance; exits with 1 if there is one. With ``--plain`` the other side is the plain
implementation (``tests/plain_qwen3.py``) run on the step's tokens, which must then be whole
requests from their first token (the reference does the same comparison between its two back ends
with its ``_trace`` hook: tests/trace_diff2.py:25-52).
"""
import argparse
import glob
import json
import os
import re
import sys

import numpy as np


def load_dump(folder, step, hidden):
    layers = {}
    for path in glob.glob(os.path.join(folder, f"{step}.h*.f32")):
        k = int(re.search(r"\.h(\d+)\.f32$", path).group(1))
        layers[k] = np.fromfile(path, dtype="<f4").reshape(-1, hidden)
    if not layers:
        sys.exit(f"no layer dumps of step {step} in {folder} (run bin/trace_run with --dump-layers)")
    return [layers[k] for k in sorted(layers)]


def plain_layers(model_dir, trace_line):
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import plain_qwen3 as plain
    cfg, t = plain.read_model(model_dir)
    per_entry = []
    for e in json.loads(trace_line)["entries"]:
        hidden = []
        plain.forward(cfg, t, e["tokens"], hidden_out=hidden)
        per_entry.append([h[e.get("want", [])].numpy() for h in hidden])
    return [np.concatenate([pe[k] for pe in per_entry]) for k in range(len(per_entry[0]))]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("a")
    ap.add_argument("b", nargs="?")
    ap.add_argument("--plain", metavar="MODEL_DIR")
    ap.add_argument("--trace", help="with --plain: the JSON line of the step")
    ap.add_argument("--step", required=True)
    ap.add_argument("--hidden", type=int, required=True)
    ap.add_argument("--tol", type=float, default=1e-3, help="relative to the layer's largest value")
    args = ap.parse_args()
    if (args.b is None) == (args.plain is None):
        ap.error("give a second dump folder or --plain MODEL_DIR")
    a = load_dump(args.a, args.step, args.hidden)
    b = load_dump(args.b, args.step, args.hidden) if args.b else plain_layers(args.plain, args.trace)
    if len(a) != len(b) or a[0].shape != b[0].shape:
        sys.exit(f"the two sides differ in shape: {len(a)} layers of {a[0].shape} against {len(b)} of {b[0].shape}")
    first = None
    for k, (x, y) in enumerate(zip(a, b)):
        rel = float(np.abs(x - y).max()) / max(1e-30, float(np.abs(y).max()))
        row = int(np.abs(x - y).max(1).argmax())
        print(f"layer {k:3d}: max |a - b| / max |b| = {rel:.3e} (wanted row {row})")
        if first is None and rel > args.tol:
            first = k
    if first is None:
        print("no difference above the tolerance")
        return 0
    print(f"first difference after layer {first}")
    return 1


if __name__ == "__main__":
    sys.exit(main())
