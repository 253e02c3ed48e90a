"""Decode and prefill throughput of the Qwen3-4B layer sizes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at the default batch of 8: K decode
steps of the captured decode loop, timed with CUDA events after W warm-up steps, every sequence
with about 3,000 tokens of context already cached (a 2,048-token prompt, ragged 1,024..2,048 for
batches above one, plus 1,024 tokens decoded so far: the midpoint of a 4,096-token context).
``e2e`` is the same measured through ``Engine.generate`` (host token lists in, host tokens out).
``prefill`` is one 2,048-token prompt; ``roofline`` relates the decode step to the bytes it must
read; ``points`` hold batch 1 and 64. The weights (8 GB) are far larger than L2, so no flush is
needed between steps. For more than one GPU it says so and exits with 2: this library runs on one.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=2560, intermediate_size=9728,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=True, max_position_embeddings=40960)
CONTEXT = 4096
PROMPT = 2048
DECODED_SO_FAR = 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.lines, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6 or not parts[0].isdigit():
                continue
            sm.append(int(parts[0]))
            mx.append(int(parts[1]))
            reasons.update(n for n, v in zip(names, parts[2:]) if v == "Active")
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def ragged_lengths(batch, seed):
    import numpy as np
    if batch == 1:
        return [PROMPT + DECODED_SO_FAR]
    r = np.random.RandomState(seed)
    return [int(x) + DECODED_SO_FAR for x in r.randint(PROMPT // 2, PROMPT + 1, batch)]


def time_decode(torch, dk, model, batch, steps, warmup, seed, sampler=None):
    """K decode steps of the generation loop's own decode state (graph replay), timed on the device."""
    import numpy as np
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.generate import GpuBackend
    from dryft_challenge_htn_2026_b200.sampling import SamplingParams

    lens = ragged_lengths(batch, seed)
    total_new = warmup + steps + 8
    need = sum((n + total_new + 63) // 64 * 64 for n in lens)
    runner = dk.Runner(model, need, max_slots=max(batch, 1))
    backend = GpuBackend(runner, use_graph=True)
    rs = np.random.RandomState(seed + 1)
    prompts = [rs.randint(0, model.spec.vocab_size, n).tolist() for n in lens]
    params = SamplingParams(total_new)
    backend.start(prompts, params, [0] * batch).wait()     # prefill (in steps of at most 32k tokens) and the first token
    st = backend.state
    count0 = api.launch_count()
    st.body(advance=False, out_tok=torch.empty_like(st.ctx.tok))
    launches_per_step = api.launch_count() - count0
    st.capture()
    for _ in range(warmup):
        st.run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    with (sampler or ClockSampler()) as cs:
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(steps):
            st.run()
        ev[1].record()
        torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / steps
    ctx_mean = sum(lens) / batch + warmup + steps / 2
    kv_bytes = sum(g.request.n_kv_heads * g.request.head_dim * 2 * len(g.entries) * 2
                   for g in runner.cache.groups if hasattr(g, "pool"))
    step_bytes = model.weight_bytes_per_step() + batch * ctx_mean * kv_bytes
    backend.finish()
    del st, backend, runner
    torch.cuda.empty_cache()
    return dict(ms=ms, tok_s=batch / ms * 1e3, bytes=step_bytes, ctx_mean=ctx_mean, launches=launches_per_step,
                clocks=cs.summary())


def timeline(torch, dk, api, model, batch):
    """One decode step inside the captured graph: for every kernel the time from the end of its
    wait for its predecessor to the end of the next kernel's wait (so overlap is counted once)."""
    import collections

    import numpy as np
    from dryft_challenge_htn_2026_b200.engine.generate import GpuBackend
    from dryft_challenge_htn_2026_b200.sampling import SamplingParams

    lens = ragged_lengths(batch, 0)
    runner = dk.Runner(model, sum((n + 64 + 63) // 64 * 64 for n in lens), max_slots=batch)
    backend = GpuBackend(runner, use_graph=True)
    rs = np.random.RandomState(1)
    backend.start([rs.randint(0, model.spec.vocab_size, n).tolist() for n in lens], SamplingParams(48), [0] * batch).wait()
    st = backend.state
    st.capture()
    for _ in range(32):
        st.run()
    torch.cuda.synchronize()
    api.kernel_trace()
    st.run()
    st.run()
    torch.cuda.synchronize()
    ev = api.kernel_trace()
    ev = ev[len(ev) // 2:] + [ev[-1]]                       # the second of the two steps
    rows = collections.OrderedDict()
    for a, b in zip(ev[:-1], ev[1:]):
        rows.setdefault((a[1], int(a[2]), int(a[3])), []).append((b[0] - a[0]) / 1e3)
    layers = len(model.spec.layers)
    print(f"decode step at batch {batch}, {layers} layers: {(ev[-1][0] - ev[0][0]) / 1e3:.1f} us, {len(ev) - 1} launches")
    for (src, grid, block), v in rows.items():
        print(f"  {src:22s} {grid:6d} x {block:4d}  launches {len(v):4d}  mean {sum(v) / len(v):7.2f} us  total {sum(v):8.1f} us")
    print("  first layer in order: " + "  ".join(f"{a[1].split('.')[0]}:{(b[0] - a[0]) / 1e3:.1f}" for a, b in list(zip(ev[:-1], ev[1:]))[:10]))
    backend.finish()
    return 0


def time_prefill(torch, dk, model, tokens, iters=3):
    import numpy as np
    runner = dk.Runner(model, tokens + 64, max_slots=2)
    prompt = np.random.RandomState(7).randint(0, model.spec.vocab_size, tokens).tolist()
    times = []
    for i in range(iters + 1):
        slot = runner.begin()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([(slot, prompt, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        runner.end(slot)
        if i:
            times.append(e0.elapsed_time(e1))
    s = model.spec
    m = s.layers[0].mixer
    per_layer = (m.num_heads + 2 * m.num_kv_heads) * m.head_dim * s.hidden_size + s.hidden_size * m.num_heads * m.head_dim \
        + 3 * s.layers[0].feed_forward.intermediate_size * s.hidden_size
    L = len(s.layers)
    flops = 2 * per_layer * L * tokens + 4 * m.num_heads * m.head_dim * tokens * (tokens + 1) / 2 * L + 2 * s.vocab_size * s.hidden_size
    del runner
    torch.cuda.empty_cache()
    return statistics.median(times), flops


def time_e2e(torch, dk, model, batch, steps, seed):
    """Decode tokens per second through Engine.generate: host lists in, host tokens out, from the
    first yielded step (end of prefill) to the last."""
    import numpy as np
    lens = ragged_lengths(batch, seed)
    rs = np.random.RandomState(seed + 1)
    prompts = [rs.randint(0, model.spec.vocab_size, n).tolist() for n in lens]
    eng = dk.Engine(model=model)
    list(eng.generate(prompts, 4))          # first call: allocations and the graph of this batch shape (kept by the engine)
    t_first = None
    n = 0
    for row in eng.generate(prompts, steps + 1):
        if t_first is None:
            t_first = time.perf_counter()
        n += 1
    t_last = time.perf_counter()
    h2d = sum(len(p) for p in prompts) * 3 * 4 / (steps + 1)              # token ids, row->sequence, positions, once
    del eng
    torch.cuda.empty_cache()
    return batch * (n - 1) / (t_last - t_first), h2d, 4 * batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=48,
                    help="untimed steps before the timed ones; the default outlasts the tens of milliseconds the SM clock "
                         "takes to come back after the power-capped prefill")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--prefill-only", action="store_true", help="only the 2,048-token prefill (for profiling its kernels)")
    ap.add_argument("--prefill-tokens", type=int, default=PROMPT, help="with --prefill-only: a prompt of another length")
    ap.add_argument("--timeline", action="store_true",
                    help="print where one decode step's time goes inside the graph (kernels built with start notes) and exit")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch on (1) or off (0)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a folder of scripts without setup.py or pyproject.toml: pip cannot install "
                          "it into baseline/_ref ('Neither setup.py nor pyproject.toml found')"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs one model on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    if args.timeline:
        os.environ["DRYFT_KERNEL_TRACE"] = "1"     # read when the package's kernels are built and loaded

    import torch

    import dryft_challenge_htn_2026_b200 as dk
    from dryft_challenge_htn_2026_b200.csrc import api

    cfg_d = dict(QWEN3_4B)
    full_layers = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    cfg = dk.config_from_dict(cfg_d)
    api.set_pdl(bool(args.pdl))
    model = dk.random_model(cfg, seed=0, dtype=torch.bfloat16)
    pk = peaks()

    if args.timeline:
        return timeline(torch, dk, api, model, args.batch)
    if args.prefill_only:
        ms, flops = time_prefill(torch, dk, model, args.prefill_tokens)
        print(json.dumps({"prefill": {"value": round(args.prefill_tokens / ms * 1e3, 1), "tokens": args.prefill_tokens, "ms": round(ms, 3),
                                      "layers": cfg.num_hidden_layers,
                                      "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    main_run = time_decode(torch, dk, model, args.batch, args.steps, warmup, seed=0)
    e2e_val, h2d, d2h = time_e2e(torch, dk, model, args.batch, args.steps, seed=0)
    points, prefill = {}, None
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(time_decode(torch, dk, model, b, max(16, args.steps // 2), warmup, seed=b)["tok_s"], 1)
        ms, flops = time_prefill(torch, dk, model, PROMPT)
        prefill = {"value": round(PROMPT / ms * 1e3, 1), "tokens": PROMPT, "ms": round(ms, 3),
                   "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-4B, bf16)", "value": round(main_run["tok_s"], 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": "Qwen3-4B layer sizes", "global_batch": args.batch, "seq_len": CONTEXT, "parallelism": "1gpu",
                   "layers": cfg.num_hidden_layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": True,
                   "prompt_len": "2048 (1024..2048 ragged above batch 1)", "ctx_mean_timed": round(main_run["ctx_mean"]),
                   "l2": "inputs larger than L2 (8 GB of weights per step)", "pdl": bool(args.pdl),
                   "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "e2e": {"value": round(e2e_val, 1), "unit": "tok/s", "h2d_bytes_per_step": round(h2d), "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        out["prefill"] = prefill
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
