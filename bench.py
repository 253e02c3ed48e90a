"""Decode and prefill throughput of Qwen3 layer sizes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--size 4b|8b|14b] [--batch 8] [--layers N]
                    [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at the default batch of 8: K decode
steps of the generation loop's own decode state (CUDA-graph replay), timed with CUDA events after W
warm-up steps (at least 32 untimed steps in both arms, see MIN_UNTIMED_STEPS; the count is named in
``config.untimed_steps``), every sequence at the midpoint of the size's workload: for ``4b`` a 2,048-token
prompt (ragged 1,024..2,048 above batch 1) plus 1,024 tokens decoded so far of a 4,096-token
context; ``8b`` 1,024 + 512 of 1,024; ``14b`` 2,048 + 256 of 512. ``e2e`` is the same measured
through ``Engine.generate`` (host token lists in, host tokens out). ``prefill`` is one 2,048-token
prompt; ``roofline`` relates the decode step to the bytes it must read; ``points`` hold the size's
other two batch sizes, each with its own step time, roofline fraction and clocks. The weights (8 to
28 GB) are far larger than L2, so no flush is needed between steps. For more than one GPU it says
so and exits with 2: this library runs on one.

``--impl reference`` times the unmodified reference engine (a copy of its folder under
``baseline/_ref``) through its own ``Engine(model_path)`` and ``Engine.generate`` on a model folder
of the same sizes written here with plain torch; nothing of this library is imported on that arm.
"""
import argparse
import contextlib
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_COMMON = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, num_key_value_heads=8, head_dim=128,
               rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960)
# layer sizes, and the workload each is quoted on: prompt length (ragged from half of it above batch 1 where
# `ragged`), decode steps of the whole run (timed at their midpoint), batch sizes
SIZES = {
    "4b": dict(config=dict(_COMMON, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                           num_attention_heads=32, tie_word_embeddings=True),
               name="Qwen3-4B", prompt=2048, ragged=True, decode=2048, batches=(1, 8, 64)),
    "8b": dict(config=dict(_COMMON, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                           num_attention_heads=32, tie_word_embeddings=False),
               name="Qwen3-8B", prompt=1024, ragged=False, decode=1024, batches=(1, 8, 64)),
    "14b": dict(config=dict(_COMMON, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40,
                            num_attention_heads=40, tie_word_embeddings=False),
                name="Qwen3-14B", prompt=2048, ragged=False, decode=512, batches=(1, 8, 32)),
}
PREFILL_TOKENS = 2048
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


def prompt_lengths(size, batch, seed):
    """Context each sequence holds when the timed steps begin: its prompt plus half of the run's decode steps."""
    import numpy as np
    w = SIZES[size]
    so_far = w["decode"] // 2
    if batch == 1 or not w["ragged"]:
        return [w["prompt"] + so_far] * batch
    r = np.random.RandomState(seed)
    return [int(x) + so_far for x in r.randint(w["prompt"] // 2, w["prompt"] + 1, batch)]


def random_prompts(vocab, lens, seed):
    import numpy as np
    rs = np.random.RandomState(seed + 1)
    return [rs.randint(0, vocab, n).tolist() for n in lens]


def kv_bytes_per_token(cfg):
    return cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def weight_bytes(cfg):
    """Bytes of bfloat16 weights a decode step reads: every matrix once, the head once (the embedding is
    read by row only, so it counts only where it is also the head)."""
    H, hd = cfg["hidden_size"], cfg["head_dim"]
    per_layer = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * hd * H + H * cfg["num_attention_heads"] * hd \
        + 3 * cfg["intermediate_size"] * H
    return 2 * (per_layer * cfg["num_hidden_layers"] + cfg["vocab_size"] * H)


def prefill_flops(cfg, tokens):
    H, hd, nh = cfg["hidden_size"], cfg["head_dim"], cfg["num_attention_heads"]
    per_layer = (nh + 2 * cfg["num_key_value_heads"]) * hd * H + H * nh * hd + 3 * cfg["intermediate_size"] * H
    L = cfg["num_hidden_layers"]
    return 2 * per_layer * L * tokens + 4 * nh * hd * tokens * (tokens + 1) / 2 * L + 2 * cfg["vocab_size"] * H


# ------------------------------------------------------------------------------------ this library
# Untimed steps before the timed ones: the W asked for, and at least this many, in both arms (after a
# prefill under the power cap the SM clock needs some tens of steps to settle; with five untimed steps
# the same step measured 5 % slower than with fifty). The count used is named in config.untimed_steps.
MIN_UNTIMED_STEPS = 32


def time_decode(torch, dk, model, cfg, size, batch, steps, warmup, seed):
    """K decode steps of the generation loop's own decode state (graph replay), timed on the device
    after ``warmup`` untimed ones."""
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.generate import GpuBackend
    from dryft_challenge_htn_2026_b200.sampling import SamplingParams

    lens = prompt_lengths(size, batch, seed)
    total_new = warmup + steps + 8
    need = sum((n + total_new + 63) // 64 * 64 for n in lens)
    runner = dk.Runner(model, need, max_slots=max(batch, 1))
    backend = GpuBackend(runner, use_graph=True)
    prompts = random_prompts(model.spec.vocab_size, lens, seed)
    backend.start(prompts, SamplingParams(total_new), [0] * batch).wait()    # prefill (steps of at most 32k tokens), first token
    st = backend.state
    count0 = api.launch_count()
    st.body(advance=False, out_tok=torch.empty_like(st.ctx.tok))
    launches_per_step = api.launch_count() - count0
    st.capture()
    for _ in range(warmup):
        st.run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    with ClockSampler() as cs:
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(steps):
            st.run()
        ev[1].record()
        torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / steps
    ctx_mean = sum(lens) / batch + warmup + steps / 2
    step_bytes = model.weight_bytes_per_step() + batch * ctx_mean * kv_bytes_per_token(cfg)
    backend.finish()
    del st, backend, runner
    torch.cuda.empty_cache()
    return dict(ms=ms, tok_s=batch / ms * 1e3, bytes=step_bytes, ctx_mean=ctx_mean, launches=launches_per_step,
                clocks=cs.summary())


def time_prefill(torch, dk, model, cfg, tokens, iters=3):
    """One prompt of ``tokens`` tokens through the step function as generation calls it (a step shape
    that repeats is replayed as a CUDA graph): two untimed runs (plain, then the capture), then the
    median of ``iters`` runs, each between synchronisations, timed with CUDA events."""
    import numpy as np
    runner = dk.Runner(model, tokens + 64, max_slots=2)
    prompt = np.random.RandomState(7).randint(0, model.spec.vocab_size, tokens).tolist()
    times = []
    for i in range(iters + 2):
        slot = runner.begin()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([(slot, prompt, [tokens - 1])], graph=True)
        e1.record()
        torch.cuda.synchronize()
        runner.end(slot)
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    del runner
    torch.cuda.empty_cache()
    return statistics.median(times), prefill_flops(cfg, tokens)


def time_e2e(torch, dk, model, size, batch, steps, warmup, seed):
    """Decode tokens per second through Engine.generate: host lists in, host tokens out; wall clock at
    each yield, the timed steps those between yield number ``warmup`` and yield ``warmup + steps`` of
    one call (what the reference arm's number is, see ref_decode)."""
    lens = prompt_lengths(size, batch, seed)
    prompts = random_prompts(model.spec.vocab_size, lens, seed)
    eng = dk.Engine(model=model)
    list(eng.generate(prompts, 4))          # first call: allocations and the graph of this batch shape (kept by the engine)
    stamps = [time.perf_counter() for _ in eng.generate(prompts, warmup + steps + 1)]
    assert len(stamps) == warmup + steps + 1
    h2d = sum(len(p) for p in prompts) * 3 * 4 / (warmup + steps + 1)     # token ids, row->sequence, positions, once
    del eng
    torch.cuda.empty_cache()
    return batch * steps / (stamps[warmup + steps] - stamps[warmup]), h2d, 4 * batch


def point(run, pk):
    achieved = run["bytes"] / (run["ms"] * 1e-3) / 1e9
    return {"value": round(run["tok_s"], 1), "ms_per_step": round(run["ms"], 4), "ctx_mean": round(run["ctx_mean"]),
            "roofline_frac": round(achieved / pk["hbm_gbs"], 4), "clocks": run["clocks"]}


def config_record(size, cfg, layers_full, batch, pk, **more):
    w = SIZES[size]
    rec = {"model": f"{w['name']} layer sizes", "global_batch": batch, "seq_len": w["prompt"] + w["decode"],
           "parallelism": "1gpu", "layers": cfg["num_hidden_layers"], "layers_full": layers_full,
           "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
           "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
           "tied_head": bool(cfg["tie_word_embeddings"]),
           "prompt_len": f"{w['prompt']}" + (f" ({w['prompt'] // 2}..{w['prompt']} ragged above batch 1)" if w["ragged"] else ""),
           "l2": "inputs larger than L2 (GBs of weights per step)", "peaks": pk["source"]}
    rec.update(more)
    return rec


def run_ours(args):
    import torch

    import dryft_challenge_htn_2026_b200 as dk
    from dryft_challenge_htn_2026_b200.csrc import api

    size = args.size
    cfg_d = dict(SIZES[size]["config"])
    full_layers = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    cfg = dk.config_from_dict(cfg_d)
    api.set_pdl(bool(args.pdl))
    model = dk.random_model(cfg, seed=0, dtype=torch.bfloat16)
    pk = peaks()
    warmup = max(3, args.warmup)

    if args.prefill_only:
        ms, flops = time_prefill(torch, dk, model, cfg_d, args.prefill_tokens)
        print(json.dumps({"prefill": {"value": round(args.prefill_tokens / ms * 1e3, 1), "tokens": args.prefill_tokens,
                                      "ms": round(ms, 3), "layers": cfg.num_hidden_layers,
                                      "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    untimed = max(warmup, MIN_UNTIMED_STEPS)
    main_run = time_decode(torch, dk, model, cfg_d, size, args.batch, args.steps, untimed, seed=0)
    e2e_val, h2d, d2h = time_e2e(torch, dk, model, size, args.batch, args.steps, untimed, seed=0)
    points, detail, prefill = {}, {}, None
    if not args.no_points:
        for b in SIZES[size]["batches"]:
            if b != args.batch:
                detail[f"decode_b{b}"] = point(time_decode(torch, dk, model, cfg_d, size, b, max(64, args.steps), untimed, seed=b), pk)
                points[f"decode_b{b}"] = detail[f"decode_b{b}"]["value"]
        ms, flops = time_prefill(torch, dk, model, cfg_d, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                   "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                   "short_ms": {str(n): round(time_prefill(torch, dk, model, cfg_d, n)[0], 3) for n in (128, 512)}}
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({SIZES[size]['name']}, bf16)", "value": round(main_run["tok_s"], 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": config_record(size, cfg_d, full_layers, args.batch, pk, ctx_mean_timed=round(main_run["ctx_mean"]),
                                pdl=bool(args.pdl), untimed_steps=untimed),
        "clocks": main_run["clocks"],
        "e2e": {"value": round(e2e_val, 1), "unit": "tok/s", "h2d_bytes_per_step": round(h2d), "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        out["prefill"] = prefill
        out["points"] = points
        out["points_detail"] = detail
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------------------ the reference arm
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
# The reference's own switches (engine/engine.py:31,98; engine/fused.py:19), set in the environment before it
# is imported. Speculative decoding and fp8 prefill products are not part of the metric (plain bf16 decoding).
# ENGINE_PDL=0: the reference patches the C launcher that Triton 3.1 generates; with the Triton of this image
# the patched text is not found, every fused kernel then fails to compile (AssertionError) and its self-test
# falls back to its torch ops, 5 times slower. Without the patch its fused Triton ops pass their self-test.
REF_ENV = {"ENGINE_SPEC": "0", "ENGINE_FP8": "0", "ENGINE_PDL": "0"}


def reference_source():
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            return json.load(f).get("reference_path") or ""
    except Exception:
        return ""


def install_reference():
    """baseline/_ref: an unmodified copy of the reference's folder (it has no setup.py or pyproject.toml
    for pip to install). Returns None, or the reason it is not there."""
    if os.path.isfile(os.path.join(REF_DIR, "engine", "engine.py")):
        return None
    src = os.environ.get("DRYFT_REFERENCE") or reference_source()
    if not src or not os.path.isfile(os.path.join(src, "engine", "engine.py")):
        return f"no copy of the reference under baseline/_ref and no source folder to copy it from ({src or 'none named'})"
    os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
    shutil.copytree(src, REF_DIR, ignore=shutil.ignore_patterns(".git", "__pycache__"))
    return None


def write_model_folder(torch, cfg, folder, seed=0, dev="cuda"):
    """config.json (rope_theta at the top level, as the reference reads it) and one safetensors file per
    layer with the checkpoint names of Qwen3ForCausalLM; matrices N(0, 0.02), norm weights 1 + N(0, 0.1)."""
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(cfg, model_type="qwen3", hidden_act="silu", attention_bias=False), f)
    gen = torch.Generator(device=dev).manual_seed(seed)
    H, hd, I, V = cfg["hidden_size"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    mat = lambda *s: (0.02 * torch.randn(s, generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16).cpu()
    nrm = lambda n: (1.0 + 0.1 * torch.randn(n, generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16).cpu()
    top = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": nrm(H)}
    if not cfg["tie_word_embeddings"]:
        top["lm_head.weight"] = mat(V, H)
    save_file(top, os.path.join(folder, "model-top.safetensors"))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        save_file({p + "input_layernorm.weight": nrm(H), p + "post_attention_layernorm.weight": nrm(H),
                   p + "self_attn.q_norm.weight": nrm(hd), p + "self_attn.k_norm.weight": nrm(hd),
                   p + "self_attn.q_proj.weight": mat(nh * hd, H), p + "self_attn.k_proj.weight": mat(nkv * hd, H),
                   p + "self_attn.v_proj.weight": mat(nkv * hd, H), p + "self_attn.o_proj.weight": mat(H, nh * hd),
                   p + "mlp.gate_proj.weight": mat(I, H), p + "mlp.up_proj.weight": mat(I, H),
                   p + "mlp.down_proj.weight": mat(H, I)}, os.path.join(folder, f"model-layer{i:03d}.safetensors"))


def ref_decode(torch, eng, prompts, steps, warmup, sample_clocks=False):
    """Decode steps of the reference's generator, as its tests/bench.py:104-111 times a run: wall clock at
    each yield; the timed steps are those between yield number ``warmup`` and yield ``warmup + steps``."""
    stamps = []
    gen = eng.generate(prompts, warmup + steps + 1)
    cs = ClockSampler() if sample_clocks else contextlib.nullcontext()
    with cs:
        for _ in gen:
            stamps.append(time.perf_counter())
    assert len(stamps) == warmup + steps + 1
    ms = (stamps[warmup + steps] - stamps[warmup]) / steps * 1e3
    return ms, (cs.summary() if sample_clocks else None)


def run_reference(args):
    why = install_reference()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    os.environ.update({k: os.environ.get(k, v) for k, v in REF_ENV.items()})
    real_stdout = sys.stdout
    sys.stdout = sys.stderr                       # the reference prints its self-test results; the JSON line stays alone
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        sys.path.insert(0, os.path.join(REF_DIR, "engine"))
        from engine import Engine                 # the reference's engine/engine.py, unmodified

        size = args.size
        w = SIZES[size]
        cfg = dict(w["config"])
        full_layers = cfg["num_hidden_layers"]
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        pk = peaks()
        warmup = max(3, args.warmup)
        untimed = max(warmup, MIN_UNTIMED_STEPS)
        folder = tempfile.mkdtemp(prefix="dryft_ref_model_")
        try:
            t0 = time.time()
            write_model_folder(torch, cfg, folder)
            print(f"[bench] model folder written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
            t0 = time.time()
            eng = Engine(folder)                  # loads, self-tests its fused ops against its torch ops, picks a back end
            print(f"[bench] reference engine ready in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        backend = type(eng.ops).__name__
        import fused
        backend += f" (PDL {'on' if getattr(fused, 'PDL', False) else 'off'})"
        V = cfg["vocab_size"]

        def decode_point(batch, equal, steps, seed, clocks=False):
            lens = prompt_lengths(size, batch, seed)
            if equal:
                lens = [max(lens)] * batch
            ms, c = ref_decode(torch, eng, random_prompts(V, lens, seed), steps, untimed, clocks)
            ctx_mean = sum(lens) / batch + untimed + steps / 2
            nbytes = weight_bytes(cfg) + batch * ctx_mean * kv_bytes_per_token(cfg)
            return dict(ms=ms, tok_s=batch / ms * 1e3, bytes=nbytes, ctx_mean=ctx_mean, clocks=c)

        decode_point(args.batch, False, 4, seed=0)                      # compiles what this shape needs
        main_run = decode_point(args.batch, False, args.steps, seed=0, clocks=True)
        points, detail, prefill = {}, {}, None
        if not args.no_points:
            psteps = max(16, min(64, args.steps))
            if w["ragged"] and args.batch > 1:
                # the reference runs a ragged batch as one stream per prompt length (engine/engine.py:1093-1105);
                # with equal lengths the same batch is one stream
                detail[f"decode_b{args.batch}_equal_lengths"] = point(decode_point(args.batch, True, psteps, seed=0, clocks=True), pk)
            for b in w["batches"]:
                if b != args.batch:
                    equal = b > 8                  # 64 streams of one sequence each would only measure batch 1 again
                    key = f"decode_b{b}" + ("_equal_lengths" if equal and w["ragged"] else "")
                    detail[key] = point(decode_point(b, equal, psteps, seed=b, clocks=True), pk)
            points = {k: v["value"] for k, v in detail.items()}
            prompt = random_prompts(V, [PREFILL_TOKENS], 6)
            times = []
            for i in range(4):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in eng.generate(prompt, 1):
                    pass
                torch.cuda.synchronize()
                if i:
                    times.append((time.perf_counter() - t0) * 1e3)
            ms = statistics.median(times)
            prefill = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                       "frac": round(prefill_flops(cfg, PREFILL_TOKENS) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                       "how": "wall clock of generate(prompt, 1), the reference's TTFT"}
        achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
        lens = prompt_lengths(size, args.batch, 0)
        out = {
            "impl": "reference",
            "metric": f"decode tok/s at batch {args.batch} ({w['name']}, bf16)", "value": round(main_run["tok_s"], 1),
            "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: random weights N(0,0.02), uniform random token ids",
            "config": config_record(size, cfg, full_layers, args.batch, pk, ctx_mean_timed=round(main_run["ctx_mean"]),
                                    reference_backend=f"{backend}, {len(set(lens))} streams",
                                    reference_env=" ".join(f"{k}={os.environ[k]}" for k in sorted(REF_ENV)),
                                    untimed_steps=untimed),
            "clocks": main_run["clocks"],
            # the reference's only interface is the host-side generator: host token lists in, host tokens out;
            # value and e2e are the same measurement (wall clock between yields)
            "e2e": {"value": round(main_run["tok_s"], 1), "unit": "tok/s",
                    "h2d_bytes_per_step": round(sum(lens) * 8 / (untimed + args.steps + 1)), "d2h_bytes_per_step": 8 * args.batch},
            "gpu_launches": None,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
        }
        if prefill is not None:
            out["prefill"] = prefill
            out["points"] = points
            out["points_detail"] = detail
    except Exception as e:                         # the arm reports, it does not fail the round
        import traceback
        traceback.print_exc(file=sys.stderr)
        out = {"impl": "reference", "unavailable": f"the reference engine did not run here: {type(e).__name__}: {str(e)[:300]}"}
    finally:
        sys.stdout = real_stdout
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=48,
                    help="untimed steps before the timed ones; the default outlasts the tens of milliseconds the SM clock "
                         "takes to come back after the power-capped prefill")
    ap.add_argument("--size", default="4b", choices=sorted(SIZES), help="layer sizes and workload (default: Qwen3-4B)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the other batch sizes and the prefill")
    ap.add_argument("--prefill-only", action="store_true", help="only the 2,048-token prefill (for profiling its kernels)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --prefill-only: a prompt of another length")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch on (1) or off (0)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs one model on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
