"""Command line in the manner of the reference's tests/bench.py (lines 18-26, 104-167):

    python -m dryft_challenge_htn_2026_b200.cli --model DIR [--shapes 1,512,32 4,2048,32 16,512,128]
           [--samples 5] [--no-check] [--check-all] [--dtype bfloat16] [--temperature 0] [--seed 0]
           [--ragged] [--random-weights CONFIG.json]

Same option names and meanings where the reference has them: ``--model`` (model folder),
``--shapes B,S,n`` (batch, prompt length, new tokens), ``--samples`` (timed runs per shape, after
one warm-up run of the same shape), ``--no-check``, ``--check-all`` (check every sample, not only
the first). Prompts are uniform random token ids in [1000, 100000) clipped to the vocabulary (the
reference's ``--random`` mode; its text corpora need a tokenizer, which this library does not
have). Per shape it prints median tok/s = B*n / total seconds (prefill included, as the reference
counts), TTFT, TPOT = (median total - median TTFT) / (n - 1), spread, peak memory and the decode
step's share of the HBM roofline. The check replays prompt + emitted tokens through this
library's true float32 path and reports the worst gap between the best logit and the emitted
token's logit; like the reference it fails above 2.0 logits (greedy runs only).
"""
import argparse
import json
import statistics
import sys
import time

import torch


def prompts(batch, length, seed, vocab, ragged):
    g = torch.Generator().manual_seed(seed)
    hi = min(100000, vocab)
    lo = min(1000, hi - 1)
    lens = [length] * batch
    if ragged and batch > 1:
        lens = torch.randint(max(1, length // 2), length + 1, (batch,), generator=g).tolist()
    return [torch.randint(lo, hi, (n,), generator=g).tolist() for n in lens]


def run(eng, ids, n, temperature, seed):
    t0 = time.perf_counter()
    out, first = [], None
    for step in eng.generate(ids, n, temperature=temperature, seed=seed):
        if first is None:
            torch.cuda.synchronize()
            first = time.perf_counter() - t0
        out.append(step)
    return time.perf_counter() - t0, first, out


def check(oracle, ids, out):
    """Worst (best logit - emitted token's logit) over all emitted tokens, from one float32 pass
    over prompt + emitted tokens per sequence."""
    from .engine import Runner

    worst = 0.0
    need = max(len(p) + len(out) for p in ids) + 64
    runner = Runner(oracle, need, max_slots=1)
    for b, p in enumerate(ids):
        emitted = [s[b] for s in out if s[b] is not None]
        slot = runner.begin()
        seq = list(p) + emitted[:-1]
        logits = runner.step([(slot, seq, list(range(len(p) - 1, len(seq))))])
        runner.end(slot)
        picked = logits.gather(1, torch.tensor(emitted, device=logits.device).view(-1, 1)).squeeze(1)
        worst = max(worst, float((logits.max(-1).values - picked).max()))
    return worst


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", help="model folder (config.json + safetensors)")
    ap.add_argument("--random-weights", metavar="CONFIG", help="config.json to build with random weights instead of --model")
    ap.add_argument("--shapes", nargs="*", default=["1,512,32", "4,2048,32", "16,512,128"])
    ap.add_argument("--samples", type=int, default=5)
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--check-all", action="store_true", help="check every sample")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ragged", action="store_true", help="prompt lengths uniform in [S/2, S] instead of all S")
    args = ap.parse_args(argv)
    if bool(args.model) == bool(args.random_weights):
        ap.error("give exactly one of --model and --random-weights")

    from . import Engine, config_from_dict, load_model, random_model
    from .config.base import read_config_json

    t0 = time.time()
    if args.model:
        model = load_model(args.model, args.dtype)
        oracle_of = lambda: load_model(args.model, "float32")
    else:
        cfg = config_from_dict(read_config_json(args.random_weights))
        model = random_model(cfg, args.seed, args.dtype)
        oracle_of = lambda: random_model(cfg, args.seed, "float32")
    eng = Engine(model=model)
    torch.cuda.synchronize()
    print(f"load+init {time.time() - t0:.1f}s", flush=True)
    vocab = model.spec.vocab_size
    kv_per_token = sum(r.n_kv_heads * r.head_dim * 2 * 2 for rs in model.entry_requests() for r in rs if hasattr(r, "n_kv_heads"))
    try:
        with open("MEASURED_PEAKS.json") as f:
            hbm = float(json.load(f)["hbm_gbs"]) * 1e9
    except Exception:
        hbm = 6650e9
    oracle, results = None, []
    for spec in args.shapes:
        B, S, n = map(int, spec.split(","))
        run(eng, prompts(B, S, 0, vocab, args.ragged), n, args.temperature, args.seed)          # warm-up, same shape
        ts, tf, outs = [], [], []
        torch.cuda.reset_peak_memory_stats()
        for k in range(args.samples):
            ids = prompts(B, S, k + 1, vocab, args.ragged)
            total, first, out = run(eng, ids, n, args.temperature, args.seed)
            assert len(out) == n and all(len(x) == B for x in out)
            ts.append(total), tf.append(first), outs.append((ids, out))
        med, ttft = statistics.median(ts), statistics.median(tf)
        tpot = (med - ttft) / max(n - 1, 1)
        floor = (model.weight_bytes_per_step() + B * (S + n / 2) * kv_per_token) / hbm
        print(f"B{B} {S}->{n}: {B * n / med:8.1f} tok/s  total {med * 1e3:7.1f} ms  ttft {ttft * 1e3:6.1f} ms  "
              f"tpot {tpot * 1e3:5.2f} ms  spread {(max(ts) - min(ts)) / med * 100:4.1f}%  "
              f"mem {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB  roofline {100 * floor / max(tpot, 1e-9):.0f}%", flush=True)
        results.append(B * n / med)
        if not args.no_check and args.temperature == 0:
            oracle = oracle or oracle_of()
            worst = max(check(oracle, ids, out) for ids, out in (outs if args.check_all else outs[:1]))
            print(f"   correctness: worst gap {worst:.3f} logits vs the float32 path", flush=True)
            assert worst <= 2.0, f"{spec}: generated tokens exceeded the 2-logit tolerance"
    gm = 1.0
    for r in results:
        gm *= r
    if results:
        print(f"geomean {gm ** (1 / len(results)):.1f} tok/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
