"""Command line in the manner of the reference's tests/bench.py (its options: lines 18-26; what it
measures: lines 104-140; its check: lines 144-167):

    python -m dryft_challenge_htn_2026_b200.cli --model DIR [--shapes 1,512,32 4,2048,32 16,512,128]
           [--samples 5] [--no-check] [--check-all] [--dtype bfloat16] [--temperature 0] [--seed 0]
           [--ragged] [--random-weights CONFIG.json [--save-model DIR]] [--print-tokens] [--json]

Same option names and meanings where the reference has them: ``--model`` (model folder),
``--shapes B,S,n`` (batch, prompt length, new tokens), ``--samples`` (timed runs per shape, after
one untimed run of the same shape), ``--no-check``, ``--check-all`` (check every sample, not only
the first). Prompts are uniform random token ids in [1000, 100000) clipped to the vocabulary (the
reference's ``--random`` mode; its text corpora need a tokenizer, which this library does not
have). Per shape it reports what the reference reports: tok/s = B*n / median total seconds
(prefill included), TTFT (time to the first step's tokens), TPOT = (median total - median TTFT) /
(n - 1), the spread of the totals, peak memory, and TPOT against the time the step's bytes take at
the measured HBM bandwidth. The check replays prompt + emitted tokens through this library's true
float32 path and reports the worst gap between the best logit and the emitted token's logit; like
the reference it fails above 2.0 logits (greedy runs only), and it fails on logits that are not
finite. ``--print-tokens`` prints the first sample's tokens, one line per sequence; ``--json``
prints one JSON record per shape instead of the text line.
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

GAP_LIMIT = 2.0          # logits; the reference's bound (tests/bench.py:144-167)


class CheckFailed(RuntimeError):
    pass


def random_prompts(batch, length, seed, vocab, ragged):
    """Token ids uniform in [1000, 100000) where the vocabulary has them, else in all of it."""
    g = torch.Generator().manual_seed(seed)
    hi = min(100000, vocab)
    lo = 1000 if hi > 2000 else 0
    lens = [length] * batch
    if ragged and batch > 1:
        lens = torch.randint(max(1, length // 2), length + 1, (batch,), generator=g).tolist()
    return [torch.randint(lo, hi, (n,), generator=g).tolist() for n in lens]


def timed_generation(eng, prompts, n, temperature, seed):
    """(total seconds, seconds to the first step, tokens per sequence) of one call of Engine.generate."""
    per_seq = [[] for _ in prompts]
    start = time.perf_counter()
    first = None
    for step in eng.generate(prompts, n, temperature=temperature, seed=seed):
        if first is None:
            first = time.perf_counter() - start
        for seq, tok in zip(per_seq, step):
            if tok is not None:
                seq.append(tok)
    return time.perf_counter() - start, first, per_seq


def teacher_forced_gap(oracle_runner, prompt, emitted):
    """Largest (best logit - logit of the emitted token) over the emitted tokens, from one float32
    pass over prompt + emitted tokens."""
    slot = oracle_runner.begin()
    try:
        seq = list(prompt) + list(emitted[:-1])
        logits = oracle_runner.step([(slot, seq, list(range(len(prompt) - 1, len(seq))))])
    finally:
        oracle_runner.end(slot)
    if not bool(torch.isfinite(logits).all()):
        raise CheckFailed("the float32 replay gives logits that are not finite (a NaN or infinity in the weights?)")
    picked = logits.gather(1, torch.tensor(emitted, device=logits.device).view(-1, 1)).squeeze(1)
    return float((logits.max(-1).values - picked).max())


def measure_shape(eng, shape, args, hbm_bytes_per_s):
    """Runs one B,S,n shape: an untimed run, then ``args.samples`` timed ones on fresh prompts.
    Returns the record that is printed, and the samples (prompts, tokens) for the check."""
    model = eng.model
    batch, length, n = shape
    vocab = model.spec.vocab_size
    timed_generation(eng, random_prompts(batch, length, 0, vocab, args.ragged), n, args.temperature, args.seed)
    torch.cuda.reset_peak_memory_stats()
    totals, firsts, samples = [], [], []
    for k in range(args.samples):
        prompts = random_prompts(batch, length, k + 1, vocab, args.ragged)
        total, first, tokens = timed_generation(eng, prompts, n, args.temperature, args.seed)
        if any(len(t) != n for t in tokens):
            raise CheckFailed(f"{batch},{length},{n}: a sequence returned {min(map(len, tokens))} tokens instead of {n}")
        totals.append(total), firsts.append(first), samples.append((prompts, tokens))
    total, ttft = statistics.median(totals), statistics.median(firsts)
    tpot = (total - ttft) / max(n - 1, 1)
    kv_per_token = sum(r.n_kv_heads * r.head_dim * 2 * r.dtype.itemsize for rs in model.entry_requests() for r in rs
                       if hasattr(r, "n_kv_heads"))
    mean_context = sum(len(p) for p in samples[0][0]) / batch + n / 2
    floor = (model.weight_bytes_per_step() + batch * mean_context * kv_per_token) / hbm_bytes_per_s
    record = {"shape": f"{batch},{length},{n}", "tok_s": batch * n / total, "total_ms": total * 1e3, "ttft_ms": ttft * 1e3,
              "tpot_ms": tpot * 1e3, "spread_pct": (max(totals) - min(totals)) / total * 100,
              "peak_gib": torch.cuda.max_memory_allocated() / 2 ** 30, "roofline_pct": 100 * floor / max(tpot, 1e-9)}
    return record, samples


def text_line(r):
    return (f"B{r['shape'].split(',')[0]} {r['shape'].split(',')[1]}->{r['shape'].split(',')[2]}: {r['tok_s']:8.1f} tok/s  "
            f"total {r['total_ms']:7.1f} ms  ttft {r['ttft_ms']:6.1f} ms  tpot {r['tpot_ms']:5.2f} ms  "
            f"spread {r['spread_pct']:4.1f}%  mem {r['peak_gib']:.1f} GiB  roofline {r['roofline_pct']:.0f}%")


def measured_hbm_bandwidth():
    """Bytes per second from MEASURED_PEAKS.json beside the package (written by the machine's
    set-up), else an earlier measurement on the same kind of GPU."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]) * 1e9
    except Exception:
        return 6650e9


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", help="model folder (config.json + safetensors)")
    ap.add_argument("--random-weights", metavar="CONFIG", help="config.json to build with random weights instead of --model")
    ap.add_argument("--save-model", metavar="DIR", help="with --random-weights: write the model folder there and load it from it")
    ap.add_argument("--shapes", nargs="*", default=["1,512,32", "4,2048,32", "16,512,128"])
    ap.add_argument("--samples", type=int, default=5)
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--check-all", action="store_true", help="check every sample")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ragged", action="store_true", help="prompt lengths uniform in [S/2, S] instead of all S")
    ap.add_argument("--print-tokens", action="store_true", help="print the tokens of each shape's first sample")
    ap.add_argument("--json", action="store_true", help="one JSON record per shape instead of the text line")
    args = ap.parse_args(argv)
    if bool(args.model) == bool(args.random_weights):
        ap.error("give exactly one of --model and --random-weights")
    if args.save_model and not args.random_weights:
        ap.error("--save-model goes with --random-weights")
    shapes = [tuple(int(x) for x in s.split(",")) for s in args.shapes]
    if any(len(s) != 3 or min(s) < 1 for s in shapes) or args.samples < 1:
        ap.error("--shapes takes B,S,n triples of positive numbers, --samples at least 1")

    from . import Engine, Runner, config_from_dict, load_model, random_model, write_random_model
    from .config.base import read_config_json

    t0 = time.time()
    folder = args.model
    if args.random_weights:
        config = config_from_dict(read_config_json(args.random_weights))
        if args.save_model:
            folder = write_random_model(config, args.save_model, seed=args.seed, dtype=torch.float32)
    if folder:
        model, make_oracle = load_model(folder, args.dtype), lambda: load_model(folder, "float32")
    else:
        model, make_oracle = random_model(config, args.seed, args.dtype), lambda: random_model(config, args.seed, "float32")
    eng = Engine(model=model)
    torch.cuda.synchronize()
    print(f"load+init {time.time() - t0:.1f}s", flush=True)
    hbm = measured_hbm_bandwidth()
    oracle_runner, rates, status = None, [], 0
    for shape in shapes:
        try:
            record, samples = measure_shape(eng, shape, args, hbm)
            if not args.no_check and args.temperature == 0:
                if oracle_runner is None:
                    oracle_runner = Runner(make_oracle(), max(s[1] + s[2] for s in shapes) + 64, max_slots=1)
                checked = samples if args.check_all else samples[:1]
                record["worst_gap"] = max(teacher_forced_gap(oracle_runner, p, t) for prompts, tokens in checked
                                          for p, t in zip(prompts, tokens))
                if not record["worst_gap"] <= GAP_LIMIT:
                    raise CheckFailed(f"{record['shape']}: emitted tokens are {record['worst_gap']:.3f} logits from the float32 "
                                      f"path's best, beyond the {GAP_LIMIT}-logit tolerance")
        except CheckFailed as e:
            print(f"CHECK FAILED: {e}", flush=True)
            status = 1
            continue
        rates.append(record["tok_s"])
        print(json.dumps(record) if args.json else text_line(record), flush=True)
        if "worst_gap" in record and not args.json:
            print(f"   correctness: worst gap {record['worst_gap']:.3f} logits vs the float32 path", flush=True)
        if args.print_tokens:
            for i, toks in enumerate(samples[0][1]):
                print(f"tokens {record['shape']} seq {i}: " + " ".join(map(str, toks)), flush=True)
    if rates:
        print(f"geomean {statistics.geometric_mean(rates):.1f} tok/s")
    return status


if __name__ == "__main__":
    sys.exit(main())
