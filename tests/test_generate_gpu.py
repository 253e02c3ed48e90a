"""Generation through the Python entry point: greedy and sampled tokens against the plain
implementation, stop tokens, batches one after another, long decoding across page boundaries,
graph replay against plain launches."""
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_qwen3 as plain
from dryft_challenge_htn_2026_b200.sampling import request_seed
from helpers import TINY, make_folder, random_tokens

pytestmark = pytest.mark.gpu


def teacher_forced_gap(cfg, t, prompt, emitted):
    """max over steps of (best plain logit - plain logit of the emitted token): 0 when the engine
    picked what the plain implementation would."""
    logits = plain.forward(cfg, t, list(prompt) + list(emitted[:-1]))[len(prompt) - 1:]
    picked = logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)
    return float((logits.max(-1).values - picked).max())


@pytest.mark.parametrize("name,lens,n", [("A", [5, 9, 13], 8), ("B", [1, 7, 16, 31], 12), ("C", [3, 70, 33], 40)])
def test_greedy_float32_equals_plain(tmp_path, name, lens, n):
    folder = make_folder(tmp_path, name, seed=7)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(TINY[name]["vocab_size"], L, 10 + i) for i, L in enumerate(lens)]
    eng = dk.Engine(folder, dtype=torch.float32)
    steps = list(eng.generate(prompts, n))
    assert len(steps) == n and all(len(s) == len(prompts) for s in steps)
    for i, p in enumerate(prompts):
        emitted = [s[i] for s in steps]
        want = plain.greedy(cfg, t, p, n)
        if emitted != want:          # a near-tie may flip in float32: then the gap must be rounding-small
            assert teacher_forced_gap(cfg, t, p, emitted) < 1e-4, (i, emitted, want)
    again = list(eng.generate(prompts, n))
    assert again == steps                                             # no state leaks between calls
    assert list(eng.generate(prompts, 0)) == []
    # one request alone gives what it gave in the batch
    alone = [s[0] for s in eng.generate([prompts[1]], n)]
    assert alone == [s[1] for s in steps]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_bfloat16_stays_within_rounding_of_plain(tmp_path, name):
    folder = make_folder(tmp_path, name, seed=8)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(TINY[name]["vocab_size"], L, 20 + i) for i, L in enumerate([4, 40, 66, 17, 9])]
    eng = dk.Engine(folder, dtype=torch.bfloat16)
    steps = list(eng.generate(prompts, 24))
    scale = max(1.0, float(plain.forward(cfg, t, prompts[1]).abs().max()))
    for i, p in enumerate(prompts):
        assert teacher_forced_gap(cfg, t, p, [s[i] for s in steps]) <= 0.12 * scale


def test_graph_replay_equals_plain_launches(tmp_path):
    folder = make_folder(tmp_path, "B", seed=9)
    prompts = [random_tokens(384, L, 30 + i) for i, L in enumerate([3, 50, 64])]
    for dtype in (torch.float32, torch.bfloat16):
        a = list(dk.Engine(folder, dtype=dtype, use_graph=True).generate(prompts, 20, temperature=0.9, seed=3))
        b = list(dk.Engine(folder, dtype=dtype, use_graph=False).generate(prompts, 20, temperature=0.9, seed=3))
        assert a == b


def test_temperature_sampling_follows_the_plain_gumbel_rule(tmp_path):
    folder = make_folder(tmp_path, "B", seed=10)
    cfg, t = plain.read_model(folder)
    lens, n, temp, seed = [1, 7, 16, 31], 12, 0.8, 1234
    prompts = [random_tokens(384, L, 40 + i) for i, L in enumerate(lens)]
    eng = dk.Engine(folder, dtype=torch.float32)
    steps = list(eng.generate(prompts, n, temperature=temp, seed=seed))
    assert steps != list(eng.generate(prompts, n, temperature=temp, seed=seed + 1))
    assert steps == list(eng.generate(prompts, n, temperature=temp, seed=seed))
    for i, p in enumerate(prompts):
        emitted = [s[i] for s in steps]
        logits = plain.forward(cfg, t, p + emitted[:-1])[len(p) - 1:]
        for k, tok in enumerate(emitted):
            want, z = plain.gumbel_argmax(logits[k], temp, request_seed(seed, i), len(p) + k)
            assert tok == want or abs(z[tok] - z[want]) < 1e-3, (i, k, tok, want)
    # a request draws the same tokens alone as in the batch (its seed goes with its index)
    alone = [s[0] for s in eng.generate([prompts[2]], n, temperature=temp, seed=seed, first_index=2)]
    assert alone == [s[2] for s in steps]


def test_stop_tokens_and_batches_one_after_another(tmp_path):
    folder = make_folder(tmp_path, "A", seed=11)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(256, 3 + (5 * i) % 23, 50 + i) for i in range(11)]
    eng = dk.Engine(folder, dtype=torch.float32)
    free = dk.Engine(folder, dtype=torch.float32).generate_all(prompts, 30, batch_size=16)
    # pick as stop tokens ids that some sequences emit in the middle
    stops = {free[0][5], free[3][11], free[7][2]}
    outs = eng.generate_all(prompts, 30, stop_token_ids=stops, batch_size=4)    # 3 batches on reused slots
    assert len(outs) == 11
    for i, o in enumerate(outs):
        cut = next((k for k, tok in enumerate(free[i]) if tok in stops), 29)
        assert o == free[i][:cut + 1], i                               # the stop token is the last one returned
    assert eng.runner.cache.slots.n_live == 0
    assert eng.runner.cache.pages_free() == [eng.runner.cache.num_pages]


def test_long_decoding_across_pages(tmp_path):
    folder = make_folder(tmp_path, "C", seed=12)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(300, 5, 60), random_tokens(300, 62, 61)]
    for dtype, bound in ((torch.float32, 1e-4), (torch.bfloat16, None)):
        eng = dk.Engine(folder, dtype=dtype)
        steps = list(eng.generate(prompts, 200))                      # lengths pass 64, 128, 192, 256 and the window
        scale = max(1.0, float(plain.forward(cfg, t, prompts[1]).abs().max()))
        for i, p in enumerate(prompts):
            gap = teacher_forced_gap(cfg, t, p, [s[i] for s in steps])
            assert gap <= (bound if bound is not None else 0.12 * scale), (dtype, i, gap)


def test_engine_refuses_bad_input(tmp_path):
    folder = make_folder(tmp_path, "A", seed=13)
    eng = dk.Engine(folder, dtype=torch.float32)
    with pytest.raises(ValueError):
        list(eng.generate([[1, 2], []], 3))
    with pytest.raises(ValueError):
        list(eng.generate([[1, 999]], 3))                             # id outside the vocabulary
    small = dk.Engine(folder, dtype=torch.float32, max_tokens=64)
    with pytest.raises(ValueError):
        list(small.generate([[1] * 60], 30))
    assert len(list(small.generate([[1] * 10], 5))) == 5


@pytest.mark.parametrize("name", ["D", "E"])
def test_prefill_projection_with_norm_rotation_and_cache_write_in_its_epilogue(tmp_path, monkeypatch, name):
    """Prefill steps of more than 128 rows whose q/k/v projection norms, rotates and writes the cache
    in the epilogue of the tensor-core product (forced here: the tiny sizes would not fill the GPU):
    the kernel really runs, and prefill and the decoding from the cache it wrote stay within rounding
    of the plain implementation."""
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.parts.attention import GQAAttention
    folder = make_folder(tmp_path, name, seed=15)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(TINY[name]["vocab_size"], L, 90 + i) for i, L in enumerate([100, 70, 33, 150])]
    monkeypatch.setattr(GQAAttention, "qkv_epilogue_min_fill", 0.0)
    seen = {"calls": 0}
    inner = api.gemm_tc_qkv

    def counting(*a, **k):
        seen["calls"] += 1
        return inner(*a, **k)

    monkeypatch.setattr(api, "gemm_tc_qkv", counting)
    steps = list(dk.Engine(folder, dtype=torch.bfloat16).generate(prompts, 12))
    assert seen["calls"] == TINY[name]["num_hidden_layers"]
    scale = max(1.0, float(plain.forward(cfg, t, prompts[0]).abs().max()))
    for i, p in enumerate(prompts):
        assert teacher_forced_gap(cfg, t, p, [s[i] for s in steps]) <= 0.12 * scale


def test_prefill_in_several_steps_gives_the_same_tokens(tmp_path):
    """Prompts that do not fit one prefill step (here: a limit of 50 tokens) are prefilled in groups of
    whole sequences and a long one in chunks; in float32 that changes no token."""
    folder = make_folder(tmp_path, "C", seed=13)
    prompts = [random_tokens(TINY["C"]["vocab_size"], L, 60 + i) for i, L in enumerate([20, 25, 130, 7, 49, 51])]
    whole = list(dk.Engine(folder, dtype=torch.float32).generate(prompts, 10, temperature=0.8, seed=4))
    pieces = list(dk.Engine(folder, dtype=torch.float32, max_prefill_tokens=50).generate(prompts, 10, temperature=0.8, seed=4))
    assert pieces == whole
    # bfloat16: continuation chunks on top of a cache, a last portion of one token (51 under a limit of 50) and
    # of two (52), steps of few rows through the skinny products, windowed layers after trimming
    cfg, t = plain.read_model(folder)
    prompts.append(random_tokens(TINY["C"]["vocab_size"], 52, 77))
    bf = list(dk.Engine(folder, dtype=torch.bfloat16, max_prefill_tokens=50).generate(prompts, 10))
    assert len(bf) == 10 and all(len(s) == len(prompts) for s in bf)
    scale = max(1.0, float(plain.forward(cfg, t, prompts[2]).abs().max()))
    for i, p in enumerate(prompts):
        assert teacher_forced_gap(cfg, t, p, [s[i] for s in bf]) <= 0.12 * scale, i


def test_twenty_sequences_decode_on_the_tensor_core_product(tmp_path):
    """A batch beyond 8 rows takes the tcgen05 decode product (a 32-row decode state here, 12 of the
    rows padding): tokens stay within rounding of the plain implementation."""
    folder = make_folder(tmp_path, "D", seed=14)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(TINY["D"]["vocab_size"], 3 + (7 * i) % 60, 80 + i) for i in range(20)]
    eng = dk.Engine(folder, dtype=torch.bfloat16)
    steps = list(eng.generate(prompts, 12))
    assert len(steps) == 12 and all(len(s) == 20 for s in steps)
    scale = max(1.0, float(plain.forward(cfg, t, prompts[5]).abs().max()))
    for i in (0, 5, 11, 19):
        assert teacher_forced_gap(cfg, t, prompts[i], [s[i] for s in steps]) <= 0.12 * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stop_tokens_repack_into_a_smaller_graph(tmp_path, dtype):
    """Greedy generation of 11 sequences under CUDA graphs with stop tokens chosen so that sequences
    end at different steps: the batch is re-packed into smaller decode states (16 -> 8 -> 4 rows, a new
    graph each), and what every sequence emits up to its stop is what it emits without stops."""
    folder = make_folder(tmp_path, "D", seed=16)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(TINY["D"]["vocab_size"], 5 + (11 * i) % 70, 300 + i) for i in range(11)]
    eng = dk.Engine(folder, dtype=dtype)
    free = list(eng.generate(prompts, 24))
    streams = [[s[i] for s in free] for i in range(len(prompts))]
    # stop tokens: what sequence i emits at step 3 + 2 i (for the first eight), so the batch shrinks again and again
    stops = {streams[i][3 + 2 * i] for i in range(8)}
    rows = list(eng.generate(prompts, 24, stop_token_ids=sorted(stops)))
    ended = 0
    for i, full in enumerate(streams):
        got = [r[i] for r in rows if r[i] is not None]
        cut = next((k for k, tok in enumerate(full) if tok in stops), len(full) - 1)
        if dtype == torch.float32:
            assert got == full[:cut + 1], i
        else:       # bfloat16: another decode state takes other product kernels; compare with the plain implementation
            assert len(got) >= 1 and (got[-1] in stops or len(got) == 24)
            scale = max(1.0, float(plain.forward(cfg, t, prompts[i]).abs().max()))
            assert teacher_forced_gap(cfg, t, prompts[i], got) <= 0.12 * scale, i
        ended += got[-1] in stops
    assert ended >= 8
    states = eng.backend.loop.states
    assert len({rows_ for rows_, _ in states}) >= 3                   # several bucket sizes were used


def test_a_decode_step_of_more_than_128_sequences(tmp_path):
    """150 sequences in one batch: the decode state has 256 rows, beyond what the decode forms of the
    products take, so its steps run the prefill forms (and the library product) on one token a row."""
    folder = make_folder(tmp_path, "D", seed=17)
    cfg, t = plain.read_model(folder)
    prompts = [random_tokens(TINY["D"]["vocab_size"], 2 + (5 * i) % 40, 500 + i) for i in range(150)]
    for dtype, bound in ((torch.float32, 1e-4), (torch.bfloat16, None)):
        steps = list(dk.Engine(folder, dtype=dtype).generate(prompts, 6))
        assert len(steps) == 6 and all(len(s) == 150 for s in steps)
        for i in (0, 7, 64, 128, 149):
            scale = max(1.0, float(plain.forward(cfg, t, prompts[i]).abs().max()))
            gap = teacher_forced_gap(cfg, t, prompts[i], [s[i] for s in steps])
            assert gap <= (bound if bound is not None else 0.12 * scale), (dtype, i, gap)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_steps_replayed_as_graphs_give_the_same_tokens(tmp_path, dtype):
    """A prompt shape that comes a second time is captured and from then on replayed (the first time it
    runs plainly): the same tokens as without graphs, also for other prompts of that shape on other
    slots, for a shape captured earlier that returns, and for prompts in several steps."""
    folder = make_folder(tmp_path, "D", seed=18)
    vocab = TINY["D"]["vocab_size"]
    lens = [150, 40, 3, 64]
    plain_eng = dk.Engine(folder, dtype=dtype, use_graph=False)
    eng = dk.Engine(folder, dtype=dtype, use_graph=True)
    for round_ in range(4):
        prompts = [random_tokens(vocab, L, 700 + 10 * round_ + i) for i, L in enumerate(lens)]
        if round_ == 3:
            prompts = prompts[::-1]                                    # another shape in between
        want = list(plain_eng.generate(prompts, 5, temperature=0.7, seed=round_))
        assert list(eng.generate(prompts, 5, temperature=0.7, seed=round_)) == want, round_
    assert len(eng.runner._graphs) == 1                               # the shape that came more than once
    prompts = [random_tokens(vocab, L, 800 + i) for i, L in enumerate(lens)]
    assert list(eng.generate(prompts, 5)) == list(plain_eng.generate(prompts, 5))     # the captured shape again, after another
    chunked = dk.Engine(folder, dtype=dtype, use_graph=True, max_prefill_tokens=100)
    want = list(dk.Engine(folder, dtype=dtype, use_graph=False, max_prefill_tokens=100).generate(prompts, 5))
    for _ in range(3):                                                 # steps of 100 + 50 | 40 + 3 | 64 tokens, each shape captured
        assert list(chunked.generate(prompts, 5)) == want
    assert len(chunked.runner._graphs) >= 3
