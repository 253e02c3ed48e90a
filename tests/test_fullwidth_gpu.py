"""Two layers at the benchmark model's widths (Qwen3-4B: 32 query and 8 key/value heads of 128, hidden
2,560, feed-forward 9,728, vocabulary 151,936) with random weights: a ragged prefill whose logits in
bfloat16 are compared with the library's own float32 path (which the other tests tie to the plain
implementation at small sizes). At these sizes the prefill runs what the tiny configurations only
reach when forced: the q/k/v product with norm, rotation and cache write in its epilogue, the gated
product, and the tcgen05 attention with six times more (tile, head) items than blocks."""
import numpy as np
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
from dryft_challenge_htn_2026_b200.csrc import api
from dryft_challenge_htn_2026_b200.parts.attention import GQAAttention

pytestmark = pytest.mark.gpu

WIDTHS = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=2560, intermediate_size=9728,
              num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
              rope_theta=1000000.0, tie_word_embeddings=True, max_position_embeddings=40960)


def prefill_logits(cfg, prompts, dtype):
    model = dk.random_model(cfg, seed=0, dtype=dtype)
    runner = dk.Runner(model, sum((len(p) + 127) // 64 * 64 for p in prompts), max_slots=len(prompts))
    slots = [runner.begin() for _ in prompts]
    out = runner.step([(s, p, [len(p) // 2, len(p) - 1]) for s, p in zip(slots, prompts)])
    torch.cuda.synchronize()
    api.gemm_tc_check()
    return out.float().cpu()


def test_ragged_prefill_at_full_width_agrees_with_float32(monkeypatch):
    cfg = dk.config_from_dict(WIDTHS)
    rs = np.random.RandomState(3)
    prompts = [rs.randint(0, cfg.vocab_size, n).tolist() for n in (1500, 700, 2048, 129, 3000)]
    calls = {"qkv": 0, "attention": 0}
    for name, key in (("gemm_tc_qkv", "qkv"), ("attention_prefill_tc", "attention")):
        inner = getattr(api, name)

        def counting(*a, _inner=inner, _key=key, **k):
            calls[_key] += 1
            return _inner(*a, **k)

        monkeypatch.setattr(api, name, counting)
    want = prefill_logits(cfg, prompts, torch.float32)
    assert calls == {"qkv": 0, "attention": 0}                       # the float32 path takes neither
    got = prefill_logits(cfg, prompts, torch.bfloat16)
    assert calls == {"qkv": 2, "attention": 2}                       # once a layer
    monkeypatch.setattr(GQAAttention, "qkv_epilogue_min_fill", 2.0)  # the same with the separate norm/rotation kernel
    apart = prefill_logits(cfg, prompts, torch.bfloat16)
    scale = float(want.abs().max())
    assert got.shape == (2 * len(prompts), cfg.vocab_size)
    for name, x in (("epilogue", got), ("separate kernel", apart)):
        err = float((x - want).abs().max())
        assert err <= 0.03 * scale, f"{name}: {err} against float32 logits of size {scale}"
    # where float32 has a clear winner, bfloat16 picks it too
    top2 = want.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.06 * scale
    assert bool((got.argmax(-1) == want.argmax(-1))[clear].all())


def stepped_logits(cfg, prompts, forced, dtype):
    """Prefill, then len(forced) decode steps with given tokens; the logits of every decode step."""
    model = dk.random_model(cfg, seed=0, dtype=dtype)
    runner = dk.Runner(model, sum((len(p) + len(forced) + 127) // 64 * 64 for p in prompts), max_slots=len(prompts))
    slots = [runner.begin() for _ in prompts]
    runner.step([(s, p, []) for s, p in zip(slots, prompts)])
    out = [runner.step([(s, [int(tok[i])], [0]) for i, s in enumerate(slots)]).float().cpu() for tok in forced]
    torch.cuda.synchronize()
    api.gemm_tc_check()
    return torch.stack(out)


@pytest.mark.parametrize("batch", [8, 20, 64])
def test_decode_steps_at_full_width_agree_with_float32(batch):
    """Decode steps of 8 rows (the streaming product) and of 20 rows (the tensor-core product in its
    decode form; at 64 rows also the two-deep rings of the split-key attention) over ragged caches,
    split-key attention and its merge, at the benchmark widths."""
    cfg = dk.config_from_dict(WIDTHS)
    rs = np.random.RandomState(5)
    prompts = [rs.randint(0, cfg.vocab_size, int(n)).tolist() for n in rs.randint(60, 700, batch)]
    forced = rs.randint(0, cfg.vocab_size, (4, batch))
    want = stepped_logits(cfg, prompts, forced, torch.float32)
    got = stepped_logits(cfg, prompts, forced, torch.bfloat16)
    scale = float(want.abs().max())
    assert got.shape == (4, batch, cfg.vocab_size)
    err = float((got - want).abs().max())
    assert err <= 0.03 * scale, f"{err} against float32 logits of size {scale}"


@pytest.mark.parametrize("hidden,inter,heads", [(2560, 9728, 32), (2816, 5008, 24)])
def test_full_width_against_the_plain_implementation(tmp_path, hidden, inter, heads):
    """Two layers at the benchmark model's widths (and at a hidden size above them, where the streaming
    product keeps the longer rows of x in blocks of eight streaming warps), float32 and bfloat16, short ragged prompts with logits
    at two places each and then decode steps of the batch, against the plain implementation on the CPU:
    not against the library's own float32 path, so a fault the two dtypes share would show."""
    import plain_qwen3 as plain
    cfg = dk.config_from_dict(dict(WIDTHS, hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads))
    folder = dk.write_random_model(cfg, str(tmp_path / "wide"), seed=4, dtype=torch.bfloat16, matrix_std=0.02)
    pcfg, t = plain.read_model(folder)
    rs = np.random.RandomState(11)
    lens, extra = (129, 300, 70), 3
    seqs = [rs.randint(0, cfg.vocab_size, n + extra).tolist() for n in lens]
    want = []
    for s, n in zip(seqs, lens):
        ref = plain.forward(pcfg, t, s)
        want.append(ref[[n // 2, n - 1] + list(range(n, n + extra))])
    scale = max(float(w.abs().max()) for w in want)
    for dtype, tol in ((torch.float32, 2e-4), (torch.bfloat16, 0.03)):
        runner = dk.Runner(dk.load_model(folder, dtype), sum((len(s) + 63) // 64 * 64 for s in seqs), max_slots=3)
        slots = [runner.begin() for _ in seqs]
        got = [runner.step([(sl, s[:n], [n // 2, n - 1]) for sl, s, n in zip(slots, seqs, lens)]).float().cpu().view(3, 2, -1)]
        for k in range(extra):
            got.append(runner.step([(sl, [s[n + k]], [0]) for sl, s, n in zip(slots, seqs, lens)]).float().cpu().view(3, 1, -1))
        torch.cuda.synchronize()
        api.gemm_tc_check()
        got = torch.cat(got, 1)
        for i in range(3):
            err = float((got[i] - want[i]).abs().max())
            assert err <= tol * scale, f"{dtype} request {i}: {err} against plain logits of size {scale}"
        del runner
