"""The order in which layers run is data: a model whose schedule runs a layer twice (each run with a
cache entry of its own) and lets another layer read the keys and values the first of those runs
stored, defined here from Qwen3's parts alone (a config class with another schedule, nothing else),
against the plain implementation's forward with the same schedule: whole prompts of unequal
lengths with logits everywhere, then tokens one by one, then a second batch in the slots the first
gave back."""
import dataclasses

import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
from dryft_challenge_htn_2026_b200.config.specs import ScheduleEntry

import plain_qwen3 as plain
from helpers import TINY, random_tokens

pytestmark = pytest.mark.gpu

# layer 0; layer 1 twice (cache entries 1 and 2); layer 2 on the keys and values of layer 1's first run
SCHEDULE = ((0, 0, True), (1, 1, True), (1, 2, True), (2, 1, False))


class TwiceConfig(dk.Qwen3Config):
    architecture = "Qwen3TwiceForCausalLM"

    def to_dict(self):
        return dict(super().to_dict(), architectures=[self.architecture])

    def to_spec(self):
        spec = super().to_spec()
        return dataclasses.replace(spec, architecture=self.architecture, schedule=tuple(ScheduleEntry(*e) for e in SCHEDULE))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_run_twice_and_a_layer_that_reads_another_layers_cache(tmp_path, dtype):
    dk.register_architecture(TwiceConfig)
    cfg = TwiceConfig.from_dict(dict(TINY["B"], architectures=[TwiceConfig.architecture]))
    folder = dk.write_random_model(cfg, str(tmp_path / "twice"), seed=3, dtype=torch.float32, matrix_std=0.08)
    assert type(dk.config_from_folder(folder)) is TwiceConfig
    pcfg, t = plain.read_model(folder)
    model = dk.load_model(folder, getattr(torch, dtype))
    assert len(model.spec.schedule) == 4 and model.spec.schedule[3].writes is False
    runner = dk.Runner(model, 64 * 4, max_slots=3)
    tol = 2e-4 if dtype == "float32" else 6e-2
    for round_ in range(2):                                    # the second round takes the slots the first gave back
        seqs = [random_tokens(cfg.vocab_size, n, 70 + 10 * round_ + i) for i, n in enumerate([9, 70, 41])]
        ref = [plain.forward(pcfg, t, s, schedule=list(SCHEDULE)) for s in seqs]
        plain_order = [plain.forward(pcfg, t, s) for s in seqs]
        assert not torch.allclose(ref[1], plain_order[1], atol=1e-3)          # the schedule matters
        cut = [4, 65, 30]
        slots = [runner.begin() for _ in seqs]
        out = runner.step([(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).float().cpu()
        rows = [(i, p) for i, c in enumerate(cut) for p in range(c)]
        for k in range(4):
            step = runner.step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).float().cpu()
            out = torch.cat([out, step])
            rows += [(i, cut[i] + k) for i in range(3)]
        for (i, p), row in zip(rows, out):
            err = float((row - ref[i][p]).abs().max())
            assert err <= tol * max(1.0, float(ref[i].abs().max())), (round_, i, p, err)
        for sl in slots:
            runner.end(sl)


def test_generation_follows_the_schedule_too(tmp_path):
    """Greedy generation through the entry point (prefill through the step function, decoding through the
    captured decode state) with that schedule, float32, against greedy decoding with the plain forward."""
    dk.register_architecture(TwiceConfig)
    cfg = TwiceConfig.from_dict(dict(TINY["B"], architectures=[TwiceConfig.architecture]))
    folder = dk.write_random_model(cfg, str(tmp_path / "twice"), seed=5, dtype=torch.float32, matrix_std=0.08)
    pcfg, t = plain.read_model(folder)
    prompts = [random_tokens(cfg.vocab_size, n, 90 + i) for i, n in enumerate([5, 37])]
    want = []
    for prompt in prompts:
        seq = list(prompt)
        for _ in range(7):
            seq.append(int(plain.forward(pcfg, t, seq, schedule=list(SCHEDULE))[-1].argmax()))
        want.append(seq[len(prompt):])
    eng = dk.Engine(folder, dtype="float32")
    got = eng.generate_all(prompts, 7)
    assert [list(g) for g in got] == want
