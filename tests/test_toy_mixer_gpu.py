"""A mixer with state of its own, defined here, registered, built and stepped without touching
the library: a decaying running sum per sequence (state [hidden], fixed size, zero at the start)
followed by a projection. The toy model mixes it with attention layers, so one model has
different mixers in different layers, two cache groups (a state group and a key/value group) and
per-sequence state that must survive ragged batches, single-token steps and slot reuse."""
from dataclasses import dataclass

import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_qwen3 as plain
from dryft_challenge_htn_2026_b200.config.base import get
from dryft_challenge_htn_2026_b200.config.specs import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec,
                                                        RotaryHalfSpec)
from dryft_challenge_htn_2026_b200.engine.engine import load_model
from dryft_challenge_htn_2026_b200.parts import ParamDecl, Part, register_part
from helpers import random_tokens

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class RunningSumSpec:
    hidden_size: int
    decay: float


class RunningSumMixer(Part):
    """state <- decay * state + x_t ;  out_t = state . W^T   (plain torch ops: it is a test toy)."""

    def param_decls(self):
        return [ParamDecl("proj.weight", (self.spec.hidden_size, self.spec.hidden_size))]

    def bind(self, tensors):
        self.w = tensors.pop("proj.weight")

    def cache_requests(self):
        return [dk.StateRequest((self.spec.hidden_size,), torch.float32)]

    def prepare(self, max_positions):
        pass

    def forward(self, ctx, views, a, writes=True):
        state = views[0].state                                        # [slots, hidden], float32
        out = torch.empty_like(a)
        if ctx.is_decode:                                              # one token per row; padding rows have position -1
            live = (ctx.row_pos >= 0).nonzero().flatten()
            slots = ctx.seq_slot.long()[live]
            s = self.spec.decay * state[slots] + a[live].float()
            state[slots] = s
            out.zero_()
            out[live] = (s @ self.w.float().T).to(a.dtype)
            return out
        cu, slots = ctx.host["cu_q"], ctx.host["slots"]
        for i, slot in enumerate(slots):
            s = state[slot].clone()
            for r in range(int(cu[i]), int(cu[i + 1])):
                s = self.spec.decay * s + a[r].float()
                out[r] = (s @ self.w.float().T).to(a.dtype)
            state[slot] = s
        return out


@dataclass(frozen=True)
class ToyConfig(dk.ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    kinds: tuple                  # per layer: "sum" or "attn"
    decay: float
    eps: float
    architecture = "ToyRunningSumForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(get(d, "vocab_size", int), get(d, "hidden_size", int), get(d, "intermediate_size", int),
                   tuple(d["kinds"]), get(d, "decay", float), get(d, "eps", float))

    def to_dict(self):
        return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                    intermediate_size=self.intermediate_size, kinds=list(self.kinds), decay=self.decay, eps=self.eps)

    def to_spec(self):
        H = self.hidden_size
        attn = AttentionSpec(H, 4, 2, 16, 0.25, RMSNormSpec(16, self.eps), RotaryHalfSpec(16, 1e4), None)
        layers = tuple(LayerSpec(f"model.layers.{i}.", RMSNormSpec(H, self.eps),
                                 RunningSumSpec(H, self.decay) if k == "sum" else attn, RMSNormSpec(H, self.eps),
                                 GatedMLPSpec(H, self.intermediate_size)) for i, k in enumerate(self.kinds))
        return ModelSpec(self.architecture, self.vocab_size, H, layers, ModelSpec.identity_schedule(len(layers)),
                         RMSNormSpec(H, self.eps), True, 512)


def plain_toy_forward(cfg, t, tokens):
    h = t["model.embed_tokens.weight"][torch.tensor(tokens)]
    sz = dict(nh=4, nkv=2, hd=16, eps=cfg.eps, theta=1e4)
    for i, kind in enumerate(cfg.kinds):
        p = f"model.layers.{i}."
        a = plain.rms_norm(h, t[p + "input_layernorm.weight"], cfg.eps)
        if kind == "sum":
            s, rows = torch.zeros(cfg.hidden_size), []
            for x in a:
                s = cfg.decay * s + x
                rows.append(s @ t[p + "self_attn.proj.weight"].T)
            h = h + torch.stack(rows)
        else:
            h = h + plain.attention_mixer(a, t, p, sz)[0]
        a = plain.rms_norm(h, t[p + "post_attention_layernorm.weight"], cfg.eps)
        h = h + plain.gated_mlp(a, t, p)
    return plain.rms_norm(h, t["model.norm.weight"], cfg.eps) @ t["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path, dtype):
    register_part(RunningSumSpec, RunningSumMixer)
    dk.register_architecture(ToyConfig)
    cfg = ToyConfig(200, 64, 96, ("sum", "attn", "sum"), 0.9, 1e-5)
    folder = dk.write_random_model(cfg, str(tmp_path / "toy"), seed=1, dtype=torch.float32, matrix_std=0.08)
    assert dk.config_from_folder(folder) == cfg
    _, t = plain.read_model(folder)
    model = load_model(folder, dtype)
    runner = dk.Runner(model, 64 * 8)
    kinds = [type(g).__name__ for g in runner.cache.groups]
    assert sorted(kinds) == ["KVGroup", "StateGroup"] and [len(g.entries) for g in runner.cache.groups] == [2, 1]
    tol = (2e-4 if dtype == torch.float32 else 6e-2)
    for round_ in range(2):                                            # the second round reuses the slots: state must restart at zero
        seqs = [random_tokens(200, n, 70 + 10 * round_ + i) for i, n in enumerate([9, 30, 70])]
        ref = [plain_toy_forward(cfg, t, s) for s in seqs]
        slots = [runner.begin() for _ in seqs]
        cut = [4, 22, 66]
        out = runner.step([(sl, s[:c], [c - 1]) for sl, s, c in zip(slots, seqs, cut)]).cpu()
        for i in range(3):
            assert float((out[i] - ref[i][cut[i] - 1]).abs().max()) <= tol * max(1.0, float(ref[i].abs().max()))
        for k in range(4):                                             # then one token each
            out = runner.step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu()
            for i in range(3):
                assert float((out[i] - ref[i][cut[i] + k]).abs().max()) <= tol * max(1.0, float(ref[i].abs().max()))
        for sl in slots:
            runner.end(sl)
    # and through the generation loop (plain launches: the toy's torch indexing is not graph-safe)
    eng = dk.Engine(model=model, use_graph=False)
    prompt = random_tokens(200, 12, 99)
    emitted = [s[0] for s in eng.generate([prompt], 6)]
    if dtype == torch.float32:
        seq = list(prompt)
        for tok in emitted:
            logits = plain_toy_forward(cfg, t, seq)[-1]
            assert tok == int(logits.argmax()) or float(logits.max() - logits[tok]) < 1e-4
            seq.append(tok)
