"""More toy parts defined here and registered from outside the library, mixed into one model layer
by layer: a feed-forward with routing (top-1 of a few small experts), a position encoding of
another form (rotation of interleaved pairs, applied by the part itself, after the attention
part's per-head q/k norm), and a norm of another kind (mean-centred), which is also the first
layer's input norm and the final norm, where the library would otherwise fuse its own RMSNorm into
the embedding and the gather of the wanted rows. None of them is anyone's architecture; they show
that the block, the schedule, the cache and the step function do not care what the parts are."""
from dataclasses import dataclass

import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_qwen3 as plain
from dryft_challenge_htn_2026_b200.config.base import get
from dryft_challenge_htn_2026_b200.config.specs import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec
from dryft_challenge_htn_2026_b200.engine.engine import load_model
from dryft_challenge_htn_2026_b200.parts import ParamDecl, Part, register_part
from helpers import random_tokens

pytestmark = pytest.mark.gpu
NH, NKV, HD = 4, 2, 16


# ------------------------------------------------------------------ a feed-forward with routing
@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    expert_size: int
    n_experts: int


class RoutedFeedForward(Part):
    """Each token goes to the expert with the largest router logit (float32 logits, ties to the
    lowest index) and gets gate * down(relu(up(x))), gate = sigmoid of that logit."""

    def param_decls(self):
        s = self.spec
        return [ParamDecl("router.weight", (s.n_experts, s.hidden_size)),
                ParamDecl("experts.up", (s.n_experts, s.expert_size, s.hidden_size)),
                ParamDecl("experts.down", (s.n_experts, s.hidden_size, s.expert_size))]

    def bind(self, tensors):
        self.router, self.up, self.down = tensors.pop("router.weight"), tensors.pop("experts.up"), tensors.pop("experts.down")

    def forward(self, ctx, a):
        return routed(a, self.router, self.up, self.down)


def routed(a, router, up, down):
    logits = a.float() @ router.float().T
    top = logits.argmax(-1)
    gate = torch.sigmoid(logits.gather(1, top[:, None]))
    hid = torch.relu(torch.einsum("th,teh->te", a.float(), up.float()[top]))
    return (gate * torch.einsum("te,the->th", hid, down.float()[top])).to(a.dtype)


# ------------------------------------------------------------- a position encoding of another form
@dataclass(frozen=True)
class PairRotarySpec:
    dim: int
    theta: float


class PairRotary(Part):
    """Rotates the pairs (2j, 2j+1) of every q and k head by position * theta^(-2j/dim); the part
    rewrites the projection rows itself (no fused tables)."""

    def apply(self, qkv, ctx, nh, nkv, hd):
        heads = qkv.view(qkv.shape[0], nh + 2 * nkv, hd)[:, :nh + nkv]
        heads.copy_(pair_rotate(heads.float(), ctx.row_pos.float(), self.spec.theta).to(qkv.dtype))


def pair_rotate(x, pos, theta):
    """x [T, heads, hd] float32, pos [T]."""
    hd = x.shape[-1]
    inv = theta ** (-torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd)
    ang = pos[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    even, odd = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = even * c - odd * s
    out[..., 1::2] = odd * c + even * s
    return out


# --------------------------------------------------------------------------- a norm of another kind
@dataclass(frozen=True)
class CentredNormSpec:
    dim: int
    eps: float


class CentredNorm(Part):
    """y = w * (x - mean(x)) * rsqrt(var(x) + eps), statistics in float32."""

    def param_decls(self):
        return [ParamDecl("weight", (self.spec.dim,), init="norm", keep_float32=True)]

    def bind(self, tensors):
        self.weight = tensors["weight"].float()

    def add_forward(self, h, delta, out, rows=None):
        if rows is not None:
            x = h[rows.long()] + (0 if delta is None else delta[rows.long()].float())
        else:
            if delta is not None:
                h += delta.float()
            x = h
        out[:x.shape[0]] = centred(x, self.weight, self.spec.eps).to(out.dtype)
        return out


def centred(x, w, eps):
    x = x.float() - x.float().mean(-1, keepdim=True)
    return w * x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------ the toy model
@dataclass(frozen=True)
class ToyPartsConfig(dk.ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    expert_size: int
    n_experts: int
    feed_forwards: tuple          # per layer: "dense" or "routed"
    theta: float
    eps: float
    architecture = "ToyPartsForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(get(d, "vocab_size", int), get(d, "hidden_size", int), get(d, "intermediate_size", int),
                   get(d, "expert_size", int), get(d, "n_experts", int), tuple(d["feed_forwards"]), get(d, "theta", float),
                   get(d, "eps", float))

    def to_dict(self):
        return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                    intermediate_size=self.intermediate_size, expert_size=self.expert_size, n_experts=self.n_experts,
                    feed_forwards=list(self.feed_forwards), theta=self.theta, eps=self.eps)

    def to_spec(self):
        H = self.hidden_size
        attn = AttentionSpec(H, NH, NKV, HD, HD ** -0.5, RMSNormSpec(HD, self.eps), PairRotarySpec(HD, self.theta), None)
        ff = {"dense": GatedMLPSpec(H, self.intermediate_size), "routed": RoutedSpec(H, self.expert_size, self.n_experts)}
        layers = tuple(LayerSpec(f"model.layers.{i}.", RMSNormSpec(H, self.eps) if i % 2 else CentredNormSpec(H, self.eps), attn,
                                 RMSNormSpec(H, self.eps), ff[k]) for i, k in enumerate(self.feed_forwards))
        return ModelSpec(self.architecture, self.vocab_size, H, layers, ModelSpec.identity_schedule(len(layers)),
                         CentredNormSpec(H, self.eps), True, 512)


def plain_forward(cfg, t, tokens):
    h = t["model.embed_tokens.weight"][torch.tensor(tokens)]
    pos = torch.arange(len(tokens), dtype=torch.float32)
    for i, kind in enumerate(cfg.feed_forwards):
        p = f"model.layers.{i}."
        w_in = t[p + "input_layernorm.weight"]
        a = plain.rms_norm(h, w_in, cfg.eps) if i % 2 else centred(h, w_in, cfg.eps)
        q, k, v = plain.project_qkv(a, t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"],
                                    t[p + "self_attn.v_proj.weight"], NH, NKV, HD)
        q, k = plain.rms_norm(q, t[p + "self_attn.q_norm.weight"], cfg.eps), plain.rms_norm(k, t[p + "self_attn.k_norm.weight"], cfg.eps)
        o = plain.causal_gqa_attention(pair_rotate(q, pos, cfg.theta), pair_rotate(k, pos, cfg.theta), v)
        h = h + o @ t[p + "self_attn.o_proj.weight"].T
        a = plain.rms_norm(h, t[p + "post_attention_layernorm.weight"], cfg.eps)
        if kind == "dense":
            h = h + plain.gated_mlp(a, t, p)
        else:
            h = h + routed(a, t[p + "mlp.router.weight"], t[p + "mlp.experts.up"], t[p + "mlp.experts.down"])
    return centred(h, t["model.norm.weight"], cfg.eps) @ t["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_feed_forward_position_and_norm_register_build_and_step(tmp_path, dtype):
    for spec, part in ((RoutedSpec, RoutedFeedForward), (PairRotarySpec, PairRotary), (CentredNormSpec, CentredNorm)):
        register_part(spec, part)
    dk.register_architecture(ToyPartsConfig)
    cfg = ToyPartsConfig(210, 64, 96, 40, 3, ("dense", "routed", "routed"), 1e4, 1e-5)
    folder = dk.write_random_model(cfg, str(tmp_path / "toy"), seed=2, dtype=torch.float32, matrix_std=0.08)
    assert dk.config_from_folder(folder) == cfg
    _, t = plain.read_model(folder)
    runner = dk.Runner(load_model(folder, dtype), 64 * 6)
    tol = 2e-4 if dtype == torch.float32 else 6e-2
    seqs = [random_tokens(210, n, 50 + i) for i, n in enumerate([7, 40, 66])]
    ref = [plain_forward(cfg, t, s) for s in seqs]
    slots = [runner.begin() for _ in seqs]
    cut = [3, 33, 62]
    out = runner.step([(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).cpu()
    rows = [(i, p) for i, c in enumerate(cut) for p in range(c)]
    for k in range(3):
        step = runner.step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu()
        out = torch.cat([out, step])
        rows += [(i, cut[i] + k) for i in range(3)]
    bad = [(i, p) for (i, p), row in zip(rows, out)
           if float((row - ref[i][p]).abs().max()) > tol * max(1.0, float(ref[i].abs().max()))]
    # float32 must agree everywhere; in bfloat16 a token whose two best router logits nearly tie may go to the other
    # expert, which changes that row for good: allow a few such rows, none of them in the first layer's reach alone
    assert len(bad) <= (0 if dtype == torch.float32 else len(rows) // 10), bad
