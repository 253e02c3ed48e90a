"""Plain, slow implementation of the Qwen3 dense decoder: the oracle of the test-suite.

Whole sequences only, no cache, no batching, one function per part, float32 (or float64) on the
CPU. It shares no code with the package under test: it reads ``config.json`` and
``model.safetensors`` itself. Every function is written from the formulas of the reference engine
(KrishP147/Dryft-Challenge-HTN-2026) and cites the lines it restates. The reference's own CPU code
path was run once against this file on tiny random models; the outputs of that run and the script
that made them are under ``tests/golden/``.

Two options go beyond what the reference computes, so that the package's general parts can be
checked: a sliding ``window`` for attention and a layer ``schedule`` that may run a layer twice or
make it read another entry's keys and values. With ``window=None`` and the identity schedule the
functions are the reference's formulas.
"""
import json
import math
import os

import torch
from safetensors import safe_open


def read_model(folder, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors by name, cast to ``dtype``.
    Names as the reference pops them: engine/engine.py:289-307."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k).to(dtype)
    return cfg, tensors


def sizes(cfg):
    """The six values the reference reads (engine/engine.py:251-258) plus the window keys."""
    nh = cfg["num_attention_heads"]
    theta = cfg["rope_theta"] if "rope_theta" in cfg else cfg["rope_parameters"]["rope_theta"]
    return dict(
        L=cfg["num_hidden_layers"], nh=nh, nkv=cfg["num_key_value_heads"],
        hd=cfg.get("head_dim") or cfg["hidden_size"] // nh,
        eps=cfg["rms_norm_eps"], theta=float(theta),
    )


def layer_windows(cfg):
    """Per layer: the sliding window (number of keys a query sees, itself included) or None.
    The reference has no window (engine/engine.py:148-164 attends to every earlier key); the
    config keys are Qwen3's own: layers with index >= max_window_layers slide when
    use_sliding_window is set."""
    L = cfg["num_hidden_layers"]
    if not cfg.get("use_sliding_window") or cfg.get("sliding_window") is None:
        return [None] * L
    first = cfg.get("max_window_layers", L)
    return [cfg["sliding_window"] if i >= first else None for i in range(L)]


def rms_norm(x, w, eps):
    """y = w * (x * rsqrt(mean(x^2) + eps)); engine/engine.py:107-110."""
    xf = x.to(torch.float32) if x.dtype != torch.float64 else x
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return w * xf.to(x.dtype)


def rope_tables(theta, hd, n, dtype=torch.float32):
    """cos/sin [n, hd]: inv_j = theta^(-2j/hd), angle = position * inv_j, both halves alike;
    engine/engine.py:118-122."""
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2).to(dtype) / hd))
    fr = torch.outer(torch.arange(n).to(dtype), inv)
    emb = torch.cat((fr, fr), -1)
    return emb.cos(), emb.sin()


def apply_rope(x, cos, sin):
    """Rotate-half: x*cos + cat(-x[hd/2:], x[:hd/2])*sin; engine/engine.py:113-115.
    x [S, heads, hd]; cos, sin [S, hd]."""
    h = x.shape[-1] // 2
    rot = torch.cat((-x[..., h:], x[..., :h]), -1)
    return x * cos[:, None, :] + rot * sin[:, None, :]


def project_qkv(a, wq, wk, wv, nh, nkv, hd):
    """No bias; q [S,nh,hd], k,v [S,nkv,hd]; engine/engine.py:300-302,169-170."""
    S = a.shape[0]
    return ((a @ wq.T).view(S, nh, hd), (a @ wk.T).view(S, nkv, hd), (a @ wv.T).view(S, nkv, hd))


def causal_gqa_attention(q, k, v, window=None):
    """Query head h reads key/value head h // (nh/nkv); scores scaled by hd^-0.5; a query at
    position i sees keys j <= i (engine/engine.py:148-152, fused.py:315-333); with a window only
    keys j > i - window. q [S,nh,hd], k,v [S,nkv,hd] -> [S, nh*hd]."""
    S, nh, hd = q.shape
    G = nh // k.shape[1]
    out = torch.empty(S, nh, hd, dtype=q.dtype)
    i = torch.arange(S)
    allowed = i[None, :] <= i[:, None]
    if window is not None:
        allowed &= i[None, :] > i[:, None] - window
    for h in range(nh):
        kh, vh = k[:, h // G], v[:, h // G]
        s = (q[:, h] @ kh.T) * hd ** -0.5
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ vh
    return out.reshape(S, nh * hd)


def attention_mixer(a, t, p, sz, window=None, kv_from=None):
    """Projections, per-head q/k RMSNorm before RoPE (engine/engine.py:173-176), attention,
    output projection without the residual add (engine/engine.py:493). Returns the mixer's
    output and the (k, v) it attended to. ``kv_from``: keys/values of another schedule entry to
    read instead of this layer's own (not in the reference)."""
    nh, nkv, hd, eps = sz["nh"], sz["nkv"], sz["hd"], sz["eps"]
    S = a.shape[0]
    q, k, v = project_qkv(a, t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"],
                          t[p + "self_attn.v_proj.weight"], nh, nkv, hd)
    cos, sin = rope_tables(sz["theta"], hd, S, a.dtype)
    q = apply_rope(rms_norm(q, t[p + "self_attn.q_norm.weight"], eps), cos, sin)
    if kv_from is None:
        k = apply_rope(rms_norm(k, t[p + "self_attn.k_norm.weight"], eps), cos, sin)
    else:
        k, v = kv_from
    o = causal_gqa_attention(q, k, v, window)
    return o @ t[p + "self_attn.o_proj.weight"].T, (k, v)


def gated_mlp(a, t, p):
    """down(silu(gate(a)) * up(a)), silu(g) = g / (1 + e^-g), no bias;
    engine/engine.py:137-146,494-495."""
    g = a @ t[p + "mlp.gate_proj.weight"].T
    u = a @ t[p + "mlp.up_proj.weight"].T
    return ((g / (1.0 + torch.exp(-g))) * u) @ t[p + "mlp.down_proj.weight"].T


def decoder_layer(h, t, i, sz, window=None, kv_from=None):
    """Pre-norm block: h += attn(norm_in(h)); h += mlp(norm_post(h));
    engine/engine.py:468-495 (there the add and the next norm are fused)."""
    p = f"model.layers.{i}."
    a = rms_norm(h, t[p + "input_layernorm.weight"], sz["eps"])
    o, kv = attention_mixer(a, t, p, sz, window, kv_from)
    h = h + o
    a = rms_norm(h, t[p + "post_attention_layernorm.weight"], sz["eps"])
    return h + gated_mlp(a, t, p), kv


def forward(cfg, t, tokens, schedule=None, hidden_out=None):
    """Logits [S, V] of one whole sequence at every position: embedding gather without scaling
    (engine/engine.py:467), the layers in schedule order, final norm, lm_head, which is the
    embedding matrix when ``lm_head.weight`` is absent (engine/engine.py:290,498).

    ``schedule``: list of (layer, cache_entry, writes) triples; an entry with writes=False reads
    the keys and values that the entry owning ``cache_entry`` produced. Default: each layer once.
    ``hidden_out``: a list that receives the residual stream [S, H] after every schedule entry (the
    reference's ``_trace`` hook, engine/engine.py:496-497)."""
    sz = sizes(cfg)
    windows = layer_windows(cfg)
    if schedule is None:
        schedule = [(i, i, True) for i in range(sz["L"])]
    h = t["model.embed_tokens.weight"][torch.as_tensor(tokens, dtype=torch.long)]
    kvs = {}
    for layer, entry, writes in schedule:
        h, kv = decoder_layer(h, t, layer, sz, windows[layer], None if writes else kvs[entry])
        if writes:
            kvs[entry] = kv
        if hidden_out is not None:
            hidden_out.append(h)
    a = rms_norm(h, t["model.norm.weight"], sz["eps"])
    head = t.get("lm_head.weight", t["model.embed_tokens.weight"])
    return a @ head.T


def greedy(cfg, t, prompt, n):
    """n greedy tokens after ``prompt``, re-running the whole sequence each time; ties go to the
    lowest index as torch.argmax does (engine/engine.py:503)."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, t, seq)[-1].argmax()))
    return seq[len(prompt):]


# --- sampling -----------------------------------------------------------------------------------
# The reference samples greedily only (engine/engine.py:503). Temperature sampling is the
# package's own: token = argmax_i(logit_i / T + g_i) with g_i = -log(-log(u_i)) and u_i a uniform
# number drawn from a counter hash of (seed, position, i). The functions below restate that
# definition in plain Python integers so the kernel can be checked against it.

M32 = 0xFFFFFFFF


def hash_u32(seed_lo, seed_hi, pos, idx):
    """Three rounds of a 32-bit multiply-xorshift mix over (seed, position, index)."""
    def mix(x):
        x ^= x >> 16
        x = (x * 0x7FEB352D) & M32
        x ^= x >> 15
        x = (x * 0x846CA68B) & M32
        x ^= x >> 16
        return x
    x = mix((idx ^ 0x9E3779B9) & M32)
    x = mix((x + pos * 0x85EBCA6B + seed_lo) & M32)
    x = mix((x ^ seed_hi) & M32)
    return x


def gumbel_argmax(logits, temperature, seed, pos):
    """Index the sampler must return for one row of logits (float32 arithmetic, ties to the
    lowest index)."""
    import numpy as np
    lo, hi = seed & M32, (seed >> 32) & M32
    V = logits.shape[0]
    u = np.array([hash_u32(lo, hi, pos & M32, i) for i in range(V)], dtype=np.uint32)
    uf = ((u >> np.uint32(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    g = -np.log(-np.log(uf.astype(np.float64)))
    z = logits.double().numpy() / float(temperature) + g
    return int(z.argmax()), z
