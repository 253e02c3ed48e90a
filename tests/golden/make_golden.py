"""Makes tests/golden/*.npz: logits of the reference engine's own CPU code on tiny random models.

Run once, by hand, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/Dryft-Challenge-HTN-2026

It imports the reference's ``engine/engine.py`` (its plain-PyTorch ops in float32 on the CPU, the
path its own tests/test_vs_hf.py uses), writes each tiny model to a temporary folder, and for one
token sequence per model records the logits after every prefix (the reference returns logits for
the last position of a forward only, engine/engine.py:476-478,498) and its greedy continuation.
``tests/test_plain.py`` rebuilds the same weights from the seed (numpy's MT19937 stream, which is
stable across versions) and compares ``tests/plain_qwen3.py`` with the stored numbers, so the
reference itself is not needed to run the tests.
"""
import json
import os
import sys
import tempfile

import numpy as np
import torch
from safetensors.torch import save_file

GOLDEN_CONFIGS = {
    # differ in every size and option; both small enough that the logits are a few KB
    "g1": dict(vocab_size=160, hidden_size=48, intermediate_size=80, num_hidden_layers=2,
               num_attention_heads=6, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
               rope_theta=10000.0, tie_word_embeddings=True, max_position_embeddings=64),
    "g2": dict(vocab_size=200, hidden_size=40, intermediate_size=72, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=4, head_dim=32, rms_norm_eps=1e-5,
               rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=96),
}
SEQ_LEN = 20
N_GREEDY = 6


def golden_weights(cfg, seed):
    """Tensors by name from a numpy RandomState: matrices N(0, 0.02) (embedding scaled up so the
    logits are not all near zero), norm weights 1 + N(0, 0.1)."""
    r = np.random.RandomState(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(o, i, s=0.02):
        return torch.from_numpy((r.standard_normal((o, i)) * s).astype(np.float32))

    def nrm(n):
        return torch.from_numpy((1.0 + 0.1 * r.standard_normal(n)).astype(np.float32))

    t = {"model.embed_tokens.weight": mat(V, H, 0.5)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = nrm(H)
        t[p + "post_attention_layernorm.weight"] = nrm(H)
        t[p + "self_attn.q_norm.weight"] = nrm(hd)
        t[p + "self_attn.k_norm.weight"] = nrm(hd)
        t[p + "self_attn.q_proj.weight"] = mat(nh * hd, H, 0.2)
        t[p + "self_attn.k_proj.weight"] = mat(nkv * hd, H, 0.2)
        t[p + "self_attn.v_proj.weight"] = mat(nkv * hd, H, 0.2)
        t[p + "self_attn.o_proj.weight"] = mat(H, nh * hd, 0.2)
        t[p + "mlp.gate_proj.weight"] = mat(I, H, 0.2)
        t[p + "mlp.up_proj.weight"] = mat(I, H, 0.2)
        t[p + "mlp.down_proj.weight"] = mat(H, I, 0.2)
    t["model.norm.weight"] = nrm(H)
    if not cfg["tie_word_embeddings"]:
        t["lm_head.weight"] = mat(V, H, 0.5)
    return t


def golden_tokens(cfg, seed):
    return np.random.RandomState(seed + 1).randint(0, cfg["vocab_size"], SEQ_LEN).tolist()


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "engine"))
    from engine import Engine  # the reference's own class

    here = os.path.dirname(os.path.abspath(__file__))
    for seed, (name, cfg) in enumerate(GOLDEN_CONFIGS.items(), start=11):
        t = golden_weights(cfg, seed)
        toks = golden_tokens(cfg, seed)
        with tempfile.TemporaryDirectory() as d:
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump(dict(cfg, architectures=["Qwen3ForCausalLM"]), f)
            save_file(t, os.path.join(d, "model.safetensors"))
            eng = Engine(d, dtype=torch.float32)
            logits = []
            for p in range(1, SEQ_LEN + 1):
                eng._dbg = []
                list(eng.generate([toks[:p]], 1))
                logits.append(eng._dbg[0][0].numpy())
            eng._dbg = None
            greedy = [s[0] for s in eng.generate([toks], N_GREEDY)]
        out = os.path.join(here, f"{name}.npz")
        np.savez_compressed(out, logits=np.stack(logits).astype(np.float32),
                            greedy=np.array(greedy, dtype=np.int64), seed=np.int64(seed))
        print(name, "logits", np.stack(logits).shape, "greedy", greedy, "->", out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
