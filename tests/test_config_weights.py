"""Configuration, registry and weight-loading errors (no GPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import dryft_challenge_htn_2026_b200 as dk
from dryft_challenge_htn_2026_b200.config.specs import AttentionSpec, ScheduleEntry
from dryft_challenge_htn_2026_b200.engine.model import CausalLM
from helpers import TINY, make_folder, tiny_config


def test_config_reads_every_size_from_its_keys():
    for name, d in TINY.items():
        c = tiny_config(name)
        for k, v in d.items():
            assert getattr(c, k) == v
        spec = c.to_spec()
        assert len(spec.layers) == d["num_hidden_layers"] and spec.vocab_size == d["vocab_size"]
        m = spec.layers[0].mixer
        assert isinstance(m, AttentionSpec)
        assert (m.num_heads, m.num_kv_heads, m.head_dim) == (d["num_attention_heads"], d["num_key_value_heads"], d["head_dim"])
        assert m.scale == d["head_dim"] ** -0.5 and m.qk_norm.eps == d["rms_norm_eps"] and m.position.theta == d["rope_theta"]
    c = tiny_config("C")
    assert [l.mixer.window for l in c.to_spec().layers] == [None, None, 37, 37]


def test_config_defaults_and_both_rope_layouts():
    d = dict(TINY["A"], architectures=["Qwen3ForCausalLM"])
    del d["head_dim"]
    assert dk.config_from_dict(d).head_dim == 16                      # hidden_size // heads
    theta = d.pop("rope_theta")
    d["rope_parameters"] = {"rope_theta": theta, "rope_type": "default"}
    assert dk.config_from_dict(d).rope_theta == theta
    del d["rope_parameters"]
    with pytest.raises(dk.ConfigError, match="rope_theta"):
        dk.config_from_dict(d)


@pytest.mark.parametrize("patch, msg", [
    ({"architectures": ["LlamaForCausalLM"]}, "not registered"),
    ({"architectures": None}, "architectures"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rms_norm_eps": "tiny"}, "rms_norm_eps"),
    ({"vocab_size": 2.5}, "vocab_size"),
    ({"num_hidden_layers": 0}, "positive"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding_window"),
])
def test_config_errors(patch, msg):
    d = dict(TINY["A"], architectures=["Qwen3ForCausalLM"])
    d.update(patch)
    with pytest.raises(dk.ConfigError, match=msg):
        dk.config_from_dict(d)


def test_registry_takes_another_architecture():
    class Other(dk.Qwen3Config):
        architecture = "OtherForCausalLM"
    dk.register_architecture(Other)
    assert "OtherForCausalLM" in dk.architectures()
    c = dk.config_from_dict(dict(TINY["B"], architectures=["OtherForCausalLM"]))
    assert type(c) is Other and c.to_spec().architecture == "OtherForCausalLM"


def test_random_weights_folder_round_trip(tmp_path):
    folder = make_folder(tmp_path, "B", seed=3, dtype=torch.bfloat16)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]
    t = load_file(os.path.join(folder, "model.safetensors"))
    assert "lm_head.weight" in t and t["model.layers.2.mlp.down_proj.weight"].shape == (96, 200)
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    again = make_folder(tmp_path / "again", "B", seed=3, dtype=torch.bfloat16)
    t2 = load_file(os.path.join(again, "model.safetensors"))
    assert all(torch.equal(t[k], t2[k]) for k in t)
    other = load_file(os.path.join(make_folder(tmp_path / "other", "B", seed=4, dtype=torch.bfloat16), "model.safetensors"))
    assert not torch.equal(t["model.norm.weight"], other["model.norm.weight"])
    w = t["model.layers.0.input_layernorm.weight"].float()
    assert abs(w.mean() - 1) < 0.1 and t["model.embed_tokens.weight"].float().std() < 0.2


def test_loader_dtypes_and_tying(tmp_path):
    folder = make_folder(tmp_path, "A", dtype=torch.bfloat16)
    m = CausalLM(dk.config_from_folder(folder).to_spec(), torch.bfloat16, "cpu")
    dk.load_weights(m, folder)
    assert m.tied and m.head is m.embed and m.embed.dtype == torch.bfloat16
    assert m.blocks[0].mixer.w_qkv.shape == ((4 + 2 * 2) * 16, 64) and m.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert m.blocks[0].norm_in.weight.dtype == torch.float32          # norm weights are held in float32
    assert m.blocks[1].feed_forward.w_gate_up.shape == (256, 64)
    # a checkpoint without tie flag: the head tensor decides
    folderB = make_folder(tmp_path, "B")
    cfg = json.load(open(os.path.join(folderB, "config.json")))
    del cfg["tie_word_embeddings"]
    json.dump(cfg, open(os.path.join(folderB, "config.json"), "w"))
    mB = CausalLM(dk.config_from_folder(folderB).to_spec(), torch.float32, "cpu")
    dk.load_weights(mB, folderB)
    assert not mB.tied and mB.head is not mB.embed and mB.head.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.self_attn.k_norm.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(128, 60)
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    t["lm_head.weight"] = torch.zeros(256, 60)                        # a head in a tied model is accepted; its shape is checked
    save_file(t, path)
    m = CausalLM(dk.config_from_folder(folder).to_spec(), torch.float32, "cpu")
    with pytest.raises(dk.WeightError) as e:
        dk.load_weights(m, folder)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_norm.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in err.wrong_shape] == ["lm_head.weight", "model.layers.0.mlp.gate_proj.weight"]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "[128, 60]", "[128, 64]"):
        assert needle in text


def test_a_tied_checkpoint_that_ships_a_head_tensor_loads(tmp_path):
    """Published checkpoints of models whose config ties the head still hold lm_head.weight; the
    reference binds a head tensor whenever the files have one (engine/engine.py:290)."""
    folder = make_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, path)
    m = CausalLM(dk.config_from_folder(folder).to_spec(), torch.float32, "cpu")
    assert m.spec.tie_embeddings is True
    dk.load_weights(m, folder)
    assert torch.equal(m.head, m.embed)


def test_schedule_is_checked():
    spec = tiny_config("A").to_spec()
    import dataclasses
    bad = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0)))
    with pytest.raises(ValueError, match="written by two"):
        CausalLM(bad, torch.float32, "cpu")
    bad = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1, writes=False)))
    with pytest.raises(ValueError, match="never written"):
        CausalLM(bad, torch.float32, "cpu")
    ok = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0, writes=False), ScheduleEntry(1, 1)))
    assert len(CausalLM(ok, torch.float32, "cpu").entry_requests()) == 2
