"""Each part alone against the plain implementation's function for it, with sizes of its own."""
import pytest
import torch

import plain_qwen3 as plain
from dryft_challenge_htn_2026_b200.cache import Cache
from dryft_challenge_htn_2026_b200.config.specs import (AttentionSpec, GatedMLPSpec, LayerSpec, RMSNormSpec,
                                                        RotaryHalfSpec)
from dryft_challenge_htn_2026_b200.engine.batch import build_context
from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
from dryft_challenge_htn_2026_b200.parts.linear import SILU, STORE_F32, linear

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, ref, dtype, what=""):
    tol = (2e-5 if dtype == torch.float32 else 3e-2) * max(1.0, float(ref.abs().max()))
    err = float((got.float().cpu() - ref.float()).abs().max())
    assert err <= tol, f"{what}: max error {err} > {tol}"


def tensor(x, dtype):
    """Products of few rows may come back as split-K partial sums; the next kernel adds them up."""
    from dryft_challenge_htn_2026_b200.csrc import api
    return x.sum(dtype) if isinstance(x, api.Partial) else x


def bind(part, tensors, dtype):
    decls = {p.name: p for p in part.param_decls()}
    assert set(decls) == set(tensors)
    part.bind({k: v.to(DEV, torch.float32 if decls[k].keep_float32 else dtype) for k, v in tensors.items()})


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    part = build_part(RMSNormSpec(200, 1e-5), Runtime(DEV, dtype))
    w = 1 + 0.1 * rnd(200, seed=1)
    bind(part, {"weight": w}, dtype)
    h0, d = rnd(9, 200, seed=2, scale=2.0), rnd(9, 200, seed=3).to(dtype)
    h = h0.to(DEV)
    out = part.add_forward(h, d.to(DEV), torch.empty(9, 200, dtype=dtype, device=DEV))
    close(out, plain.rms_norm(h0 + d.float(), w, 1e-5), dtype, "RMSNorm")
    close(h, h0 + d.float(), torch.float32, "residual stream")


def test_rotary_tables_are_float32_angles():
    part = build_part(RotaryHalfSpec(48, 500000.0), Runtime(DEV, torch.bfloat16))
    cos, sin = part.tables(300)
    rc, rs = plain.rope_tables(500000.0, 48, 300)
    assert cos.dtype == torch.float32 and cos.shape[0] >= 300 and cos.shape[1] == 24
    assert float((cos[:300].cpu() - rc[:, :24]).abs().max()) < 2e-5 and float((sin[:300].cpu() - rs[:, :24]).abs().max()) < 2e-5
    assert part.tables(100)[0].data_ptr() == cos.data_ptr()          # no rebuild for a shorter need


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M", [1, 7, 64, 65, 200])
def test_linear_picks_a_kernel_by_rows_and_all_agree(dtype, M):
    x, w = rnd(M, 72, seed=4).to(DEV, dtype), rnd(2 * 104, 72, seed=5, scale=0.2).to(DEV, dtype)
    ref = x.float().cpu() @ w.float().cpu().T
    close(linear(x, w), ref, dtype, "linear")
    y = linear(x, w, STORE_F32)
    assert y.dtype == torch.float32
    close(y, ref, dtype, "linear f32 out")
    g, u = ref[:, :104], ref[:, 104:]
    close(linear(x, w, SILU), g / (1 + torch.exp(-g)) * u, dtype, "linear silu")


def mixer_weights(H, nh, nkv, hd, seed):
    p = "model.layers.0."
    return {
        p + "self_attn.q_proj.weight": rnd(nh * hd, H, seed=seed, scale=0.15),
        p + "self_attn.k_proj.weight": rnd(nkv * hd, H, seed=seed + 1, scale=0.15),
        p + "self_attn.v_proj.weight": rnd(nkv * hd, H, seed=seed + 2, scale=0.15),
        p + "self_attn.o_proj.weight": rnd(H, nh * hd, seed=seed + 3, scale=0.15),
        p + "self_attn.q_norm.weight": 1 + 0.1 * rnd(hd, seed=seed + 4),
        p + "self_attn.k_norm.weight": 1 + 0.1 * rnd(hd, seed=seed + 5),
    }


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,nh,nkv,hd,window", [(40, 5, 5, 16, None), (88, 6, 2, 32, None), (64, 4, 1, 64, 20)])
def test_attention_part_whole_then_token_by_token(dtype, H, nh, nkv, hd, window):
    spec = AttentionSpec(H, nh, nkv, hd, hd ** -0.5, RMSNormSpec(hd, 1e-6), RotaryHalfSpec(hd, 1e4), window)
    part = build_part(spec, Runtime(DEV, dtype))
    t = mixer_weights(H, nh, nkv, hd, 10)
    bind(part, {k.split("self_attn.")[1]: v for k, v in t.items()}, dtype)
    if dtype == torch.bfloat16:
        t = {k: v.to(dtype).float() for k, v in t.items()}
    sz = dict(nh=nh, nkv=nkv, hd=hd, eps=1e-6, theta=1e4)
    S = 90
    a = rnd(S, H, seed=20).to(dtype)
    ref, _ = plain.attention_mixer(a.float(), t, "model.layers.0.", sz, window)
    cache = Cache([part.cache_requests()], 64 * 4, 4, DEV)
    slot = cache.begin()
    # 70 tokens in one step, then 20 one at a time: the part never knows the difference
    ctx = build_context(cache, [(slot, [0] * 70, [])], DEV, plans=part.step_plans())
    out = [tensor(part.forward(ctx, cache.views(0), a[:70].to(DEV)), dtype)]
    cache.commit(slot, 70)
    for p in range(70, S):
        ctx = build_context(cache, [(slot, [0], [])], DEV, plans=part.step_plans())
        out.append(tensor(part.forward(ctx, cache.views(0), a[p:p + 1].to(DEV)), dtype))
        cache.commit(slot, 1)
    close(torch.cat(out), ref, dtype, "attention part")


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    part = build_part(GatedMLPSpec(72, 104), Runtime(DEV, dtype))
    t = {"gate_proj.weight": rnd(104, 72, seed=30, scale=0.2), "up_proj.weight": rnd(104, 72, seed=31, scale=0.2),
         "down_proj.weight": rnd(72, 104, seed=32, scale=0.2)}
    bind(part, dict(t), dtype)
    if dtype == torch.bfloat16:
        t = {k: v.to(dtype).float() for k, v in t.items()}
    a = rnd(11, 72, seed=33).to(dtype)
    ref = plain.gated_mlp(a.float(), {"mlp." + k: v for k, v in t.items()}, "")
    close(tensor(part.forward(None, a.to(DEV)), dtype), ref, dtype, "GatedMLP")


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    H, nh, nkv, hd, I = 56, 2, 1, 32, 120
    spec = LayerSpec("model.layers.0.", RMSNormSpec(H, 1e-5),
                     AttentionSpec(H, nh, nkv, hd, hd ** -0.5, RMSNormSpec(hd, 1e-5), RotaryHalfSpec(hd, 1e5), None),
                     RMSNormSpec(H, 1e-5), GatedMLPSpec(H, I))
    part = build_part(spec, Runtime(DEV, dtype))
    t = mixer_weights(H, nh, nkv, hd, 40)
    p = "model.layers.0."
    t.update({p + "input_layernorm.weight": 1 + 0.1 * rnd(H, seed=50), p + "post_attention_layernorm.weight": 1 + 0.1 * rnd(H, seed=51),
              p + "mlp.gate_proj.weight": rnd(I, H, seed=52, scale=0.2), p + "mlp.up_proj.weight": rnd(I, H, seed=53, scale=0.2),
              p + "mlp.down_proj.weight": rnd(H, I, seed=54, scale=0.2)})
    bind(part, {k[len(p):]: v for k, v in t.items()}, dtype)
    if dtype == torch.bfloat16:
        t = {k: (v if "norm" in k else v.to(dtype).float()) for k, v in t.items()}
    h0 = rnd(75, H, seed=55)
    ref, _ = plain.decoder_layer(h0, t, 0, dict(nh=nh, nkv=nkv, hd=hd, eps=1e-5, theta=1e5))
    cache = Cache([part.cache_requests()], 64 * 2, 2, DEV)
    slot = cache.begin()
    ctx = build_context(cache, [(slot, [0] * 75, [])], DEV, plans=part.step_plans())
    h = h0.to(DEV)
    pending = part.forward(ctx, h, None, cache.views(0))
    close(h + tensor(pending, dtype).float(), ref, dtype, "block")                   # the block leaves its last add to the next norm
