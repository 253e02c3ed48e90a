"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same operation, at
sizes other than the models' (odd row counts, widths that are no power of two, shuffled pages)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from dryft_challenge_htn_2026_b200.csrc import api

pytestmark = pytest.mark.gpu
DEV = "cuda"
PAGE = api.PAGE


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, ref, dtype, what=""):
    tol = (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(ref.abs().max()))
    err = float((got.float() - ref.float()).abs().max())
    assert err <= tol, f"{what}: max error {err} > {tol}"


def rms(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,V", [(1, 40, 50), (37, 2560, 300), (130, 72, 1000)])
def test_embed_rmsnorm(dtype, T, H, V):
    embed, w = rnd(V, H, dtype=dtype, seed=1), 1 + 0.1 * rnd(H, seed=2)
    tok = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    h = torch.empty(T, H, device=DEV)
    a = torch.empty(T, H, dtype=dtype, device=DEV)
    api.embed_rmsnorm(tok, embed, w, 1e-5, h, a)
    assert torch.equal(h, embed[tok.long()].float())
    close(a, rms(h, w, 1e-5), dtype, "embed_rmsnorm")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H", [(1, 64), (33, 2560), (70, 200), (130, 2560), (67, 512), (100, 4096), (8, 5120), (40, 8192), (3, 8200)])
def test_add_rmsnorm_and_row_gather(dtype, T, H):
    h0, delta, w = rnd(T, H, seed=3, scale=3.0), rnd(T, H, dtype=dtype, seed=4), 1 + 0.1 * rnd(H, seed=5)
    h = h0.clone()
    a = torch.empty(T, H, dtype=dtype, device=DEV)
    api.add_rmsnorm(h, delta, w, 1e-6, a)
    ref_h = h0 + delta.float()
    assert torch.allclose(h, ref_h, atol=1e-6)
    close(a, rms(ref_h, w, 1e-6), dtype, "add_rmsnorm")
    api.add_rmsnorm(h, None, w, 1e-6, a)                                  # norm only
    assert torch.allclose(h, ref_h, atol=1e-6)
    close(a, rms(ref_h, w, 1e-6), dtype, "rmsnorm")
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    h = h0.clone()
    ag = torch.empty(3, H, dtype=dtype, device=DEV)
    api.add_rmsnorm(h, delta, w, 1e-6, ag, rows)
    assert torch.equal(h, h0)                                             # gathering leaves h alone
    close(ag, rms(ref_h[rows.long()], w, 1e-6), dtype, "gathered add_rmsnorm")
    # split-K partial sums in place of the delta (every row count takes the few-rows kernel then, up to 8,192 columns)
    parts = rnd(3, T, H, seed=6)
    h = h0.clone()
    api.add_rmsnorm(h, api.Partial(parts), w, 1e-6, a)
    assert torch.allclose(h, h0 + parts.sum(0), atol=1e-5)
    close(a, rms(h0 + parts.sum(0), w, 1e-6), dtype, "add_rmsnorm(partial sums)")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    gu = rnd(45, 2 * 200, dtype=dtype, seed=6, scale=3.0)
    out = torch.empty(45, 200, dtype=dtype, device=DEV)
    api.silu_mul(gu, out)
    g, u = gu[:, :200].float(), gu[:, 200:].float()
    close(out, g / (1 + torch.exp(-g)) * u, dtype, "silu_mul")


# --------------------------------------------------------------------------- paged cache helpers
def paged_setup(lens_before, lens_new, nkv, hd, dtype, seed=0, extra_pages=3):
    """Random sequences with ``lens_before`` cached tokens and ``lens_new`` new ones, pages handed
    out in shuffled order. Returns dense k/v per sequence and the step's index arrays."""
    rs = np.random.RandomState(seed)
    n_seq = len(lens_new)
    total = [b + n for b, n in zip(lens_before, lens_new)]
    need = [(t + PAGE - 1) // PAGE for t in total]
    n_pages = sum(need) + extra_pages
    perm = rs.permutation(n_pages).tolist()
    width = max(need)
    table = -np.ones((n_seq, width), dtype=np.int32)
    for i, n in enumerate(need):
        table[i, :n] = [perm.pop() for _ in range(n)]
    row_seq = np.repeat(np.arange(n_seq), lens_new).astype(np.int32)
    row_pos = np.concatenate([np.arange(b, b + n) for b, n in zip(lens_before, lens_new)]).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum(lens_new)]).astype(np.int32)
    k_store = torch.zeros(n_pages, nkv, PAGE, hd, dtype=dtype, device=DEV)
    v_store = torch.zeros_like(k_store)
    dense_k = [rnd(t, nkv, hd, dtype=dtype, seed=seed * 100 + 2 * i) for i, t in enumerate(total)]
    dense_v = [rnd(t, nkv, hd, dtype=dtype, seed=seed * 100 + 2 * i + 1) for i, t in enumerate(total)]
    for i in range(n_seq):
        for p in range(total[i]):
            k_store[table[i, p // PAGE], :, p % PAGE] = dense_k[i][p]
            v_store[table[i, p // PAGE], :, p % PAGE] = dense_v[i][p]
    tiles = sorted(((lens_before[i] + min(q0 + 64, lens_new[i]), i, q0) for i in range(n_seq)
                    for q0 in range(0, lens_new[i], 64)), reverse=True)
    t = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return dict(table=t(table), row_seq=t(row_seq), row_pos=t(row_pos), cu_q=t(cu), pos0=t(lens_before),
                tiles=t([(x[1], x[2]) for x in tiles]).reshape(-1, 2), k_store=k_store, v_store=v_store,
                dense_k=dense_k, dense_v=dense_v, n_tok=int(cu[-1]))


def ref_attention(q, s, nh, nkv, hd, window, scale):
    """q [T, nh*hd] -> [T, nh*hd] in float32 from the dense per-sequence keys and values."""
    out = torch.zeros(q.shape[0], nh, hd, device=DEV)
    G = nh // nkv
    qf = q.float().view(-1, nh, hd)
    for t in range(q.shape[0]):
        i, p = int(s["row_seq"][t]), int(s["row_pos"][t])
        lo = max(0, p - window + 1) if window else 0
        K, V = s["dense_k"][i][lo:p + 1].float(), s["dense_v"][i][lo:p + 1].float()
        for h in range(nh):
            w = torch.softmax((K[:, h // G] @ qf[t, h]) * scale, 0)
            out[t, h] = w @ V[:, h // G]
    return out.view(q.shape[0], nh * hd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 1, 48), (3, 3, 128)])
def test_qk_norm_rope_write(dtype, nh, nkv, hd):
    before, new = [0, 70, 5], [9, 3, 130]
    s = paged_setup(before, new, nkv, hd, dtype, seed=7)
    s["k_store"].zero_(), s["v_store"].zero_()
    T = s["n_tok"]
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=8)
    qn, kn = 1 + 0.1 * rnd(hd, seed=9), 1 + 0.1 * rnd(hd, seed=10)
    cos, sin = plain.rope_tables(1e4, hd, 256)
    cos_h, sin_h = cos[:, :hd // 2].contiguous().to(DEV), sin[:, :hd // 2].contiguous().to(DEV)
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    # a padding row in the middle must leave no trace
    s["row_pos"][4] = -1
    api.qk_norm_rope_write(qkv, q_out, qn, kn, cos_h, sin_h, s["row_pos"], s["row_seq"], s["table"], s["k_store"],
                           s["v_store"], nh, nkv, hd, 1e-6)
    x = qkv.float().view(T, nh + 2 * nkv, hd)
    pos = s["row_pos"].long().clamp(min=0).cpu()
    c, sn = cos[pos].to(DEV), sin[pos].to(DEV)
    q_ref = plain.apply_rope(rms(x[:, :nh], qn, 1e-6), c, sn)
    k_ref = plain.apply_rope(rms(x[:, nh:nh + nkv], kn, 1e-6), c, sn)
    v_ref = x[:, nh + nkv:]
    keep = s["row_pos"] >= 0
    close(q_out.view(T, nh, hd)[keep], q_ref[keep], dtype, "q")
    for t in range(T):
        i, p = int(s["row_seq"][t]), int(s["row_pos"][t])
        if p < 0:
            continue
        page = int(s["table"][i, p // PAGE])
        close(s["k_store"][page, :, p % PAGE], k_ref[t], dtype, f"k row {t}")
        close(s["v_store"][page, :, p % PAGE], v_ref[t], dtype, f"v row {t}")
    # nothing else was written: the padding row's place and the unused pages are still zero
    written = sum(1 for t in range(T) if int(s["row_pos"][t]) >= 0)
    assert int((s["k_store"].float().abs().sum((1, 3)) > 0).sum()) == written
    # without norm, rotation or writing
    k_before = s["k_store"].clone()
    api.qk_norm_rope_write(qkv, q_out, None, None, None, None, s["row_pos"], s["row_seq"], s["table"], s["k_store"],
                           s["v_store"], nh, nkv, hd, 1e-6, write_kv=False)
    assert torch.equal(q_out.view(T, nh, hd)[keep], qkv.view(T, nh + 2 * nkv, hd)[:, :nh][keep])
    assert torch.equal(s["k_store"], k_before)
    # the norm alone into a dense tensor (the step before a position encoding that a part applies itself):
    # q and k normalised, v copied, the cache and q_out left alone
    dense = torch.zeros_like(qkv)
    q_before = q_out.clone()
    api.qk_norm_rope_write(qkv, None, qn, kn, None, None, s["row_pos"], s["row_seq"], s["table"], s["k_store"],
                           s["v_store"], nh, nkv, hd, 1e-6, dense_out=dense)
    d = dense.view(T, nh + 2 * nkv, hd)
    close(d[:, :nh][keep], rms(x[:, :nh], qn, 1e-6)[keep], dtype, "dense q")
    close(d[:, nh:nh + nkv][keep], rms(x[:, nh:nh + nkv], kn, 1e-6)[keep], dtype, "dense k")
    assert torch.equal(d[:, nh + nkv:][keep], qkv.view(T, nh + 2 * nkv, hd)[:, nh + nkv:][keep])
    assert torch.equal(s["k_store"], k_before) and torch.equal(q_out[keep], q_before[keep]) and float(dense[4].abs().sum()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 48, 0), (8, 2, 32, 50), (2, 2, 256, 0)])
def test_attention_generic(dtype, nh, nkv, hd, window):
    s = paged_setup([0, 100, 7, 64], [70, 3, 1, 1], nkv, hd, dtype, seed=11)
    q = rnd(s["n_tok"], nh * hd, dtype=dtype, seed=12)
    out = torch.empty_like(q)
    api.attention_generic(q, out, s["k_store"], s["v_store"], s["row_pos"], s["row_seq"], s["table"], nh, nkv, hd,
                          window, hd ** -0.5)
    close(out, ref_attention(q, s, nh, nkv, hd, window, hd ** -0.5), dtype, "attention_generic")


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (8, 2, 128, 0), (6, 2, 48, 0), (3, 1, 64, 90), (4, 4, 32, 10),
                                              (20, 1, 16, 0)])
def test_attention_prefill_bf16(nh, nkv, hd, window):
    s = paged_setup([0, 100, 0, 64, 130], [70, 150, 1, 64, 5], nkv, hd, torch.bfloat16, seed=13)
    q = rnd(s["n_tok"], nh * hd, dtype=torch.bfloat16, seed=14)
    out = torch.full_like(q, float("nan"))
    api.attention_prefill_bf16(q, out, s["k_store"], s["v_store"], s["tiles"], s["cu_q"], s["pos0"], s["table"], nh,
                               nkv, hd, window, hd ** -0.5)
    close(out, ref_attention(q, s, nh, nkv, hd, window, hd ** -0.5), torch.bfloat16, "attention_prefill_bf16")


@pytest.mark.parametrize("nh,nkv,hd,window,nsplit", [(4, 2, 16, 0, 1), (32, 8, 128, 0, 4), (6, 2, 48, 0, 8),
                                                     (3, 1, 64, 90, 2), (20, 1, 32, 0, 4), (4, 4, 256, 0, 16), (8, 2, 128, 0, 32),
                                                     (3, 1, 48, 0, 24)])
def test_attention_decode_bf16(nh, nkv, hd, window, nsplit):
    before = [0, 63, 64, 300, 1000, 5]
    s = paged_setup(before, [1] * len(before), nkv, hd, torch.bfloat16, seed=15)
    n = len(before)
    q = rnd(n + 2, nh * hd, dtype=torch.bfloat16, seed=16)           # two padding rows at the end
    row_pos = torch.cat([s["row_pos"], torch.tensor([-1, -1], dtype=torch.int32, device=DEV)])
    table = torch.cat([s["table"], -torch.ones(2, s["table"].shape[1], dtype=torch.int32, device=DEV)])
    out = torch.full_like(q, float("nan"))
    ws_acc, ws_ml = api.attention_decode_ws(n + 2, nh, hd, nsplit, DEV)
    want = ref_attention(q[:n], s, nh, nkv, hd, window, hd ** -0.5)
    api.attention_decode_bf16(q, out, s["k_store"], s["v_store"], row_pos, table, nh, nkv, hd, window, hd ** -0.5,
                              nsplit, ws_acc, ws_ml)
    close(out[:n], want, torch.bfloat16, "attention_decode_bf16")
    assert float(out[n:].float().abs().max()) == 0.0                 # padding rows give zeros, not garbage


@pytest.mark.parametrize("kernel", ["generic_f32", "prefill", "decode"])
def test_attention_finds_one_far_key_and_respects_the_window_edge(kernel):
    """One key among hundreds matches the query strongly, so the output must be that key's value:
    a kernel that drops a page, a split or the last key of a window shows it at once."""
    nh = nkv = 1
    hd = 32
    L = 777
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    for target, window, visible in [(3, 0, True), (700, 0, True), (L - 1, 0, True), (L - 50, 50, True),
                                    (L - 51, 50, False), (64 * 5, 0, True), (64 * 5 - 1, 0, True)]:
        s = paged_setup([L - 1], [1], nkv, hd, dtype, seed=17)
        page, slot = int(s["table"][0, target // PAGE]), target % PAGE
        direction = torch.zeros(hd, device=DEV)
        direction[5] = 1.0
        s["k_store"][:, :, :, :] *= 0.05
        s["k_store"][page, 0, slot] = (direction * 40).to(dtype)
        marker = torch.full((hd,), 7.0, device=DEV)
        s["v_store"][page, 0, slot] = marker.to(dtype)
        q = (direction * 10).to(dtype).view(1, hd)
        out = torch.empty_like(q)
        if kernel == "generic_f32":
            api.attention_generic(q, out, s["k_store"], s["v_store"], s["row_pos"], s["row_seq"], s["table"], 1, 1, hd,
                                  window, hd ** -0.5)
        elif kernel == "prefill":
            api.attention_prefill_bf16(q, out, s["k_store"], s["v_store"], s["tiles"], s["cu_q"], s["pos0"], s["table"],
                                       1, 1, hd, window, hd ** -0.5)
        else:
            ws = api.attention_decode_ws(1, 1, hd, 8, DEV)
            api.attention_decode_bf16(q, out, s["k_store"], s["v_store"], s["row_pos"], s["table"], 1, 1, hd, window,
                                      hd ** -0.5, 8, *ws)
        hit = float((out.float() - marker).abs().max()) < 0.1
        assert hit == visible, f"{kernel}: key {target} window {window}: expected visible={visible}"


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 300, 72), (64, 100, 200), (130, 96, 257)])
def test_sgemm(M, N, K):
    x, w = rnd(M, K, seed=18), rnd(N, K, seed=19)
    out = torch.empty(M, N, device=DEV)
    api.sgemm(x, w, out)
    ref = (x.double() @ w.double().T).float()
    close(out, ref, torch.float32, "sgemm")
    w2 = rnd(2 * N, K, seed=20, scale=0.3)
    api.sgemm(x, w2, out, api.MODE_SILU)
    y = x.double() @ w2.double().T
    g, u = y[:, :N], y[:, N:]
    close(out, (g / (1 + torch.exp(-g)) * u).float(), torch.float32, "sgemm silu")
    # a row's result does not depend on the rows beside it
    one = torch.empty(1, N, device=DEV)
    api.sgemm(x[M // 2:M // 2 + 1].contiguous(), w, one)
    api.sgemm(x, w, out)
    assert torch.equal(one[0], out[M // 2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_consumers_add_up_partial_sums(dtype):
    """add_rmsnorm and qk_norm_rope_write given split-K partial sums equal the same kernels given the sum."""
    T, H = 6, 200
    parts = rnd(3, T, H, seed=40)
    whole = parts.sum(0)
    h0, w = rnd(T, H, seed=41), 1 + 0.1 * rnd(H, seed=42)
    ha, hb = h0.clone(), h0.clone()
    aa, ab = torch.empty(T, H, dtype=dtype, device=DEV), torch.empty(T, H, dtype=dtype, device=DEV)
    api.add_rmsnorm(ha, api.Partial(parts), w, 1e-6, aa)
    assert torch.allclose(ha, h0 + whole, atol=1e-5)
    close(aa, rms(h0 + whole, w, 1e-6), dtype, "add_rmsnorm(partial)")
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    api.add_rmsnorm(hb, api.Partial(parts), w, 1e-6, ab, rows)
    close(ab[:2], rms((h0 + whole)[rows.long()], w, 1e-6), dtype, "gathered add_rmsnorm(partial)")
    nh, nkv, hd = 4, 2, 32
    s = paged_setup([0, 10], [3, 3], nkv, hd, dtype, seed=43)
    qparts = rnd(4, 6, (nh + 2 * nkv) * hd, seed=44)
    qn, kn = 1 + 0.1 * rnd(hd, seed=45), 1 + 0.1 * rnd(hd, seed=46)
    cos, sin = plain.rope_tables(1e4, hd, 64)
    cos_h, sin_h = cos[:, :hd // 2].contiguous().to(DEV), sin[:, :hd // 2].contiguous().to(DEV)
    outs = []
    for arg in (api.Partial(qparts), qparts.sum(0).to(dtype)):
        s["k_store"].zero_(), s["v_store"].zero_()
        q_out = torch.empty(6, nh * hd, dtype=dtype, device=DEV)
        api.qk_norm_rope_write(arg, q_out, qn, kn, cos_h, sin_h, s["row_pos"], s["row_seq"], s["table"], s["k_store"],
                               s["v_store"], nh, nkv, hd, 1e-6)
        outs.append((q_out.float(), s["k_store"].float().clone(), s["v_store"].float().clone()))
    for a, b in zip(*outs):
        close(a, b, dtype, "qk_norm_rope_write(partial)")


def test_kernels_refuse_what_they_cannot_do():
    x, w = rnd(17, 64, dtype=torch.bfloat16), rnd(32, 64, dtype=torch.bfloat16)
    with pytest.raises(api.KernelError):
        api.gemv_stream(x, w)                                   # more than 16 rows
    x, w = rnd(2, 24, dtype=torch.bfloat16), rnd(32, 24, dtype=torch.bfloat16)
    with pytest.raises(api.KernelError):
        api.gemv_stream(x, w)                                   # K no multiple of 16
    x, w = rnd(2, 12, dtype=torch.bfloat16), rnd(32, 12, dtype=torch.bfloat16)
    with pytest.raises(api.KernelError):
        api.gemm_tc(x, w)                                       # K no multiple of 8
    with pytest.raises(api.KernelError):
        api.attention_prefill_bf16(rnd(1, 24, dtype=torch.bfloat16), rnd(1, 24, dtype=torch.bfloat16), None, None,
                                   torch.zeros(1, 2, dtype=torch.int32, device=DEV),
                                   torch.zeros(2, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                   torch.zeros(1, 1, dtype=torch.int32, device=DEV), 1, 1, 24, 0, 1.0)


@pytest.mark.parametrize("V", [50, 4096, 151936])
def test_sampler_greedy_and_gumbel(V):
    n = 5
    logits = rnd(n, V, seed=23, scale=2.0)
    logits[1, 7] = logits[1, V - 1] = 50.0                           # a tie: the lowest index wins
    chunks = api.sample_chunks(V)
    ws_v, ws_i = torch.empty(n * chunks, device=DEV), torch.empty(n * chunks, dtype=torch.int32, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    temps = torch.zeros(n, device=DEV)
    seeds = torch.zeros(n, 2, dtype=torch.int32, device=DEV)
    pos = torch.tensor([3, 9, -1, 0, 100], dtype=torch.int32, device=DEV)
    api.sample(logits, temps, seeds, pos, None, ws_v, ws_i, out)
    ref = logits.argmax(-1).tolist()
    ref[1], ref[2] = 7, 0                                            # tie; padding row
    assert out.tolist() == ref and pos.tolist() == [3, 9, -1, 0, 100]
    api.sample(logits, temps, seeds, pos, None, ws_v, ws_i, out, advance=True)
    assert pos.tolist() == [4, 10, -1, 1, 101]
    if V > 5000:
        return
    # temperature: the kernel's choice is the plain Gumbel-max choice for (seed, position + 1)
    temps[:] = 0.7
    seed64 = [0x123456789ABCDEF0 + 977 * b for b in range(n)]
    from dryft_challenge_htn_2026_b200.sampling import seed_words
    seeds.copy_(torch.tensor([seed_words(s) for s in seed64], dtype=torch.int32))
    pos = torch.tensor([3, 9, 20, 0, 100], dtype=torch.int32, device=DEV)
    api.sample(logits, temps, seeds, pos, None, ws_v, ws_i, out)
    for b in range(n):
        want, z = plain.gumbel_argmax(logits[b].cpu(), 0.7, seed64[b], int(pos[b]) + 1)
        got = int(out[b])
        assert got == want or abs(z[got] - z[want]) < 1e-4, (b, got, want)
    # same seed, other position: other draws; frequencies follow softmax(logits / T)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device=DEV).repeat(4000, 1).contiguous()
    t4, s4 = torch.full((4000,), 1.0, device=DEV), torch.zeros(4000, 2, dtype=torch.int32, device=DEV)
    p4 = torch.arange(4000, dtype=torch.int32, device=DEV)
    o4 = torch.empty(4000, dtype=torch.int32, device=DEV)
    api.sample(small, t4, s4, p4, None, torch.empty(4000, device=DEV), torch.empty(4000, dtype=torch.int32, device=DEV), o4)
    freq = torch.bincount(o4.long(), minlength=4).float() / 4000
    assert float((freq.cpu() - torch.softmax(small[0].cpu(), 0)).abs().max()) < 0.03


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(64, 64), (300, 96), (200, 2560), (2560, 2448), (100, 4096), (136, 5120), (40, 5552), (48, 9728)])
def test_gemv_stream(M, N, K):
    """The streaming product against x.w^T: every mode, slices of K, few and many blocks, both block
    shapes (four streaming warps, eight for the longer rows of x)."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=51), rnd(N, K, dtype=torch.bfloat16, seed=52, scale=0.05)
    ref = x.float() @ w.float().T
    fits = lambda sk, warps: api._stream_smem(M, K, sk, warps) <= 227 * 1024
    for sk, blocks, warps in [(1, 296, 4), (1, 1, 4), (1, 5, 8), (1, 148, 8), (2, 296, 4), (4, 7, 8), (8, 296, 4)]:
        plan = (sk, blocks, warps)
        if not fits(sk, warps):
            with pytest.raises(api.KernelError):
                api.gemv_stream(x, w, None, api.MODE_STORE_F32, plan)
            continue
        r = api.gemv_stream(x, w, None, api.MODE_STORE_F32, plan)
        if sk > 1:
            assert isinstance(r, api.Partial) and tuple(r.ws.shape) == (sk, M, N)
            r = r.ws.sum(0)
        assert float((r - ref).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max())), plan
        if sk == 1:
            close(api.gemv_stream(x, w, None, api.MODE_STORE, plan), ref, torch.bfloat16, f"stream store {plan}")
            if N % 2 == 0:
                half = N // 2
                g, u = ref[:, :half], ref[:, half:]
                close(api.gemv_stream(x, w, None, api.MODE_SILU, plan), g / (1 + torch.exp(-g)) * u, torch.bfloat16,
                      f"stream silu {plan}")
    # the plan the model uses
    plan = api.stream_plan(M, N, K, api.MODE_STORE, allow_partial=True)
    r = api.gemv_stream(x, w, None, api.MODE_STORE, plan)
    close(r.sum() if isinstance(r, api.Partial) else r, ref, torch.bfloat16, "stream planned")
    # the rows of x of one slice must fit a block: beyond that the gated product has no plan, the plain one is cut
    assert api.stream_plan(M, N, 20000, api.MODE_SILU) is None and api.stream_plan(M, N, 20000, api.MODE_STORE, True)[0] >= 2
    if M <= 8:
        assert api.stream_plan(M, N, 5120, api.MODE_SILU) == (1, api.sm_count(), 8)
        assert api.stream_plan(M, N, 9728, api.MODE_SILU) == (1, api.sm_count(), 4)   # 8 rows of 9,728: one block of four warps
    else:
        assert api.stream_plan(M, N, 9728, api.MODE_SILU) is None


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (100, 300, 72), (300, 200, 136), (1000, 520, 2560), (65, 2560, 1024),
                                   (1157, 600, 20544)])
def test_gemm_tc(M, N, K):
    """The TMA + tcgen05 product against x.w^T in float32: full tiles, ragged edges in M, N and K,
    several tiles per block (persistent loop, both accumulators), plain and SiLU*up epilogues; and
    rows of x so long that the row tiles are walked in more than one group (ten row tiles in groups
    of eight: every tile once, none twice)."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=81), rnd(2 * N, K, dtype=torch.bfloat16, seed=82, scale=0.05 * min(1.0, (2560 / K) ** 0.5))
    ref = x.float() @ w.float().T
    close(api.gemm_tc(x, w[:N].contiguous()), ref[:, :N], torch.bfloat16, "gemm_tc")
    g, u = ref[:, :N], ref[:, N:]
    close(api.gemm_tc(x, w, api.MODE_SILU), g / (1 + torch.exp(-g)) * u, torch.bfloat16, "gemm_tc silu")
    for bn in (128, 144, 160, 192):                                   # the tile heights the planner picks for short prefill steps
        close(api.gemm_tc(x, w, api.MODE_SILU, None, (bn, 1)), g / (1 + torch.exp(-g)) * u, torch.bfloat16, f"gemm_tc silu, {bn} rows a tile")
    api.gemm_tc_check()
    with pytest.raises(api.KernelError):
        api.gemm_tc(rnd(70, 12, dtype=torch.bfloat16), rnd(8, 12, dtype=torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,hd,K,before,new,norm,rope", [
    (4, 2, 64, 264, [0, 100], [200, 129], True, True), (3, 1, 128, 512, [300, 0, 5], [140, 70, 1], True, True),
    (2, 2, 128, 72, [0], [130], False, True), (5, 1, 64, 136, [64, 0], [100, 100], True, False)])
def test_gemm_tc_qkv_epilogue(nh, nkv, hd, K, before, new, norm, rope):
    """The q/k/v projection with norm, rotation and cache write in its epilogue against the plain
    formulas in float32 on the unrounded product: q, and the rows of the paged cache it wrote; a
    padding row, a last tile that is not full (widths that are no multiple of 256), no norm, no
    rotation, and a layer that only reads the cache."""
    s = paged_setup(before, new, nkv, hd, torch.bfloat16, seed=95)
    T = s["n_tok"]
    x = rnd(T + 1, K, dtype=torch.bfloat16, seed=96)
    w = rnd((nh + 2 * nkv) * hd, K, dtype=torch.bfloat16, seed=97, scale=K ** -0.5)
    qn = 1 + 0.1 * rnd(hd, seed=98) if norm else None
    kn = 1 + 0.1 * rnd(hd, seed=99) if norm else None
    cos, sin = plain.rope_tables(1e4, hd, 600)
    cos_h, sin_h = cos[:, :hd // 2].contiguous().to(DEV), sin[:, :hd // 2].contiguous().to(DEV)
    row_pos = torch.cat([s["row_pos"], torch.tensor([-1], dtype=torch.int32, device=DEV)])     # one padding row
    row_seq = torch.cat([s["row_seq"], torch.zeros(1, dtype=torch.int32, device=DEV)])
    # plain formulas on the float32 product
    y = (x.float() @ w.float().t()).view(T + 1, nh + 2 * nkv, hd)
    def norm_rope(v, nw):
        if nw is not None:
            v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * nw
        if rope:
            c, sn = cos_h[row_pos[:T].long()][:, None, :], sin_h[row_pos[:T].long()][:, None, :]
            v1, v2 = v[..., :hd // 2], v[..., hd // 2:]
            v = torch.cat([v1 * c - v2 * sn, v2 * c + v1 * sn], -1)
        return v
    q_want = norm_rope(y[:T, :nh], qn)
    k_want, v_want = norm_rope(y[:T, nh:nh + nkv], kn), y[:T, nh + nkv:]
    k0, v0 = s["k_store"].clone(), s["v_store"].clone()
    q = torch.full((T + 1, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    api.gemm_tc_qkv(x, w, q, qn, kn, cos_h if rope else None, sin_h if rope else None, 1e-6, row_pos, row_seq, s["table"],
                    s["k_store"], s["v_store"], nh, nkv, hd)
    api.gemm_tc_check()
    close(q[:T].view(T, nh, hd), q_want, torch.bfloat16, "q")
    assert bool(torch.isnan(q[T:].float()).all())                    # nothing is stored for the padding row
    pages = s["table"][row_seq[:T].long(), (row_pos[:T] // 64).long()].long()
    slots = (row_pos[:T] % 64).long()
    close(s["k_store"][pages, :, slots], k_want, torch.bfloat16, "k in the cache")
    close(s["v_store"][pages, :, slots], v_want, torch.bfloat16, "v in the cache")
    touched = torch.zeros_like(k0, dtype=torch.bool)
    touched[pages, :, slots] = True
    assert torch.equal(s["k_store"][~touched], k0[~touched]) and torch.equal(s["v_store"][~touched], v0[~touched])
    # a layer that reads another layer's cache: q only
    s["k_store"].copy_(k0), s["v_store"].copy_(v0)
    api.gemm_tc_qkv(x, w, q, qn, kn, cos_h if rope else None, sin_h if rope else None, 1e-6, row_pos, row_seq, s["table"],
                    s["k_store"], s["v_store"], nh, nkv, hd, write_kv=False)
    close(q[:T].view(T, nh, hd), q_want, torch.bfloat16, "q, read-only")
    assert torch.equal(s["k_store"], k0) and torch.equal(s["v_store"], v0)


@pytest.mark.parametrize("nh,nkv,hd,window,before,new", [
    (2, 1, 128, 0, [0], [128]), (8, 2, 128, 0, [0, 100, 0, 64, 130], [70, 150, 1, 64, 5]), (4, 4, 64, 0, [0, 100], [200, 129]),
    (3, 1, 64, 90, [0, 100], [200, 129]), (6, 2, 128, 40, [300, 0], [140, 400]),
    (16, 4, 64, 0, [0, 100, 37, 64, 300], [700, 450, 300, 129, 1000]), (16, 2, 128, 200, [50, 0, 500], [900, 640, 1100])])
def test_attention_prefill_tc(nh, nkv, hd, window, before, new):
    """The tcgen05 prefill attention against the float32 reference: ragged chunks on top of cached
    tokens, several key blocks per tile (rescaling of O), group sizes 1..8, a window, padding rows;
    the last two cases have more (tile, head) items than the grid has blocks, so that a block works
    through several, with odd and even numbers of steps, on the same barriers."""
    s = paged_setup(before, new, nkv, hd, torch.bfloat16, seed=90)
    q = rnd(s["n_tok"], nh * hd, dtype=torch.bfloat16, seed=91)
    tiles = sorted(((before[i] + min(q0 + 128, new[i]), i, q0) for i in range(len(new)) for q0 in range(0, new[i], 128)),
                   reverse=True)
    tiles = torch.tensor([(t[1], t[2]) for t in tiles], dtype=torch.int32, device=DEV).reshape(-1, 2)
    out = torch.full_like(q, float("nan"))
    api.attention_prefill_tc(q, out, s["k_store"], s["v_store"], tiles, s["cu_q"], s["pos0"], s["table"], nh, nkv, hd, window,
                             hd ** -0.5)
    api.gemm_tc_check()
    close(out, ref_attention(q, s, nh, nkv, hd, window, hd ** -0.5), torch.bfloat16, "attention_prefill_tc")
    again = torch.full_like(q, float("nan"))
    api.attention_prefill_tc(q, again, s["k_store"], s["v_store"], tiles, s["cu_q"], s["pos0"], s["table"], nh, nkv, hd, window,
                             hd ** -0.5)
    assert torch.equal(again, out)                                   # which block took which item changes nothing
    assert all(int(c.abs().sum()) == 0 for c in api._attn_sched.values())   # the work counter is left at zero


@pytest.mark.parametrize("M,N,K", [(64, 6144, 2560), (33, 2560, 4096), (128, 2560, 9728), (17, 300, 520), (100, 1000, 1288),
                                   (40, 1002, 520)])
def test_gemm_tc_on_a_decode_step_of_17_to_128_rows(M, N, K):
    """One tile of rows, K in slices with float32 partial sums, weights requested before the wait
    for the previous kernel (programmatic launch on, a kernel in front); the epilogue through
    shared memory with whole 16-byte pieces of a row, and element by element where the width is no
    multiple of four (1,002 outputs, 501 gated ones)."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=80), rnd(N, K, dtype=torch.bfloat16, seed=81, scale=K ** -0.5)
    ref = x.float() @ w.float().t()
    api.set_pdl(True)
    try:
        plans = {api.skinny_tc_plan(M, N, K, api.MODE_STORE, True), (128, 1), (256, 1), (128, 2), (256, 3), (144, 2), (176, 1),
                 (208, 3), (240, 2)}
        for bn, sk in sorted(plans):
            if sk > 1 and (sk - 1) * (((K + 63) // 64 + sk - 1) // sk) >= (K + 63) // 64:
                continue
            x2 = x.clone()                                               # a kernel in front of the product
            r = api.gemm_tc(x2, w, api.MODE_STORE, None, (bn, sk))
            assert isinstance(r, api.Partial) == (sk > 1)
            close(r.sum() if sk > 1 else r, ref, torch.bfloat16, f"gemm_tc rows {M} plan {(bn, sk)}")
        r = api.gemm_tc(x, w, api.MODE_STORE_F32)
        assert r.dtype == torch.float32
        close(r, ref, torch.bfloat16, "gemm_tc float32 out")
        if N % 2 == 0:
            g, u = ref.chunk(2, dim=1)
            for bn in api.TC_TILE_HEIGHTS:
                close(api.gemm_tc(x, w, api.MODE_SILU, None, (bn, 1)), g / (1 + torch.exp(-g)) * u, torch.bfloat16,
                      f"gemm_tc silu, few rows, {bn} weight rows a tile")
        api.gemm_tc_check()
    finally:
        api.set_pdl(False)


def test_gemm_tc_decode_form_at_random_shapes_and_plans():
    """Forty random shapes (17 to 128 rows, widths and inner sizes that are multiples of 8 only, widths
    below one tile) with random tile heights and slice counts: plain and gated epilogues, partial sums."""
    rs = np.random.RandomState(123)
    api.set_pdl(True)
    try:
        for case in range(40):
            M = int(rs.randint(17, 129))
            N = int(rs.choice([8, 24, 100, 136, 300, 1000, 1002, 2560])) if case % 2 else int(rs.randint(1, 200)) * 8
            K = int(rs.randint(8, 400)) * 8
            bn = int(rs.choice(api.TC_TILE_HEIGHTS))
            kb = (K + 63) // 64
            sk = int(rs.randint(1, 9))
            while sk > 1 and (sk - 1) * ((kb + sk - 1) // sk) >= kb:
                sk -= 1
            x = rnd(M, K, dtype=torch.bfloat16, seed=1000 + case)
            w = rnd(2 * N, K, dtype=torch.bfloat16, seed=2000 + case, scale=K ** -0.5)
            ref = x.float() @ w.float().t()
            r = api.gemm_tc(x, w[:N].contiguous(), api.MODE_STORE, None, (bn, sk))
            close(r.sum() if sk > 1 else r, ref[:, :N], torch.bfloat16, f"case {case}: rows {M} width {N} inner {K} plan {(bn, sk)}")
            g, u = ref[:, :N], ref[:, N:]
            close(api.gemm_tc(x, w, api.MODE_SILU, None, (bn, 1)), g / (1 + torch.exp(-g)) * u, torch.bfloat16,
                  f"case {case} gated: rows {M} width {N} inner {K} tile {bn}")
        api.gemm_tc_check()
    finally:
        api.set_pdl(False)
