"""dk_sample_noalloc, the sampler entry point for callers that cannot allocate device memory (its
scratch is a fixed array inside the library), called through its exported C symbol and compared
with the ordinary sampler, which gets its scratch from the caller. Collected last on purpose: if
it fails, a run that stops at the first failure has already run everything else."""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

from dryft_challenge_htn_2026_b200.csrc import api, build
from dryft_challenge_htn_2026_b200.sampling import seed_words

pytestmark = pytest.mark.gpu


def _lib():
    lib = ctypes.CDLL(build.compile_lib("sample_noalloc.cu"))
    lib.dk_sample_noalloc.restype = c_int
    lib.dk_sample_noalloc.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    lib.dk_sample_noalloc_error.restype = ctypes.c_char_p
    lib.dk_sample_noalloc_error.argtypes = [c_int]
    return lib


def test_no_alloc_sampler_matches_the_ordinary_one_twice_in_a_row():
    lib = _lib()
    dev = "cuda"
    n, V = 7, 151936
    gen = torch.Generator().manual_seed(5)
    temps = torch.tensor([0.0, 0.8, 1.3, 0.0, 0.5, 2.0, 0.0], device=dev)
    seeds = torch.tensor([seed_words(0x9E3779B97F4A7C15 * (b + 1) & (2**64 - 1)) for b in range(n)], dtype=torch.int32, device=dev)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    chunks = api.sample_chunks(V)
    ws_v, ws_i = torch.empty(n * chunks, device=dev), torch.empty(n * chunks, dtype=torch.int32, device=dev)
    for call in range(2):                                              # the second call finds the first call's leftovers
        logits = (torch.randn(n, V, generator=gen) * 3).to(dev)
        pos_a = torch.tensor([4, 99, 0, -1, 7, 1000, 63], dtype=torch.int32, device=dev)
        pos_b = pos_a.clone()
        want = torch.full((n,), -5, dtype=torch.int32, device=dev)
        got = torch.full((n,), -7, dtype=torch.int32, device=dev)
        api.sample(logits, temps, seeds, pos_a, None, ws_v, ws_i, want, advance=True)
        err = lib.dk_sample_noalloc(logits.data_ptr(), n, V, temps.data_ptr(), seeds.data_ptr(), pos_b.data_ptr(), None,
                                    got.data_ptr(), 1, stream)
        assert err == 0, lib.dk_sample_noalloc_error(err).decode()
        torch.cuda.synchronize()
        assert got.tolist() == want.tolist()                           # same kernels, same arithmetic: same tokens
        assert pos_b.tolist() == pos_a.tolist()
        assert got[3].item() == 0 and got[0].item() == int(logits[0].argmax())


def test_no_alloc_sampler_refuses_what_does_not_fit():
    lib = _lib()
    t = torch.zeros(8, device="cuda")
    i = torch.zeros(8, dtype=torch.int32, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # 16385 rows of one chunk each: one more partial result than the built-in scratch holds
    err = lib.dk_sample_noalloc(t.data_ptr(), 16385, 8, t.data_ptr(), i.data_ptr(), i.data_ptr(), None, i.data_ptr(), 0, stream)
    assert err == -1 and b"16384" in lib.dk_sample_noalloc_error(err)
    err = lib.dk_sample_noalloc(None, 1, 8, t.data_ptr(), i.data_ptr(), i.data_ptr(), None, i.data_ptr(), 0, stream)
    assert err == -2
    torch.cuda.synchronize()


def test_calls_back_to_back_on_the_same_positions_and_on_rows_without_alignment():
    """Two calls in a row that advance the same positions, with programmatic dependent launch on (the
    second call's first kernel may start while the first call's last kernel, which moves the positions on,
    still runs): the second call draws at the advanced positions. And logits whose rows do not start on
    16-byte boundaries (an offset view) are read with narrower loads, with the same result."""
    lib = _lib()
    lib.dk_set_pdl.argtypes = [c_int]
    dev = "cuda"
    n, V = 5, 8192 + 4
    gen = torch.Generator().manual_seed(9)
    buf = (torch.randn(n * V + 1, generator=gen) * 2).to(dev)
    aligned, shifted = buf[:n * V].view(n, V), buf[1:].view(n, V)         # the second view starts 4 bytes off
    temps = torch.full((n,), 0.9, device=dev)
    seeds = torch.tensor([seed_words(77 + b) for b in range(n)], dtype=torch.int32, device=dev)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    chunks = api.sample_chunks(V)
    ws_v, ws_i = torch.empty(n * chunks, device=dev), torch.empty(n * chunks, dtype=torch.int32, device=dev)
    lib.dk_set_pdl(1)
    try:
        for logits in (aligned, shifted):
            pos = torch.tensor([3, 10, 0, 500, 64], dtype=torch.int32, device=dev)
            first = torch.empty(n, dtype=torch.int32, device=dev)
            second = torch.empty(n, dtype=torch.int32, device=dev)
            for out in (first, second):
                err = lib.dk_sample_noalloc(logits.data_ptr(), n, V, temps.data_ptr(), seeds.data_ptr(), pos.data_ptr(), None,
                                            out.data_ptr(), 1, stream)
                assert err == 0, lib.dk_sample_noalloc_error(err).decode()
            torch.cuda.synchronize()
            assert pos.tolist() == [5, 12, 2, 502, 66]
            for k, out in enumerate((first, second)):                      # each call against the ordinary sampler at its positions
                want = torch.empty(n, dtype=torch.int32, device=dev)
                at = torch.tensor([3 + k, 10 + k, k, 500 + k, 64 + k], dtype=torch.int32, device=dev)
                api.sample(logits.contiguous(), temps, seeds, at, None, ws_v, ws_i, want)
                torch.cuda.synchronize()
                assert out.tolist() == want.tolist(), (k, logits.data_ptr() % 16)
            assert first.tolist() != second.tolist()                       # another position: other draws
    finally:
        lib.dk_set_pdl(0)
