"""The error path of the tensor-core kernels' bounded waits, made to run without any fault: a test
build of each kernel (a short wait limit, and a flag that keeps its loading thread from requesting
anything) lets every other role's wait run out. The kernel must return by itself with a code in its
error word, ``gemm_tc_check`` must raise, and the next ordinary launch must be right again: tensor
memory was given back and the work counters were left in order. Nothing here traps, faults or
waits without a limit."""
import pytest
import torch

from dryft_challenge_htn_2026_b200.csrc import api, build

pytestmark = pytest.mark.gpu
DEV = "cuda"
TEST_BUILD = {"DK_TEST_STALL": 1, "DK_WAIT_CYCLES": "4000000LL"}      # about two milliseconds a wait


@pytest.fixture
def stalled(monkeypatch):
    """api._lib hands out the test builds of the two tensor-core sources; yields a switch for their flag."""
    real = api._lib
    libs = []

    def lib_for(source, defines=None):
        if source in ("gemm_tc.cu", "attention_tc.cu"):
            lib = real(source, dict(defines or {}, **TEST_BUILD))
            if lib not in libs:
                libs.append(lib)
            return lib
        return real(source, defines)

    monkeypatch.setattr(api, "_lib", lib_for)

    def switch(on):
        for source, defines in (("gemm_tc.cu", None), ("attention_tc.cu", {"HD": 128})):
            assert lib_for(source, defines).dk_test_stall(int(on)) == 0
    yield switch
    switch(False)
    torch.cuda.synchronize()


def test_a_product_whose_loads_never_come_reports_and_the_next_one_is_right(stalled):
    x = torch.randn(300, 512, device=DEV).to(torch.bfloat16)
    w = (torch.randn(640, 512, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    stalled(False)
    assert float((api.gemm_tc(x, w).float() - ref).abs().max()) <= 0.02 * float(ref.abs().max())
    api.gemm_tc_check()
    stalled(True)
    for plan, rows in ((None, 300), ((128, 2), 20)):                   # the prefill form and the decode form with slices of K
        api.gemm_tc(x[:rows].contiguous(), w, api.MODE_STORE, None, plan)
        torch.cuda.synchronize()                                       # the kernel came back by itself
        with pytest.raises(api.KernelError, match="bounded wait"):
            api.gemm_tc_check()
        api.gemm_tc_check()                                            # the error word was cleared
    stalled(False)
    out = api.gemm_tc(x, w)
    g = api.gemm_tc(x, torch.cat([w, w]), api.MODE_SILU)
    api.gemm_tc_check()
    assert float((out.float() - ref).abs().max()) <= 0.02 * float(ref.abs().max())
    want = ref / (1 + torch.exp(-ref)) * ref
    assert float((g.float() - want).abs().max()) <= 0.03 * float(want.abs().max())


def test_attention_whose_loads_never_come_reports_and_the_next_one_is_right(stalled):
    nh, nkv, hd, T = 4, 2, 128, 200
    q = torch.randn(T, nh * hd, device=DEV).to(torch.bfloat16)
    k_store = torch.randn(4, nkv, 64, hd, device=DEV).to(torch.bfloat16)
    v_store = torch.randn(4, nkv, 64, hd, device=DEV).to(torch.bfloat16)
    table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=DEV)
    tiles = torch.tensor([[0, 128], [0, 0]], dtype=torch.int32, device=DEV)
    cu_q = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    pos0 = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run():
        out = torch.zeros_like(q)
        api.attention_prefill_tc(q, out, k_store, v_store, tiles, cu_q, pos0, table, nh, nkv, hd, 0, hd ** -0.5)
        torch.cuda.synchronize()
        return out

    stalled(False)
    good = run()
    api.gemm_tc_check()
    stalled(True)
    run()
    with pytest.raises(api.KernelError, match="bounded wait"):
        api.gemm_tc_check()
    stalled(False)
    again = run()
    api.gemm_tc_check()
    assert torch.equal(again, good)                                    # the work counter and tensor memory are in order
    K = k_store[table[0].long()].permute(1, 0, 2, 3).reshape(nkv, 256, hd).float()
    V = v_store[table[0].long()].permute(1, 0, 2, 3).reshape(nkv, 256, hd).float()
    qf = q.float().view(T, nh, hd)
    for h in (0, 3):
        s = (qf[:, h] @ K[h // 2, :T].T) * hd ** -0.5
        s = s.masked_fill(torch.ones(T, T, device=DEV).triu(1).bool(), float("-inf"))
        want = torch.softmax(s, -1) @ V[h // 2, :T]
        assert float((good.float().view(T, nh, hd)[:, h] - want).abs().max()) <= 0.03 * float(want.abs().max())
