"""out = x . W^T for a weight [out, in] without bias: picks the kernel by dtype and row count.

float32: the CUDA-core sgemm for every size (a true 32-bit product). bfloat16: up to 8 rows the
streaming kernel (cp.async rings, weights read once); up to 128 rows the TMA + tcgen05 kernel in its
decode form (one tile of rows, K in slices); for more rows (prefill) the same kernel, always for the
gated product (SiLU*up fused into its epilogue) and otherwise when its 128 x 256 tiles fill the
GPU's waves, else the library matrix product (the reference uses the library for all of these,
engine/fused.py:993-995)."""
import torch

from ..csrc import api

STORE, STORE_F32, SILU = api.MODE_STORE, api.MODE_STORE_F32, api.MODE_SILU


def linear(x, w, mode=STORE, allow_partial=False):
    """mode STORE: [M, N] in x's dtype; STORE_F32: float32 (logits); SILU: w = [gate; up] rows,
    returns silu(x.gate^T) * (x.up^T) of width N/2. ``allow_partial``: the caller can take
    ``csrc.api.Partial`` (split-K partial sums, added up by the kernel that consumes them) instead
    of a tensor."""
    M, K = x.shape
    N = w.shape[0] // 2 if mode == SILU else w.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        api.sgemm(x, w, out, mode)
        return out
    if M <= api.STREAM_BEST_ROWS and K % 16 == 0:
        plan = api.stream_plan(M, N, K, mode, allow_partial)
        if plan is not None:
            return api.gemv_stream(x, w, None, mode, plan)
    if M <= api.TC_SKINNY_MAX_ROWS:
        # a decode step of up to 128 rows: weights streamed once by TMA, one 128-row tile of x,
        # K in slices so that the few weight tiles still cover the SMs
        return api.gemm_tc(x, w, mode, None, api.skinny_tc_plan(M, N, K, mode, allow_partial))
    if mode == STORE_F32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    if mode == SILU:
        return api.gemm_tc(x, w, mode, None, api.gated_tc_plan(M, N))   # TMA + tcgen05, SiLU*up fused into the epilogue
    if api.gemm_tc_fills_gpu(M, N):
        return api.gemm_tc(x, w, mode)
    return torch.mm(x, w.t())
