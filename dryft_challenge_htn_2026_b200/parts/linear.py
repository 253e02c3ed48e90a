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


def linear(x, w, mode=STORE, ctx=None, allow_partial=False, residual=None):
    """mode STORE: [M, N] in x's dtype; STORE_F32: float32 (logits); SILU: w = [gate; up] rows,
    returns silu(x.gate^T) * (x.up^T) of width N/2. ``ctx``: the step context; when it carries a
    weight prefetcher, the kernel asks (the head of) the matrix the step uses next into L2 while
    it runs. ``allow_partial``: the caller can take ``csrc.api.Partial`` (split-K
    partial sums, added up by the kernel that consumes them) instead of a tensor.
    ``x`` may be a ``csrc.api.Normed`` (a norm of the residual stream not computed yet): the
    streaming kernel applies it while it loads x, every other path computes it first.
    ``residual``: the float32 residual stream this product is to be added to. Where the kernel can
    add it in place, ``csrc.api.Added`` comes back; else the product, for the caller to add."""
    pf = getattr(ctx, "prefetcher", None)
    return _linear(x, w, mode, allow_partial, residual, pf.next_after(w) if pf is not None else None)


def _linear(x, w, mode, allow_partial, residual, prefetch):
    M, K = x.shape
    N = w.shape[0] // 2 if mode == SILU else w.shape[0]
    if isinstance(x, api.Normed):
        if x.dtype == torch.bfloat16 and M <= api.STREAM_BEST_ROWS and K % 16 == 0 and mode != STORE_F32:
            plan = api.stream_plan(M, N, K, mode, allow_partial)
            if plan is not None:
                return api.gemv_stream(x, w, None, mode, plan, prefetch=prefetch)
        x = x.tensor()
    if x.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        api.sgemm(x, w, out, mode)
        return out
    if M <= (api.STREAM_BEST_ROWS if K % 8 == 0 else api.STREAM_MAX_ROWS) and K % 16 == 0:
        fuse = residual is not None and mode == STORE
        plan = api.stream_plan(M, N, K, mode, allow_partial or fuse)
        if plan is not None:
            return api.gemv_stream(x, w, None, mode, plan, residual if fuse else None, prefetch)
    if M <= api.TC_SKINNY_MAX_ROWS and K % 8 == 0:
        # a decode step of 17 to 128 rows: weights streamed once by TMA, one 128-row tile of x,
        # K in slices so that the few weight tiles still cover the SMs
        return api.gemm_tc(x, w, mode, None, api.skinny_tc_plan(M, N, K, mode, allow_partial))
    if M <= api.GEMV_MAX_ROWS:
        return api.gemv_bf16(x, w, None, mode, api.gemv_plan(M, N, K, mode, allow_partial))
    if mode == STORE_F32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    if K % 8 == 0 and (mode == SILU or api.gemm_tc_fills_gpu(M, N)):
        return api.gemm_tc(x, w, mode)          # TMA + tcgen05, SiLU*up fused into the epilogue
    y = torch.mm(x, w.t())
    if mode == SILU:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
        api.silu_mul(y, out)
        return out
    return y
