"""out = x . W^T for a weight [out, in] without bias: picks the kernel by dtype and row count.

float32: the CUDA-core sgemm for every size (a true 32-bit product). bfloat16: the skinny
tensor-core kernel that streams the weights once for up to 64 rows (decode), the library matrix
product for more rows (prefill; the reference uses the library there too, engine/fused.py:993-995)."""
import torch

from ..csrc import api

STORE, STORE_F32, SILU = api.MODE_STORE, api.MODE_STORE_F32, api.MODE_SILU


def linear(x, w, mode=STORE):
    """mode STORE: [M, N] in x's dtype; STORE_F32: float32 (logits); SILU: w = [gate; up] rows,
    returns silu(x.gate^T) * (x.up^T) of width N/2."""
    M, K = x.shape
    N = w.shape[0] // 2 if mode == SILU else w.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        api.sgemm(x, w, out, mode)
        return out
    if M <= api.GEMV_MAX_ROWS:
        out = torch.empty((M, N), dtype=torch.float32 if mode == STORE_F32 else torch.bfloat16, device=x.device)
        api.gemv_bf16(x, w, out, mode)
        return out
    if mode == STORE_F32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    y = torch.mm(x, w.t())
    if mode == SILU:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
        api.silu_mul(y, out)
        return out
    return y
