"""Python entry points of the CUDA kernels: thin ctypes wrappers that take torch tensors.

Every function launches on torch's current CUDA stream and returns without synchronising, so
the calls can be captured in a CUDA graph. Arguments are checked here (device, dtype, contiguity,
the sizes a kernel supports); a kernel that cannot take a size raises ``KernelError`` rather than
compute something else. There is no CPU or library fallback behind these functions.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

PAGE = 64  # tokens per cache page; must equal DK_PAGE in common.cuh


class KernelError(RuntimeError):
    pass


_pdl = False


def set_pdl(on):
    """Programmatic dependent launch for every kernel launched from here on."""
    global _pdl
    _pdl = bool(on)
    for lib in list(build._libs.values()):
        lib.dk_set_pdl(int(_pdl))


_cuda_seen = False


def _lib(source, defines=None):
    global _cuda_seen
    if not _cuda_seen:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the kernels of this library run on an NVIDIA B200 (sm_100a) only")
        _cuda_seen = True
    key = (source, tuple(sorted((defines or {}).items())))
    fresh = key not in build._libs
    lib = build.load_lib(source, defines)
    if fresh:
        lib.dk_set_pdl.argtypes = [c_int]
        lib.dk_set_pdl(int(_pdl))
        lib.dk_error_string.restype = ctypes.c_char_p
    return lib


_sm_count = None


def sm_count():
    """Multiprocessors of the device the kernels run on; every launch plan is sized by it. Without
    a CUDA device (plans looked at on another machine) the B200's 148."""
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _sm_count


_launches = 0


def launch_count():
    """Kernels of this library launched so far through these wrappers (library products not counted)."""
    return _launches


def _check(lib, err, what, kernels=1):
    global _launches
    _launches += kernels
    if err != 0:
        msg = lib.dk_error_string(err).decode()
        raise KernelError(f"{what}: CUDA error {err} ({msg})")


# torch's current stream as a raw pointer. The call through torch.cuda.current_stream() builds a Stream
# object (3.6 us, a quarter of what a launch costs on the host: short prefill steps are bound by that);
# the raw getter takes 0.1 us. One device: its index is looked up once.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream_ptr():
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _stream():
    return c_void_p(_stream_ptr())


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _dt(t):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 or bfloat16")


def _need(t, name, dtype=None, dim=None):
    if t is None:
        return
    if not t.is_cuda or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


class Partial:
    """The output of a split-K product that has not been added up yet: float32 [slices, rows,
    cols]; the true value is the sum over slices. ``add_rmsnorm`` and ``qk_norm_rope_write`` take
    it in place of a tensor and add the slices up while they read; anything else calls ``sum()``."""

    def __init__(self, ws):
        self.ws = ws

    @property
    def shape(self):
        return self.ws.shape[1:]

    def sum(self, dtype=torch.bfloat16):
        out = torch.empty(self.shape, dtype=torch.bfloat16, device=self.ws.device)
        lib = _lib("gemm.cu")
        _check(lib, lib.dk_sum_partials(_p(self.ws), _p(out), c_longlong(out.numel()), self.ws.shape[0], _stream()),
               "sum_partials")
        return out.to(dtype)


def _parts(x):
    """(tensor or None, partial pointer, slices, stride) of an argument that may be a Partial."""
    if isinstance(x, Partial):
        return None, _p(x.ws), x.ws.shape[0], c_longlong(x.ws.shape[1] * x.ws.shape[2])
    return x, c_void_p(0), 0, c_longlong(0)


# ------------------------------------------------------------------------------------ row kernels
def embed_rmsnorm(tok, embed, norm_w, eps, h_out, a_out):
    """h_out[t] = embed[tok[t]] (float32); a_out[t] = rmsnorm(h_out[t]) * norm_w."""
    _need(tok, "tok", torch.int32, 1), _need(embed, "embed", None, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(h_out, "h_out", torch.float32, 2), _need(a_out, "a_out", embed.dtype, 2)
    lib = _lib("elementwise.cu")
    n, (V, H) = tok.numel(), embed.shape
    _check(lib, lib.dk_embed_rmsnorm(_dt(embed), _p(tok), _p(embed), _p(norm_w), c_float(eps), n, H, V, _p(h_out),
                                     _p(a_out), _stream()), "embed_rmsnorm")


def add_rmsnorm(h, delta, norm_w, eps, a_out, rows=None):
    """h += delta (delta may be None); a_out = rmsnorm(h) * norm_w. With ``rows`` (int32 indices)
    only those rows are normalised into a_out[0..len(rows)) and h is left unchanged."""
    delta, parts, n_parts, stride = _parts(delta)
    _need(h, "h", torch.float32, 2), _need(delta, "delta", a_out.dtype, 2), _need(norm_w, "norm_w", torch.float32, 1)
    _need(rows, "rows", torch.int32, 1), _need(a_out, "a_out", None, 2)
    lib = _lib("elementwise.cu")
    n = h.shape[0] if rows is None else rows.numel()
    _check(lib, lib.dk_add_rmsnorm(_dt(a_out), _p(h), _p(delta), parts, n_parts, stride, _p(rows), _p(norm_w),
                                   c_float(eps), n, h.shape[1], _p(a_out), _stream()), "add_rmsnorm")


def silu_mul(gu, out):
    """out[r, c] = silu(gu[r, c]) * gu[r, I + c] for gu [rows, 2I]."""
    _need(gu, "gu", None, 2), _need(out, "out", gu.dtype, 2)
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_silu_mul(_dt(gu), _p(gu), _p(out), c_longlong(gu.shape[0]), out.shape[1], _stream()), "silu_mul")


def gather_rows_f32(src, rows, out):
    _need(src, "src", torch.float32, 2), _need(rows, "rows", torch.int32, 1), _need(out, "out", torch.float32, 2)
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_gather_rows_f32(_p(src), _p(rows), _p(out), rows.numel(), src.shape[1], _stream()), "gather_rows")


def qk_norm_rope_write(qkv, q_out, q_norm_w, k_norm_w, cos, sin, row_pos, row_seq, page_table, k_store, v_store,
                       n_heads, n_kv_heads, head_dim, eps, write_kv=True, dense_out=None):
    """Per-head RMSNorm (weights may be None), rotate-half rotation (cos/sin [positions, hd/2]
    float32, may be None), q to q_out [T, nh*hd], k and v into the paged stores
    [pages, n_kv, PAGE, hd] at each token's position. Rows with position < 0 are skipped.
    With ``dense_out`` [T, (nh + 2 nkv) * hd] the heads go there instead (q and k normalised and
    rotated as asked, v copied) and neither q_out nor the cache is written."""
    width, n_tok = qkv.shape[1], qkv.shape[0]
    qkv, parts, n_parts, stride = _parts(qkv)
    if dense_out is not None:
        _need(dense_out, "dense_out", None, 2)
        if tuple(dense_out.shape) != (n_tok, width):
            raise KernelError(f"dense_out {tuple(dense_out.shape)} must have the projection's shape {(n_tok, width)}")
        q_out = dense_out if q_out is None else q_out
    _need(qkv, "qkv", q_out.dtype, 2), _need(q_out, "q_out", None, 2)
    _need(q_norm_w, "q_norm_w", torch.float32, 1), _need(k_norm_w, "k_norm_w", torch.float32, 1)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", q_out.dtype), _need(v_store, "v_store", q_out.dtype)
    if head_dim % 2 or head_dim > 256:
        raise KernelError(f"head size {head_dim} not supported: even, at most 256")
    if width != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"qkv width {width} != (nh + 2 nkv) * hd")
    lib = _lib("elementwise.cu")
    _check(lib, lib.dk_qk_norm_rope_write(_dt(q_out), _p(qkv), parts, n_parts, stride, _p(q_out), _p(dense_out), _p(q_norm_w),
                                          _p(k_norm_w), _p(cos), _p(sin), _p(row_pos), _p(row_seq), _p(page_table),
                                          page_table.shape[1], _p(k_store), _p(v_store), n_tok, n_heads, n_kv_heads,
                                          head_dim, c_float(eps), int(bool(write_kv)), _stream()), "qk_norm_rope_write")


# -------------------------------------------------------------------------------------- attention
def attention_generic(q, out, k_store, v_store, row_pos, row_seq, page_table, n_heads, n_kv_heads, head_dim, window,
                      scale):
    """Float32-arithmetic attention of every token row over its sequence's cached keys up to its
    own position (window: keys a query sees, 0 = all). Any phase; float32 or bfloat16 storage."""
    _need(q, "q", None, 2), _need(out, "out", q.dtype, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    if head_dim > 256 or n_heads % n_kv_heads:
        raise KernelError(f"attention: head size {head_dim} (max 256) / heads {n_heads}:{n_kv_heads} not supported")
    lib = _lib("attention_generic.cu")
    _check(lib, lib.dk_attention_generic(_dt(q), _p(q), _p(out), _p(k_store), _p(v_store), _p(row_pos), _p(row_seq),
                                         _p(page_table), page_table.shape[1], q.shape[0], n_heads, n_kv_heads,
                                         head_dim, int(window or 0), c_float(scale), _stream()), "attention_generic")


def _attn_lib(head_dim):
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"bfloat16 attention: head size {head_dim} not supported (multiples of 16 up to 256)")
    return _lib("attention_bf16.cu", {"HD": head_dim})


MMA_TILE_ROWS = 64   # queries a block of attention_prefill_bf16 takes


def attention_prefill_bf16(q, out, k_store, v_store, tiles, cu_q, seq_pos0, page_table, n_heads, n_kv_heads, head_dim,
                           window, scale):
    """Ragged causal attention of query chunks (tensor cores). tiles [n, 2] int32 = (sequence,
    first query of a 64-row tile within its chunk); cu_q [nseq+1]; seq_pos0 [nseq] cached length
    before the chunk."""
    _need(q, "q", torch.bfloat16, 2), _need(out, "out", torch.bfloat16, 2), _need(tiles, "tiles", torch.int32, 2)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} query heads are not a multiple of {n_kv_heads} kv heads")
    lib = _attn_lib(head_dim)
    _check(lib, lib.dk_attn_prefill_bf16(_p(q), _p(out), _p(k_store), _p(v_store), _p(tiles), tiles.shape[0], _p(cu_q),
                                         _p(seq_pos0), _p(page_table), page_table.shape[1], n_heads, n_kv_heads,
                                         int(window or 0), c_float(scale), _stream()), "attention_prefill_bf16")


DECODE_MAX_SPLITS = 32          # the merge kernel takes 4 x 32 parts a head


def decode_splits(n_seq, n_kv_heads, group, table_pages=0, max_splits=8, resident_blocks=None):
    """Number of key splits for decode attention, fixed for a batch size and a page-table width (it
    must not depend on sequence lengths, which change under a captured graph; the table width is
    the graph's own). While all blocks fit the GPU at once (two per SM with the three-deep rings):
    as many splits as keep it so, up to ``max_splits``, and for long tables up to DECODE_MAX_SPLITS
    while a split keeps 16 pages (one sequence of 32,768 tokens in 8 splits of its 8 kv heads kept
    64 of 296 block slots busy: 0.55 of the copy peak for the step). Beyond that: enough for about
    six waves of blocks, which evens out sequences of unequal lengths (measured at batch 64: 133 us
    unsplit, 115 us in four splits)."""
    if resident_blocks is None:
        resident_blocks = 2 * sm_count()
    blocks = n_seq * n_kv_heads * ((group + 15) // 16)
    if blocks <= resident_blocks:
        room = resident_blocks // blocks
        return max(1, min(max_splits, room), min(DECODE_MAX_SPLITS, room, table_pages // 16))
    return max(1, min(max_splits, -(-6 * resident_blocks // blocks)))


def attention_decode_ws(n_seq, n_heads, head_dim, nsplit, device):
    """Scratch for attention_decode_bf16: float32 partial outputs and (max, sum) pairs, one per warp
    of every block: 4 * nsplit a head."""
    parts = 4 * nsplit
    return (torch.empty(n_seq * n_heads * parts * head_dim, dtype=torch.float32, device=device),
            torch.empty(n_seq * n_heads * parts * 2, dtype=torch.float32, device=device))


def attention_decode_bf16(q, out, k_store, v_store, row_pos, page_table, n_heads, n_kv_heads, head_dim, window, scale,
                          nsplit, ws_acc, ws_ml):
    """One query token per sequence over its cached keys [.., row_pos] (tensor cores). The keys are
    split over ``nsplit`` blocks of four warps; every warp leaves a partial result and a second
    kernel merges the 4 * nsplit of a head."""
    _need(q, "q", torch.bfloat16, 2), _need(out, "out", torch.bfloat16, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(page_table, "page_table", torch.int32, 2)
    _need(ws_acc, "ws_acc", torch.float32), _need(ws_ml, "ws_ml", torch.float32)
    n_seq = q.shape[0]
    if not 1 <= nsplit <= DECODE_MAX_SPLITS:
        raise KernelError(f"attention_decode_bf16: {nsplit} splits, the merge takes 1 to {DECODE_MAX_SPLITS}")
    if ws_acc is None or ws_ml is None or ws_acc.numel() < n_seq * n_heads * 4 * nsplit * head_dim \
            or ws_ml.numel() < n_seq * n_heads * 4 * nsplit * 2:
        raise KernelError("attention_decode_bf16: scratch too small for this batch and split count")
    lib = _attn_lib(head_dim)
    _check(lib, lib.dk_attn_decode_bf16(_p(q), _p(out), _p(ws_acc), _p(ws_ml), _p(k_store), _p(v_store), _p(row_pos),
                                        _p(page_table), page_table.shape[1], n_seq, n_heads, n_kv_heads,
                                        int(window or 0), c_float(scale), nsplit, _stream()), "attention_decode_bf16", 2)


# ---------------------------------------------------------------------------------------- products
MODE_STORE, MODE_STORE_F32, MODE_SILU = 0, 1, 2


def sgemm(x, w, out, mode=MODE_STORE):
    """float32 out = x . w^T on CUDA cores; mode MODE_SILU: w = [gate; up], out = silu(g) * u."""
    _need(x, "x", torch.float32, 2), _need(w, "w", torch.float32, 2), _need(out, "out", torch.float32, 2)
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N if mode == MODE_SILU else N), K) or out.shape[0] != M:
        raise KernelError(f"sgemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
    lib = _lib("gemm.cu")
    _check(lib, lib.dk_sgemm(_p(x), _p(w), _p(out), M, N, K, mode, _stream()), "sgemm")


# ---------------------------------------------------------------------------------------- sampling
def sample_chunks(vocab):
    return _lib("sampling.cu").dk_sample_chunks(vocab)


def sample(logits, temperature, seeds, pos, rows, ws_val, ws_idx, out_tok, advance=False):
    """out_tok[b] = argmax (temperature 0) or Gumbel-max draw of logits[b]. temperature [n]
    float32, seeds [n, 2] int32 (low, high word of each row's 64-bit seed), pos int32 positions
    indexed through ``rows`` (or directly when rows is None); the draw's counter is that position
    + 1, the place the new token will take. ``advance`` moves those positions on by one."""
    _need(logits, "logits", torch.float32, 2), _need(temperature, "temperature", torch.float32, 1)
    _need(seeds, "seeds", torch.int32, 2), _need(pos, "pos", torch.int32, 1), _need(rows, "rows", torch.int32, 1)
    _need(ws_val, "ws_val", torch.float32), _need(ws_idx, "ws_idx", torch.int32), _need(out_tok, "out_tok", torch.int32, 1)
    n, V = logits.shape
    lib = _lib("sampling.cu")
    need = n * lib.dk_sample_chunks(V)
    if ws_val.numel() < need or ws_idx.numel() < need:
        raise KernelError("sample: scratch too small")
    _check(lib, lib.dk_sample(_p(logits), n, V, _p(temperature), _p(seeds), _p(pos), _p(rows), _p(ws_val), _p(ws_idx),
                              _p(out_tok), int(bool(advance)), _stream()), "sample", 2)


# ------------------------------------------------------------------- streaming product (M <= 16)
STREAM_MAX_ROWS = 16
# rows up to which the streaming product is the fastest: with 9 to 16 rows its copy of x doubles and
# the tensor-core product in its decode form wins (measured at 12, 16, 17)
STREAM_BEST_ROWS = 8
_STREAM_SMEM_BLOCK = 227 * 1024              # dynamic shared memory one block may ask for
_STREAM_SMEM_PAIR = (228 * 1024) // 2 - 1024  # ... and what each of two blocks sharing an SM may use


def _stream_smem(rows, K, sk, warps):
    """Shared memory of a block of the streaming product: ``warps`` two-deep rings of 16 weight rows
    x 256 columns, two buffers of the warps' sums, and the rows (8 or 16) of one slice of x. Must
    equal smem_bytes() in gemv_stream.cu."""
    mr = 8 if rows <= 8 else 16
    per = ((K + sk - 1) // sk + 15) // 16 * 16
    return warps * 2 * 16 * (256 * 2 + 16) + 2 * warps * 16 * mr * 4 + mr * (per * 2 + 16)


def stream_plan(M, N, K, mode, allow_partial=False):
    """(slices of K, blocks, streaming warps a block) for gemv_stream, or None if it cannot take
    the shape. Four warps and two persistent blocks per SM while the rows of x leave room for two
    blocks; for a longer K eight warps and one block per SM (as many bytes in flight); beyond that
    K is cut into slices, which needs a caller that takes partial sums (never the SiLU epilogue).
    With partial sums allowed K is cut so that the blocks fill the SMs' shared memory with their
    rings, and further while there are fewer than two tiles per block (more slices cost the
    consumer more partial sums to add)."""
    sms = sm_count()

    def shape(sk):                            # (warps, blocks, whether the SMs' shared memory is full of rings)
        if _stream_smem(M, K, sk, 4) <= _STREAM_SMEM_PAIR:
            return 4, 2 * sms, True
        if _stream_smem(M, K, sk, 8) <= _STREAM_SMEM_BLOCK:
            return 8, sms, True
        if _stream_smem(M, K, sk, 4) <= _STREAM_SMEM_BLOCK:
            return 4, sms, False              # one block of four warps an SM: half the bytes in flight
        return None

    sk = 1
    while shape(sk) is None:
        sk *= 2
        if sk > 64:
            return None
    can_slice = allow_partial and mode != MODE_SILU
    if sk > 1 and not can_slice:
        return None
    if can_slice:
        # two blocks of four warps an SM where up to four slices allow it (what the kernel was tuned on);
        # else the fewest slices that fill the SMs' shared memory at all, rather than half-empty SMs
        pair = next((k for k in (1, 2, 4) if k >= sk and shape(k)[:2] == (4, 2 * sms)), None)
        full = next((k for k in (1, 2, 4, 8) if k >= sk and shape(k)[2]), None)
        sk = pair or full or sk
        tiles = (N + 15) // 16
        while sk < 8 and tiles * sk < 2 * shape(sk)[1] and K // (sk * 2) >= 512 and shape(sk * 2)[2]:
            sk *= 2
    warps, blocks, _ = shape(sk)
    return sk, blocks, warps


def gemv_stream(x, w, out=None, mode=MODE_STORE, plan=None):
    """The weight-streaming skinny product (asynchronous copies into shared-memory rings,
    tensor-core multiply) for at most 16 rows of x and K a multiple of 16. Returns ``out`` [M, N]
    (bfloat16 for MODE_STORE and MODE_SILU, float32 for MODE_STORE_F32), or, when the plan splits K
    (plan[0] > 1), a ``Partial``."""
    _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _need(out, "out", None, 2)
    M, K = x.shape
    N = w.shape[0] // 2 if mode == MODE_SILU else w.shape[0]
    if M > STREAM_MAX_ROWS or K % 16:
        raise KernelError(f"gemv_stream: {M} rows (max {STREAM_MAX_ROWS}) / inner size {K} (multiple of 16) not supported")
    if w.shape[1] != K:
        raise KernelError(f"gemv_stream: shapes x{tuple(x.shape)} w{tuple(w.shape)} do not match")
    sk, blocks, warps = plan or stream_plan(M, N, K, mode) or (0, 0, 0)
    if sk < 1 or blocks < sk or warps not in (4, 8) or _stream_smem(M, K, sk, warps) > _STREAM_SMEM_BLOCK:
        raise KernelError(f"gemv_stream: K = {K} in {sk} slices on {blocks} blocks of {warps} warps is not supported "
                          f"(the {M} rows of a slice of x must fit a block's shared memory, and there is a block per slice at least)")
    ws = None
    if sk > 1:
        if mode == MODE_SILU:
            raise KernelError("gemv_stream: the SiLU epilogue cannot be split over K")
        ws = torch.empty((sk, M, N), dtype=torch.float32, device=w.device)
    else:
        want = torch.float32 if mode == MODE_STORE_F32 else torch.bfloat16
        if out is None:
            out = torch.empty((M, N), dtype=want, device=w.device)
        elif out.dtype != want or tuple(out.shape) != (M, N):
            raise KernelError(f"gemv_stream: out {tuple(out.shape)} {out.dtype} does not fit mode {mode}")
    lib = _lib("gemv_stream.cu")
    _check(lib, lib.dk_gemv_stream(_p(x), _p(w), _p(out), _p(ws), M, N, K, mode, sk, blocks, warps, _stream()), "gemv_stream")
    return Partial(ws) if sk > 1 else out


# ------------------------------------------------------------- tensor-core product for many rows
_tc_err = None


def gemm_tc(x, w, mode=MODE_STORE, out=None, plan=None):
    """out = x . w^T (mode MODE_STORE, MODE_STORE_F32) or silu(x . gate^T) * (x . up^T) (mode
    MODE_SILU, w = [gate; up]) on tcgen05 tensor cores, TMA-fed, float32 accumulation in tensor
    memory. ``plan`` = (weight rows per tile, one of TC_TILE_HEIGHTS; slices of K): with more than
    one slice (mode MODE_STORE) a ``Partial`` comes back instead of a tensor."""
    global _tc_err
    _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _need(out, "out", None, 2)
    M, K = x.shape
    N = w.shape[0] // 2 if mode == MODE_SILU else w.shape[0]
    bn, sk = plan or (256, 1)
    if K % 8 or w.shape[1] != K or mode not in (MODE_STORE, MODE_STORE_F32, MODE_SILU) \
            or bn not in TC_TILE_HEIGHTS:
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} mode {mode} not supported (K % 8 == 0)")
    kb = (K + 63) // 64
    if sk < 1 or (sk > 1 and (mode != MODE_STORE or (sk - 1) * ((kb + sk - 1) // sk) >= kb)):
        raise KernelError(f"gemm_tc: {sk} slices of K = {K} in mode {mode} not supported")
    ws = None
    if sk > 1:
        ws = torch.empty((sk, M, N), dtype=torch.float32, device=x.device)
    elif mode == MODE_STORE_F32:
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        ws = out
    elif out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    want = torch.float32 if mode == MODE_STORE_F32 else torch.bfloat16
    if sk == 1 and (out.dtype != want or tuple(out.shape) != (M, N)):
        raise KernelError(f"gemm_tc: out {tuple(out.shape)} {out.dtype} does not fit mode {mode}")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=x.device)
    lib = _lib("gemm_tc.cu")
    _check(lib, lib.dk_gemm_tc(_p(x), _p(w), _p(None if ws is not None else out), M, N, K,
                               MODE_STORE if mode == MODE_STORE_F32 else mode, _p(_tc_err), sk, _p(ws), bn, _stream()),
           "gemm_tc")
    return Partial(ws) if sk > 1 else out


TC_QKV_HEAD_DIMS = (64, 128)


def gemm_tc_qkv(x, w, q_out, q_norm_w, k_norm_w, cos, sin, eps, row_pos, row_seq, page_table, k_store, v_store, n_heads,
                n_kv_heads, head_dim, write_kv=True):
    """The fused q/k/v projection x . [Wq; Wk; Wv]^T of a prefill step with ``qk_norm_rope_write``
    in the epilogue of the tensor-core product: the float32 accumulator rows go through the per-head
    norm and the rotation, q to ``q_out``, k and v into the paged cache; the projection itself is
    never written. Head sizes 64 and 128; arguments as ``qk_norm_rope_write``."""
    global _tc_err
    _need(x, "x", torch.bfloat16, 2), _need(w, "w", torch.bfloat16, 2), _need(q_out, "q_out", torch.bfloat16, 2)
    _need(q_norm_w, "q_norm_w", torch.float32, 1), _need(k_norm_w, "k_norm_w", torch.float32, 1)
    _need(cos, "cos", torch.float32, 2), _need(sin, "sin", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1), _need(row_seq, "row_seq", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16), _need(v_store, "v_store", torch.bfloat16)
    M, K = x.shape
    if head_dim not in TC_QKV_HEAD_DIMS or K % 8 or tuple(w.shape) != ((n_heads + 2 * n_kv_heads) * head_dim, K) \
            or tuple(q_out.shape) != (M, n_heads * head_dim) or row_pos.numel() < M or row_seq.numel() < M:
        raise KernelError(f"gemm_tc_qkv: x{tuple(x.shape)} w{tuple(w.shape)} heads {n_heads}:{n_kv_heads} of {head_dim} "
                          "not supported (head size 64 or 128, K % 8 == 0)")
    if cos is not None and (cos.shape[1] != head_dim // 2 or sin.shape != cos.shape):
        raise KernelError("gemm_tc_qkv: angle tables must be [positions, head_dim / 2]")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=x.device)
    lib = _lib("gemm_tc.cu")
    _check(lib, lib.dk_gemm_tc_qkv(_p(x), _p(w), M, K, _p(_tc_err), _p(q_out), _p(k_store), _p(v_store), _p(q_norm_w),
                                   _p(k_norm_w), _p(cos), _p(sin), _p(row_pos), _p(row_seq), _p(page_table),
                                   page_table.shape[1], n_heads, n_kv_heads, head_dim, c_float(eps), int(bool(write_kv)),
                                   _stream()), "gemm_tc_qkv")


TC_SKINNY_MAX_ROWS = 128


TC_TILE_HEIGHTS = (128, 144, 160, 176, 192, 208, 224, 240, 256)   # weight rows a tile of gemm_tc


def skinny_tc_plan(M, N, K, mode, allow_partial=False):
    """(weight rows per tile, slices of K) for gemm_tc on a decode step of up to 128 rows. A unit of
    work is (tile, slice), with a block of its own while the units fit the SMs; all blocks stream
    at once, so the step takes as long as its largest unit: tile height x blocks of 64 columns in
    a slice (x waves, should the tiles alone exceed the SMs). The plan with the smallest such unit
    wins; among plans within 3 % of it the one with the fewest slices (partial sums are written and
    added up again), then the larger tile. Slices hold at least 8 blocks of 64 columns (fewer
    cannot keep the load ring busy). The gated product has no slices (SiLU needs whole sums)."""
    kb = (K + 63) // 64
    sms = sm_count()
    if mode == MODE_SILU:
        def span(bn):
            tiles = (N + bn // 2 - 1) // (bn // 2)
            return bn * -(-tiles // sms)
        return min(TC_TILE_HEIGHTS, key=lambda bn: (span(bn), bn)), 1
    if mode != MODE_STORE or not allow_partial:
        return 256, 1
    plans = []
    for bn in TC_TILE_HEIGHTS:
        tiles = (N + bn - 1) // bn
        sk = max(1, min(sms // tiles, kb // 8))
        while sk > 1 and (sk - 1) * ((kb + sk - 1) // sk) >= kb:
            sk -= 1
        waves = -(-tiles * sk // sms)
        plans.append((bn * ((kb + sk - 1) // sk) * waves, sk, bn))
    least = min(p[0] for p in plans)
    _, sk, bn = min((p for p in plans if p[0] <= 1.03 * least), key=lambda p: (p[1], p[0], -p[2]))
    return bn, sk


def gated_tc_plan(M, N):
    """Weight rows per tile for the gated product of a prefill step (gemm_tc, MODE_SILU; N outputs).
    One persistent block an SM works through the tiles in waves, and a step takes waves x what a
    wave of that tile costs. Measured at 512 to 8,192 rows of three model sizes: a wave of 192-row
    tiles costs 0.86 of a wave of 256-row tiles, and lower tiles no less than that (their share of
    the rows of x per output grows), so the choice is between those two: 512 rows of the benchmark
    model are 304 tiles of 256 (3 waves) or 408 of 192 (3 waves at 0.86)."""
    sms = sm_count()
    m_tiles = (M + 127) // 128

    def cost(bn, wave):
        tiles = m_tiles * ((N + bn // 2 - 1) // (bn // 2))
        return -(-tiles // sms) * wave
    return (192 if cost(192, 0.86) < cost(256, 1.0) else 256), 1


def gemm_tc_fills_gpu(M, N, min_fill=0.8):
    """Whether gemm_tc's 128 x 256 output tiles, one persistent block per SM, keep the last wave
    at least ``min_fill`` full on average; below that the library's smaller tiles win."""
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    waves = tiles / sm_count()
    return waves / -(-tiles // sm_count()) >= min_fill


def gemm_tc_check():
    """Raises if a bounded wait inside gemm_tc or attention_prefill_tc ran out since the last check (synchronises)."""
    if _tc_err is not None:
        code = int(_tc_err.item())
        if code:
            _tc_err.zero_()
            for t in _attn_sched.values():
                t.zero_()
            raise KernelError(f"gemm_tc: a bounded wait ran out (code {code}); its results are not valid")


# --------------------------------------------------------------- tensor-core prefill attention
TC_ATTENTION_HEAD_DIMS = (64, 128)
TC_TILE_ROWS = 128
_attn_sched = {}


def attention_prefill_tc(q, out, k_store, v_store, tiles, cu_q, seq_pos0, page_table, n_heads, n_kv_heads, head_dim, window,
                         scale):
    """Ragged causal attention of query chunks on tcgen05 tensor cores (head sizes 64 and 128).
    Arguments as ``attention_prefill_bf16`` except that ``tiles`` lists 128-row tiles."""
    global _tc_err
    _need(q, "q", torch.bfloat16, 2), _need(out, "out", torch.bfloat16, 2), _need(tiles, "tiles", torch.int32, 2)
    _need(cu_q, "cu_q", torch.int32, 1), _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2), _need(k_store, "k_store", torch.bfloat16, 4)
    if head_dim not in TC_ATTENTION_HEAD_DIMS or n_heads % n_kv_heads:
        raise KernelError(f"attention_prefill_tc: head size {head_dim} (64 or 128) / heads {n_heads}:{n_kv_heads} not supported")
    if _tc_err is None:
        _tc_err = torch.zeros(1, dtype=torch.int32, device=q.device)
    stream = _stream_ptr()
    sched = _attn_sched.get(stream)          # the kernel's work counter: launches of one stream share it, in turn
    if sched is None:
        sched = _attn_sched[stream] = torch.zeros(2, dtype=torch.int32, device=q.device)
    lib = _lib("attention_tc.cu", {"HD": head_dim})
    _check(lib, lib.dk_attn_prefill_tc(_p(q), _p(out), _p(k_store), _p(v_store), c_longlong(q.shape[0]),
                                       c_longlong(k_store.shape[0]), _p(tiles), tiles.shape[0], _p(cu_q), _p(seq_pos0),
                                       _p(page_table), page_table.shape[1], n_heads, n_kv_heads, int(window or 0),
                                       c_float(scale), _p(_tc_err), _p(sched), c_void_p(stream)), "attention_prefill_tc")

