"""Causal grouped-query attention mixer over the paged key/value cache.

forward = fused q/k/v projection -> per-head q/k norm + rotary + cache write (one kernel; in a
prefill step of head size 64 or 128 the epilogue of the projection itself) ->
attention over the cache -> output projection (reference: engine/engine.py:472-493; the residual
add belongs to the block). The same forward serves whole prompts, continued chunks and single
tokens: the step context says where each token row sits, the cache says what came before.
"""
import torch

from ..cache.requests import KVRequest
from ..config.specs import AttentionSpec
from ..csrc import api
from .base import ParamDecl, Part, build_part, register_part
from .linear import linear


class GQAAttention(Part):
    # forward takes residual= and a deferred norm (see parts.block); measured slower than the separate
    # add+norm kernel on B200 (the small kernel hides behind the next product's weight prefetch), so off
    fuses_residual = False
    # how full the last wave of the tensor-core product's tiles must be for a prefill step's projection
    # to run as that product with norm, rotation and cache write in its epilogue (csrc.api.gemm_tc_qkv)
    qkv_epilogue_min_fill = 0.8

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if rt.dtype == torch.bfloat16 and (s.head_dim % 16 or s.head_dim > 256):
            raise ValueError(f"bfloat16 attention kernels take head sizes in steps of 16 up to 256, not {s.head_dim}")
        if s.head_dim % 2 or s.head_dim > 256:
            raise ValueError(f"attention kernels take even head sizes up to 256, not {s.head_dim}")
        if rt.dtype == torch.bfloat16 and s.hidden_size % 8:
            raise ValueError(f"bfloat16 projections need a hidden size that is a multiple of 8, not {s.hidden_size}")
        self.q_norm = build_part(s.qk_norm, rt) if s.qk_norm is not None else None
        self.k_norm = build_part(s.qk_norm, rt) if s.qk_norm is not None else None
        self.position = build_part(s.position, rt) if s.position is not None else None
        if self.position is not None and not getattr(self.position, "fused_tables", False) and s.qk_norm is not None:
            raise ValueError("a position encoding that rewrites q and k itself (no fused tables) runs before the "
                             "per-head q/k norm; with qk_norm set that is not the order of this mixer")
        self.max_positions = 0
        # decode attention that norms and rotates q and k itself and writes the cache (one launch
        # fewer a layer); measured 1 to 5 percent slower inside the full step on B200: its blocks
        # must wait for the projection's shared memory, which the small kernel between them hides
        self.fuse_decode = False

    def param_decls(self):
        s = self.spec
        d = [ParamDecl("q_proj.weight", (s.num_heads * s.head_dim, s.hidden_size)),
             ParamDecl("k_proj.weight", (s.num_kv_heads * s.head_dim, s.hidden_size)),
             ParamDecl("v_proj.weight", (s.num_kv_heads * s.head_dim, s.hidden_size)),
             ParamDecl("o_proj.weight", (s.hidden_size, s.num_heads * s.head_dim))]
        if self.q_norm is not None:
            d += [ParamDecl("q_norm." + p.name, p.shape, p.init, p.keep_float32) for p in self.q_norm.param_decls()]
            d += [ParamDecl("k_norm." + p.name, p.shape, p.init, p.keep_float32) for p in self.k_norm.param_decls()]
        return d

    def bind(self, tensors):
        # one fused projection [q; k; v] as the reference does (engine/engine.py:300-302)
        self.w_qkv = torch.cat([tensors.pop("q_proj.weight"), tensors.pop("k_proj.weight"),
                                tensors.pop("v_proj.weight")], 0).contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        if self.q_norm is not None:
            self.q_norm.bind({"weight": tensors.pop("q_norm.weight")})
            self.k_norm.bind({"weight": tensors.pop("k_norm.weight")})

    def weights_in_order(self):
        return [self.w_qkv, self.w_o]

    def cache_requests(self):
        s = self.spec
        return [KVRequest(s.num_kv_heads, s.head_dim, s.window, self.rt.dtype)]

    def prepare(self, max_positions):
        self.max_positions = max_positions
        if self.position is not None and getattr(self.position, "fused_tables", False):
            self.position.tables(max_positions)

    def forward(self, ctx, views, a, writes=True, residual=None):
        s, kv = self.spec, views[0]
        dtype, dev = self.rt.dtype, self.rt.device
        nh, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        table = ctx.tables[kv.group]
        fusable = self.position is None or getattr(self.position, "fused_tables", False)
        if dtype == torch.bfloat16 and fusable and self._qkv_in_epilogue(a):
            # prefill: the projection's epilogue norms and rotates q and k and writes the cache
            cos, sin = self.position.tables(max(self.max_positions, ctx.max_position + 1)) if self.position else (None, None)
            q = torch.empty((ctx.n_tok, nh * hd), dtype=dtype, device=dev)
            api.gemm_tc_qkv(a, self.w_qkv, q, self.q_norm.weight if self.q_norm else None,
                            self.k_norm.weight if self.k_norm else None, cos, sin, s.qk_norm.eps if s.qk_norm else 0.0,
                            ctx.row_pos, ctx.row_seq, table, kv.k, kv.v, nh, nkv, hd, write_kv=writes)
            return self._attend(ctx, kv, table, q, residual)
        qkv = linear(a, self.w_qkv, ctx=ctx, allow_partial=True)
        cos = sin = None
        if self.position is not None:
            if fusable:
                cos, sin = self.position.tables(max(self.max_positions, ctx.max_position + 1))
            else:
                if isinstance(qkv, api.Partial):
                    qkv = qkv.sum(dtype)
                self.position.apply(qkv, ctx, nh, nkv, hd)
        qn = self.q_norm.weight if self.q_norm else None
        kn = self.k_norm.weight if self.k_norm else None
        eps = s.qk_norm.eps if s.qk_norm else 0.0
        if dtype == torch.bfloat16 and ctx.is_decode and self.fuse_decode:
            # q/k norm + rotation and the cache write inside the attention kernel
            o = torch.empty((ctx.n_tok, nh * hd), dtype=dtype, device=dev)
            nsplit = api.decode_splits(ctx.n_seq, nkv, nh // nkv)
            ws_acc, ws_ml = ctx.scratch(("attn_decode", ctx.n_seq, nh, hd, nsplit),
                                        lambda: api.attention_decode_ws(ctx.n_seq, nh, hd, nsplit, dev))
            api.attention_decode_fused(qkv, o, qn, kn, cos, sin, eps, kv.k, kv.v, ctx.row_pos, table, nh, nkv, hd,
                                       s.window or 0, s.scale, nsplit, ws_acc, ws_ml, write_kv=writes)
            return linear(o, self.w_o, ctx=ctx, allow_partial=True, residual=residual)
        q = torch.empty((ctx.n_tok, nh * hd), dtype=dtype, device=dev)
        api.qk_norm_rope_write(qkv, q, qn, kn, cos, sin, ctx.row_pos, ctx.row_seq, table, kv.k, kv.v, nh, nkv, hd, eps,
                               write_kv=writes)
        return self._attend(ctx, kv, table, q, residual)

    def _qkv_in_epilogue(self, a):
        """Whether this step's projection runs as the tensor-core product with norm, rotation and
        cache write in its epilogue: a prefill step (more rows than the decode forms take) of a
        size where that product is the one ``linear`` would pick anyway."""
        s = self.spec
        M, K = a.shape
        return (not isinstance(a, api.Normed) and M > api.TC_SKINNY_MAX_ROWS and K % 8 == 0
                and s.head_dim in api.TC_QKV_HEAD_DIMS
                and api.gemm_tc_fills_gpu(M, self.w_qkv.shape[0], self.qkv_epilogue_min_fill))

    def _attend(self, ctx, kv, table, q, residual):
        """Attention of the rotated queries over the cache, then the output projection."""
        s = self.spec
        dtype, dev = self.rt.dtype, self.rt.device
        nh, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        window = s.window or 0
        o = torch.empty((ctx.n_tok, nh * hd), dtype=dtype, device=dev)
        if dtype == torch.float32:
            api.attention_generic(q, o, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, nh, nkv, hd, window, s.scale)
        elif ctx.is_decode:
            nsplit = api.decode_splits(ctx.n_seq, nkv, nh // nkv)
            ws_acc, ws_ml = ctx.scratch(("attn_decode", ctx.n_seq, nh, hd, nsplit),
                                        lambda: api.attention_decode_ws(ctx.n_seq, nh, hd, nsplit, dev))
            api.attention_decode_bf16(q, o, kv.k, kv.v, ctx.row_pos, table, nh, nkv, hd, window, s.scale, nsplit,
                                      ws_acc, ws_ml)
        elif hd in api.TC_ATTENTION_HEAD_DIMS:   # tcgen05: S and P.V in tensor memory, TMA-fed
            api.attention_prefill_tc(q, o, kv.k, kv.v, ctx.tiles_wide, ctx.cu_q, ctx.seq_pos0, table, nh, nkv, hd,
                                     window, s.scale)
        else:
            api.attention_prefill_bf16(q, o, kv.k, kv.v, ctx.tiles, ctx.cu_q, ctx.seq_pos0, table, nh, nkv, hd,
                                       window, s.scale)
        return linear(o, self.w_o, ctx=ctx, allow_partial=True, residual=residual)


register_part(AttentionSpec, GQAAttention)
