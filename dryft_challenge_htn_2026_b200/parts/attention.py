"""Causal grouped-query attention mixer over the paged key/value cache.

forward = fused q/k/v projection -> per-head q/k norm + rotary + cache write (one kernel; in a
prefill step of head size 64 or 128 the epilogue of the projection itself) ->
attention over the cache -> output projection (reference: engine/engine.py:472-493; the residual
add belongs to the block). The same forward serves whole prompts, continued chunks and single
tokens: the step context says where each token row sits, the cache says what came before.
"""
import numpy as np
import torch

from ..cache.requests import KVRequest
from ..config.specs import AttentionSpec
from ..csrc import api
from .base import ParamDecl, Part, StepPlan, build_part, register_part
from .linear import linear


class QueryTiles(StepPlan):
    """Work list of a prefill attention kernel whose blocks take ``rows`` consecutive queries of one
    sequence: (sequence, first query within this step's chunk) per tile, the tile that sees the
    most keys first. Empty for a decode step."""

    def __init__(self, rows):
        self.rows = rows
        self.key = ("query_tiles", rows)

    def build(self, lens, pos0, is_decode):
        if is_decode:
            return np.zeros((0, 2), np.int32)
        tiles = [(int(pos0[i]) + min(q0 + self.rows, int(lens[i])), i, q0)
                 for i in range(len(lens)) for q0 in range(0, int(lens[i]), self.rows)]
        tiles.sort(key=lambda t: -t[0])
        return np.array([(t[1], t[2]) for t in tiles], dtype=np.int32).reshape(-1, 2)


class GQAAttention(Part):
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
        # tables the fused kernels rotate with, or a position encoding that rewrites q and k itself
        self.fused_position = self.position is None or getattr(self.position, "fused_tables", False)
        self.max_positions = 0
        # the prefill kernel this mixer's steps use, and so the tiles they need planned
        self.tc_prefill = rt.dtype == torch.bfloat16 and s.head_dim in api.TC_ATTENTION_HEAD_DIMS
        self.tiles = QueryTiles(api.TC_TILE_ROWS if self.tc_prefill else api.MMA_TILE_ROWS) \
            if rt.dtype == torch.bfloat16 else None

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

    def step_weights(self):
        return [self.w_qkv, self.w_o]

    def step_plans(self):
        return [self.tiles] if self.tiles is not None else []

    def cache_requests(self):
        s = self.spec
        return [KVRequest(s.num_kv_heads, s.head_dim, s.window, self.rt.dtype)]

    def prepare(self, max_positions):
        self.max_positions = max_positions
        if self.position is not None and self.fused_position:
            self.position.tables(max_positions)

    def forward(self, ctx, views, a, writes=True):
        s, kv = self.spec, views[0]
        dtype, dev = self.rt.dtype, self.rt.device
        nh, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        table = ctx.tables[kv.group]
        qn = self.q_norm.weight if self.q_norm else None
        kn = self.k_norm.weight if self.k_norm else None
        eps = s.qk_norm.eps if s.qk_norm else 0.0
        cos = sin = None
        if self.position is not None and self.fused_position:
            cos, sin = self.position.tables(max(self.max_positions, ctx.max_position + 1))
        q = torch.empty((ctx.n_tok, nh * hd), dtype=dtype, device=dev)
        if dtype == torch.bfloat16 and self.fused_position and self._qkv_in_epilogue(a):
            # prefill: the projection's epilogue norms and rotates q and k and writes the cache
            api.gemm_tc_qkv(a, self.w_qkv, q, qn, kn, cos, sin, eps, ctx.row_pos, ctx.row_seq, table, kv.k, kv.v,
                            nh, nkv, hd, write_kv=writes)
            return self._attend(ctx, kv, table, q)
        qkv = linear(a, self.w_qkv, allow_partial=True)
        if not self.fused_position:
            # the position encoding rewrites q and k itself: after the per-head norm, before the cache write
            if qn is not None or isinstance(qkv, api.Partial):
                normed = torch.empty((ctx.n_tok, (nh + 2 * nkv) * hd), dtype=dtype, device=dev)
                api.qk_norm_rope_write(qkv, None, qn, kn, None, None, ctx.row_pos, ctx.row_seq, table, kv.k, kv.v,
                                       nh, nkv, hd, eps, dense_out=normed)
                qkv, qn, kn = normed, None, None
            self.position.apply(qkv, ctx, nh, nkv, hd)
        api.qk_norm_rope_write(qkv, q, qn, kn, cos, sin, ctx.row_pos, ctx.row_seq, table, kv.k, kv.v, nh, nkv, hd, eps,
                               write_kv=writes)
        return self._attend(ctx, kv, table, q)

    def _qkv_in_epilogue(self, a):
        """Whether this step's projection runs as the tensor-core product with norm, rotation and
        cache write in its epilogue: a prefill step (more rows than the decode forms take) of a
        size where that product is the one ``linear`` would pick anyway."""
        s = self.spec
        M, K = a.shape
        return (M > api.TC_SKINNY_MAX_ROWS and K % 8 == 0 and s.head_dim in api.TC_QKV_HEAD_DIMS
                and api.gemm_tc_fills_gpu(M, self.w_qkv.shape[0], self.qkv_epilogue_min_fill))

    def _attend(self, ctx, kv, table, q):
        """Attention of the rotated queries over the cache, then the output projection."""
        s = self.spec
        dtype, dev = self.rt.dtype, self.rt.device
        nh, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        window = s.window or 0
        o = torch.empty((ctx.n_tok, nh * hd), dtype=dtype, device=dev)
        if dtype == torch.float32:
            api.attention_generic(q, o, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, nh, nkv, hd, window, s.scale)
        elif ctx.is_decode:
            nsplit = api.decode_splits(ctx.n_seq, nkv, nh // nkv, table.shape[1])
            ws_acc, ws_ml = ctx.scratch(("attn_decode", ctx.n_seq, nh, hd, nsplit),
                                        lambda: api.attention_decode_ws(ctx.n_seq, nh, hd, nsplit, dev))
            api.attention_decode_bf16(q, o, kv.k, kv.v, ctx.row_pos, table, nh, nkv, hd, window, s.scale, nsplit,
                                      ws_acc, ws_ml)
        elif self.tc_prefill:                    # tcgen05: S and P.V in tensor memory, TMA-fed
            api.attention_prefill_tc(q, o, kv.k, kv.v, ctx.plans[self.tiles.key], ctx.cu_q, ctx.seq_pos0, table, nh, nkv,
                                     hd, window, s.scale)
        else:
            api.attention_prefill_bf16(q, o, kv.k, kv.v, ctx.plans[self.tiles.key], ctx.cu_q, ctx.seq_pos0, table, nh, nkv,
                                       hd, window, s.scale)
        return linear(o, self.w_o, allow_partial=True)


register_part(AttentionSpec, GQAAttention)
