"""Grouped-query softmax attention without rotation over the paged cache, with a chunk mask or a
window, a logarithmic distance bias, a sink in the softmax's denominator and an output gate, each
switched on by its specification; key and value heads may differ in size.

forward = one fused projection [q; k; v; gate] -> k and v into the cache -> attention over the cache
with the gate in its epilogue -> output projection. Kernels: bfloat16 prompts with equal head sizes of 64
or 128 on tcgen05 tensor cores, other head sizes in steps of 16 on mma.sync, single tokens by a kernel of
their own, and float32 (or any other size) on the float32-arithmetic kernel that serves every phase. The part also runs as a branch of a
``ParallelMixer``, which does the projections of all its branches in one product each: ``mix`` takes
the projected rows and leaves scale * (gated heads) where the caller wants them.
"""
import torch

from ..cache.requests import KVRequest
from ..config.specs import MaskedAttentionSpec
from ..csrc import api
from .attention import QueryTiles
from .base import ParamDecl, Part, register_part
from .linear import linear


class MaskedAttention(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if max(s.head_dim, s.v_head_dim) > 256:
            raise ValueError(f"attention kernels take head sizes up to 256, not {s.head_dim} / {s.v_head_dim}")
        if s.chunk is not None and s.chunk < 1:
            raise ValueError(f"a chunk of {s.chunk} positions")
        self.n_q, self.n_k = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        self.n_v, self.n_mid = s.num_kv_heads * s.v_head_dim, s.num_heads * s.v_head_dim
        self.n_in = self.n_q + self.n_k + self.n_v + (self.n_mid if s.output_gate else 0)
        self.r1 = self.r2 = self.sink = None
        # the tensor-core kernels take bfloat16 with head sizes in steps of 16; everything else (float32, odd
        # head sizes) runs on the float32-arithmetic kernel, which serves every phase
        self.tensor_core = rt.dtype == torch.bfloat16 and api.masked_bf16_takes(s.head_dim, s.v_head_dim)
        self.tiles = QueryTiles(api.MASKED_TILE_ROWS) if self.tensor_core else None
        # equal head sizes of 64 or 128: prompts run on the tcgen05 kernel (its masked build), in tiles of 128 queries
        self.tc_tiles = QueryTiles(api.TC_TILE_ROWS) if self.tensor_core and s.head_dim == s.v_head_dim \
            and s.head_dim in api.TC_ATTENTION_HEAD_DIMS else None

    def step_plans(self):
        return [t for t in (self.tiles, self.tc_tiles) if t is not None]

    def param_decls(self):
        s = self.spec
        d = [ParamDecl("q", (self.n_q, s.hidden_size)), ParamDecl("k", (self.n_k, s.hidden_size)),
             ParamDecl("v", (self.n_v, s.hidden_size)), ParamDecl("o", (s.hidden_size, self.n_mid))]
        if s.output_gate:
            d.append(ParamDecl("g", (self.n_mid, s.hidden_size)))
        if s.distance_bias:
            d += [ParamDecl("r1", (s.num_heads,), init="positive", keep_float32=True),
                  ParamDecl("r2", (s.num_heads,), init="positive", keep_float32=True)]
        if s.sink:
            d.append(ParamDecl("sink", (s.num_heads,), init="unit", keep_float32=True))
        return d

    def bind(self, tensors):
        rows = [tensors.pop("q"), tensors.pop("k"), tensors.pop("v")]
        if self.spec.output_gate:
            rows.append(tensors.pop("g"))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_o = tensors.pop("o").contiguous()
        if self.spec.distance_bias:
            self.r1 = tensors.pop("r1").to(torch.float32).contiguous()
            self.r2 = tensors.pop("r2").to(torch.float32).contiguous()
        if self.spec.sink:
            self.sink = tensors.pop("sink").to(torch.float32).contiguous()

    def step_weights(self):
        return [self.w_in, self.w_o]

    def cache_requests(self):
        s = self.spec
        return [KVRequest(s.num_kv_heads, s.head_dim, s.window, self.rt.dtype, s.v_head_dim, s.chunk)]

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        """``proj`` [tokens, n_in]: this part's rows of a projection (possibly columns of a wider matrix);
        ``mid`` [tokens, n_mid]: where scale * (gated heads) go."""
        s, kv = self.spec, views[0]
        table = ctx.tables[kv.group]
        q = proj[:, :self.n_q]
        k = proj[:, self.n_q:self.n_q + self.n_k]
        v = proj[:, self.n_q + self.n_k:self.n_q + self.n_k + self.n_v]
        gate = proj[:, self.n_q + self.n_k + self.n_v:] if s.output_gate else None
        sizes = (s.num_heads, s.num_kv_heads, s.head_dim, s.v_head_dim, s.window, s.chunk, s.scale)
        if self.tensor_core and ctx.is_decode and api.masked_decode_streams(q, mid, gate, s.head_dim, s.v_head_dim):
            # single tokens, keys and values of one size: the library's split decode kernel in its masked build
            if writes:
                api.kv_write(k, v, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, s.num_kv_heads, s.head_dim, s.v_head_dim)
            nsplit = api.masked_decode_splits(ctx.n_seq, s.num_kv_heads, s.num_heads // s.num_kv_heads, table.shape[1],
                                              s.window, s.chunk)
            ws_acc, ws_ml = ctx.scratch(("attn_decode", ctx.n_seq, s.num_heads, s.head_dim, nsplit),
                                        lambda: api.attention_decode_ws(ctx.n_seq, s.num_heads, s.head_dim, nsplit, self.rt.device))
            return api.attention_decode_masked_bf16(q, mid, gate, scale, kv.k, kv.v, ctx.row_pos, table, s.num_heads,
                                                    s.num_kv_heads, s.head_dim, s.window, s.chunk, s.scale, nsplit, ws_acc,
                                                    ws_ml, self.r1, self.r2, self.sink)
        span = api.masked_decode_span(s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.chunk, table.shape[1], ctx.n_tok) \
            if self.tensor_core and ctx.is_decode and all(t is None or t.stride(0) % 2 == 0 for t in (q, mid, gate)) else None
        if span is not None:      # single tokens: the kernel stores each token's key and value itself
            ws = None
            if span[1] > 1:
                ws = ctx.scratch(("masked_decode", ctx.n_tok, s.num_heads, s.v_head_dim, span[1]),
                                 lambda: api.masked_decode_ws(ctx.n_tok, s.num_heads, s.v_head_dim, span[1], self.rt.device))
            return api.attention_masked_decode_bf16(q, mid, gate, scale, kv.k, kv.v, ctx.row_pos, table, *sizes, span,
                                                    self.r1, self.r2, self.sink, k if writes else None, v if writes else None, ws)
        if writes:
            api.kv_write(k, v, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, s.num_kv_heads, s.head_dim, s.v_head_dim)
        if self.tc_tiles is not None and not ctx.is_decode and api.masked_tc_takes(q, mid, gate, s.head_dim, s.v_head_dim):
            return api.attention_masked_prefill_tc(q, mid, gate, scale, kv.k, kv.v, ctx.plans[self.tc_tiles.key], ctx.cu_q,
                                                   ctx.seq_pos0, table, s.num_heads, s.num_kv_heads, s.head_dim, s.window,
                                                   s.chunk, s.scale, self.r1, self.r2, self.sink)
        even = all(t is None or (t.stride(0) % 2 == 0 and t.data_ptr() % 4 == 0) for t in (q, mid, gate))
        if self.tensor_core and not ctx.is_decode and even:
            return api.attention_masked_prefill_bf16(q, mid, gate, scale, kv.k, kv.v, ctx.plans[self.tiles.key], ctx.cu_q,
                                                     ctx.seq_pos0, table, *sizes, self.r1, self.r2, self.sink)
        api.attention_masked(q, mid, gate, scale, kv.k, kv.v, ctx.row_pos, ctx.row_seq, table, *sizes, self.r1, self.r2,
                             self.sink)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(MaskedAttentionSpec, MaskedAttention)
