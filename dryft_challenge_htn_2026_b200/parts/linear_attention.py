"""Linear attention with a constant decay per head over a per-sequence state.

forward = one fused projection [q; k; v; gate] -> the recurrence S <- d S + k v^T, o = S^T q with
q, k, v = silu(projection) and the state in float32 in the cache's state storage -> all heads together
through a weighted RMS norm, times sigmoid(gate) -> output projection. Like the attention parts it also
runs as a branch of a ``ParallelMixer`` (``mix``).
"""
import torch

from ..cache.requests import StateRequest
from ..config.specs import LinearAttentionSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part
from .linear import linear


class LinearAttention(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if len(s.decay) != s.num_heads:
            raise ValueError(f"{len(s.decay)} decays for {s.num_heads} heads")
        if max(s.head_dim, s.v_head_dim) > 256:
            raise ValueError(f"linear attention takes head sizes up to 256, not {s.head_dim} / {s.v_head_dim}")
        self.n_qk, self.n_mid = s.num_heads * s.head_dim, s.num_heads * s.v_head_dim
        self.n_in = 2 * self.n_qk + self.n_mid + (self.n_mid if s.output_gate else 0)
        self.decay = torch.tensor(s.decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.norm_weight = None

    def param_decls(self):
        s = self.spec
        d = [ParamDecl("q", (self.n_qk, s.hidden_size)), ParamDecl("k", (self.n_qk, s.hidden_size)),
             ParamDecl("v", (self.n_mid, s.hidden_size)), ParamDecl("o", (s.hidden_size, self.n_mid))]
        if s.output_gate:
            d.append(ParamDecl("g", (self.n_mid, s.hidden_size)))
        if s.out_norm is not None:
            d.append(ParamDecl("norm", (self.n_mid,), init="norm", keep_float32=True))
        return d

    def bind(self, tensors):
        rows = [tensors.pop("q"), tensors.pop("k"), tensors.pop("v")]
        if self.spec.output_gate:
            rows.append(tensors.pop("g"))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_o = tensors.pop("o").contiguous()
        if self.spec.out_norm is not None:
            self.norm_weight = tensors.pop("norm").to(torch.float32).contiguous()
        else:
            self.norm_weight = None

    def step_weights(self):
        return [self.w_in, self.w_o]

    def cache_requests(self):
        s = self.spec
        return [StateRequest((s.num_heads, s.head_dim, s.v_head_dim), torch.float32)]

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        s, state = self.spec, views[0].state
        if not writes:
            raise ValueError("a linear-attention layer cannot read another layer's state: it has no keys to read")
        q = proj[:, :self.n_qk]
        k = proj[:, self.n_qk:2 * self.n_qk]
        v = proj[:, 2 * self.n_qk:2 * self.n_qk + self.n_mid]
        gate = proj[:, 2 * self.n_qk + self.n_mid:] if s.output_gate else None
        o = torch.empty((ctx.n_tok, self.n_mid), dtype=torch.float32, device=self.rt.device)
        if ctx.is_decode:      # one token a row; padding rows carry position -1
            api.linear_attention(q, k, v, o, state, None, ctx.row_pos, ctx.seq_slot, self.decay, ctx.n_tok,
                                 s.num_heads, s.head_dim, s.v_head_dim, 1)
        else:
            api.linear_attention(q, k, v, o, state, ctx.cu_q, ctx.seq_pos0, ctx.seq_slot, self.decay, ctx.n_seq,
                                 s.num_heads, s.head_dim, s.v_head_dim, int(ctx.host["lens"].max()))
        if self.norm_weight is None:
            raise ValueError("linear attention without an output norm is not implemented")
        api.norm_gate(o, self.norm_weight, s.out_norm.eps, gate, scale, mid)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(LinearAttentionSpec, LinearAttention)
