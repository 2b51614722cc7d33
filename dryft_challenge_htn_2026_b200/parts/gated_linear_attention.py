"""Gated linear attention: linear attention whose state decays per key channel and token.

forward = one fused projection [q; k; v; gate; a1] -> the decay's second step z = W_a2 (a1 rows) in float32
-> the recurrence S <- diag(alpha) S + k v^T, o = S^T q with alpha = sigmoid(z + b)^(1/tau), state and decay in
float32 (the state lives in the cache's state storage; a warp per 8 value columns keeps its part of the state in
registers for key sizes of 32, 64, 128 and 256, a block form serves the others) -> per head an RMS norm over the value size, times
silu(gate) -> output projection. Like the other mixers it can be a branch of a ``ParallelMixer`` (``mix``).
"""
import torch

from ..cache.requests import StateRequest
from ..config.specs import GatedLinearAttentionSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part
from .linear import STORE_F32, linear


class GatedLinearAttention(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if max(s.head_dim, s.v_head_dim) > 256:
            raise ValueError(f"gated linear attention takes head sizes up to 256, not {s.head_dim} / {s.v_head_dim}")
        if not s.tau > 0 or s.decay_rank < 1:
            raise ValueError(f"tau {s.tau} / decay rank {s.decay_rank}")
        self.n_qk, self.n_mid = s.num_heads * s.head_dim, s.num_heads * s.v_head_dim
        # the rows of the fused projection: q, k, v, gate, then the decay's first step
        self.n_main = 2 * self.n_qk + 2 * self.n_mid
        self.n_in = self.n_main + s.decay_rank
        self.q_scale = float(s.head_dim) ** -0.5

    def param_decls(self):
        s = self.spec
        return [ParamDecl("q", (self.n_qk, s.hidden_size)), ParamDecl("k", (self.n_qk, s.hidden_size)),
                ParamDecl("v", (self.n_mid, s.hidden_size)), ParamDecl("g", (self.n_mid, s.hidden_size)),
                ParamDecl("o", (s.hidden_size, self.n_mid)), ParamDecl("norm", (s.v_head_dim,), init="norm", keep_float32=True),
                ParamDecl("a1", (s.decay_rank, s.hidden_size)), ParamDecl("a2", (self.n_qk, s.decay_rank), init="wide"),
                ParamDecl("a2.b", (self.n_qk,), init="unit", keep_float32=True)]

    def bind(self, tensors):
        self.w_in = torch.cat([tensors.pop("q"), tensors.pop("k"), tensors.pop("v"), tensors.pop("g"), tensors.pop("a1")],
                              0).contiguous()
        self.w_o = tensors.pop("o").contiguous()
        self.w_a2 = tensors.pop("a2").contiguous()
        self.z_bias = tensors.pop("a2.b").to(torch.float32).contiguous()
        self.norm_weight = tensors.pop("norm").to(torch.float32).contiguous()

    def step_weights(self):
        return [self.w_in, self.w_a2, self.w_o]

    def cache_requests(self):
        s = self.spec
        return [StateRequest((s.num_heads, s.head_dim, s.v_head_dim), torch.float32)]

    def mix(self, ctx, views, proj, mid, scale, writes=True):
        s, state = self.spec, views[0].state
        if not writes:
            raise ValueError("a gated-linear-attention layer cannot read another layer's state: it has no keys to read")
        q = proj[:, :self.n_qk]
        k = proj[:, self.n_qk:2 * self.n_qk]
        v = proj[:, 2 * self.n_qk:2 * self.n_qk + self.n_mid]
        gate = proj[:, 2 * self.n_qk + self.n_mid:self.n_main]
        a1 = proj[:, self.n_main:self.n_in].contiguous()
        z = linear(a1, self.w_a2, STORE_F32)                      # float32 rows: they enter the recurrence
        o = torch.empty((ctx.n_tok, self.n_mid), dtype=torch.float32, device=self.rt.device)
        if ctx.is_decode:      # one token a row; padding rows carry position -1
            api.gated_linear_attention(q, k, v, o, state, None, ctx.row_pos, ctx.seq_slot, z, self.z_bias, s.tau,
                                       self.q_scale, ctx.n_tok, s.num_heads, s.head_dim, s.v_head_dim)
        else:
            api.gated_linear_attention(q, k, v, o, state, ctx.cu_q, ctx.seq_pos0, ctx.seq_slot, z, self.z_bias, s.tau,
                                       self.q_scale, ctx.n_seq, s.num_heads, s.head_dim, s.v_head_dim)
        api.norm_gate(o, self.norm_weight, s.norm_eps, gate, scale, mid, group=s.v_head_dim, gate_act="silu")

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        self.mix(ctx, views, proj, mid, 1.0, writes)
        return linear(mid, self.w_o, allow_partial=True)


register_part(GatedLinearAttentionSpec, GatedLinearAttention)
