"""Several mixers side by side on the same input: out = sum_i scale_i * mixer_i(x).

The branches' input projections are one product (their weights stacked by rows), and so are their
output projections (their weights side by side along the inner dimension, each branch's activations
already multiplied by its scale): sum_i scale_i * W_i m_i = [W_1 | W_2 | ..] [scale_1 m_1; scale_2 m_2; ..].
A branch is any mixer part that offers ``w_in`` [n_in, hidden], ``w_o`` [hidden, n_mid] and
``mix(ctx, views, proj, mid, scale, writes)``; the cache views are dealt out in the order of the
branches' requests.
"""
import torch

from ..config.specs import ParallelMixerSpec
from .base import ParamDecl, Part, build_part, register_part
from .linear import linear


class ParallelMixer(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.branches = [(pre, build_part(sub, rt), float(scale)) for pre, sub, scale in spec.branches]
        for _, b, _ in self.branches:
            if not hasattr(b, "mix"):
                raise TypeError(f"{type(b).__name__} cannot be a branch of a parallel mixer: it has no mix()")
        self.n_in = sum(b.n_in for _, b, _ in self.branches)
        self.n_mid = sum(b.n_mid for _, b, _ in self.branches)

    def param_decls(self):
        return [ParamDecl(pre + p.name, p.shape, p.init, p.keep_float32) for pre, b, _ in self.branches
                for p in b.param_decls()]

    def bind(self, tensors):
        for pre, b, _ in self.branches:
            b.bind({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})
        self.w_in = torch.cat([b.w_in for _, b, _ in self.branches], 0).contiguous()
        self.w_o = torch.cat([b.w_o for _, b, _ in self.branches], 1).contiguous()
        r = c = 0
        for _, b, _ in self.branches:      # the branches keep views of the stacked weights, not copies
            b.w_in, b.w_o = self.w_in[r:r + b.n_in], self.w_o[:, c:c + b.n_mid]
            r, c = r + b.n_in, c + b.n_mid

    def step_weights(self):
        return [self.w_in, self.w_o]

    def step_plans(self):
        return [p for _, b, _ in self.branches for p in b.step_plans()]

    def cache_requests(self):
        return [r for _, b, _ in self.branches for r in b.cache_requests()]

    def prepare(self, max_positions):
        for _, b, _ in self.branches:
            b.prepare(max_positions)

    def forward(self, ctx, views, a, writes=True):
        proj = linear(a, self.w_in)
        mid = torch.empty((ctx.n_tok, self.n_mid), dtype=self.rt.dtype, device=self.rt.device)
        r = c = v = 0
        for _, b, scale in self.branches:
            nv = len(b.cache_requests())
            b.mix(ctx, views[v:v + nv], proj[:, r:r + b.n_in], mid[:, c:c + b.n_mid], scale, writes)
            r, c, v = r + b.n_in, c + b.n_mid, v + nv
        return linear(mid, self.w_o, allow_partial=True)


register_part(ParallelMixerSpec, ParallelMixer)
