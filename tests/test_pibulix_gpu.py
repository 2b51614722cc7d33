"""The Pibulix decoder in the library against the plain implementation (``plain_pibulix``): every mechanism
alone, then whole models of several small shapes through the step function, the cache, the decode state and the
entry points. The shapes differ in every size and option: key/value groups of 1 to 3, key and value heads of
different sizes, convolutions of 1 to 4 taps, rotations over the whole head, a part of it and none, windows
smaller and larger than a page and none, more kept first tokens than the window is wide, experts in 1 to 4
groups, with and without a shared expert, a layer without feed-forward, layers that run on another layer's
weights, head sizes the tensor-core kernels take and ones they do not."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_pibulix as plain
from dryft_challenge_htn_2026_b200.cache import Cache
from dryft_challenge_htn_2026_b200.config.specs import (GatedLinearAttentionSpec, GatedMLPSpec, MaskedAttentionSpec,
                                                        OnePlusRMSNormSpec, RMSNormSpec, RotaryPartSpec, RoutedMLPSpec)
from dryft_challenge_htn_2026_b200.csrc import api
from dryft_challenge_htn_2026_b200.engine import DecodeLoop, Runner, load_model
from dryft_challenge_htn_2026_b200.engine.batch import build_context
from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
from helpers import ROOT, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def attn(heads, kv, dim, vdim, conv, scale, softcap, rot, mask, mlp, **more):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "softcap": softcap}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return dict({"type": "attention", "mixer": m, "mlp": mlp}, **more)


def gla(heads, dim, vdim, tau, mlp, **more):
    return dict({"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}, **more)


def moe(experts, ff, top, groups, keep, scale, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale,
                                                        "groups": {"count": groups, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


_A0 = attn(4, 2, 32, 16, 4, 0.2, 30.0, (32, 10000.0), (24, 3), {"kind": "dense", "ff": 96})
_A1 = gla(2, 16, 24, 4.0, moe(8, 40, 2, 4, 2, 1.5, 48))
SHAPES = {
    # groups of 2, value heads smaller than key heads, 4 taps, a rotation over the whole head, a window smaller than a
    # page with 3 kept tokens, two layers that run on other layers' weights, a last layer without feed-forward
    "A": dict(architecture="Pibulix", vocab=200, width=64, norm={"eps": 1e-5}, postln_alpha=2.0, decay_rank=[None, 4, None, 4, 12],
              layers=[_A0, _A1, dict(_A0, weights_of=0), dict(_A1, weights_of=1), gla(1, 32, 8, 1.0, None)]),
    # a gla layer first, as many key/value heads as query heads, 2 taps, no cap, a rotation over a quarter of the head,
    # a window of exactly one page without kept tokens, experts in one group without a shared expert; then a layer
    # without convolution and without rotation whose 9 kept tokens outnumber its window of 7, one expert of 4 chosen
    "B": dict(architecture="Pibulix", vocab=264, width=96, norm={"eps": 3e-6}, postln_alpha=1.0, decay_rank=[8, None, None],
              layers=[gla(3, 16, 32, 8.0, {"kind": "dense", "ff": 128}),
                      attn(3, 3, 32, 48, 2, 0.3, 0.0, (8, 500.0), (64, 0), moe(6, 24, 3, 1, 1, 1.0, None)),
                      attn(6, 2, 16, 16, 1, 0.25, 12.0, None, (7, 9), moe(4, 32, 1, 2, 1, 2.0, 16))]),
    # head sizes 64 and 128 (what the tensor-core kernels are built for), a window that spans pages, no mask at all
    "C": dict(architecture="Pibulix", vocab=320, width=128, norm={"eps": 1e-6}, postln_alpha=3.0, decay_rank=[None, 16, None],
              layers=[attn(2, 1, 64, 64, 3, 0.125, 20.0, (32, 250000.0), (100, 5), {"kind": "dense", "ff": 192}),
                      gla(2, 64, 64, 16.0, moe(8, 64, 2, 2, 2, 2.5, 64)),
                      attn(2, 2, 128, 128, 3, 0.09, 50.0, (128, 10000.0), None, {"kind": "dense", "ff": 160})]),
    # sizes that no tensor-core kernel takes: heads of 20 / 10 / 24 / 12, an expert size of 20, a dense feed-forward of
    # 52 (no multiple of 8), a decay rank of 5
    "D": dict(architecture="Pibulix", vocab=136, width=48, norm={"eps": 1e-5}, postln_alpha=1.5, decay_rank=[None, 5],
              layers=[attn(3, 1, 20, 10, 3, 0.22, 8.0, (10, 100.0), (33, 2), moe(3, 20, 2, 3, 2, 1.0, 20)),
                      gla(1, 24, 12, 2.0, {"kind": "dense", "ff": 52})]),
}


def make_model(tmp_path, name, seed=0):
    cfg = dk.config_from_dict(SHAPES[name])
    folder = str(tmp_path / f"pibulix{name}_{seed}")
    dk.write_random_model(cfg, folder, seed=seed, dtype=torch.float32, matrix_std=0.08)
    return folder, cfg


def tol(dtype, ref):
    return (2e-4 if dtype in (torch.float32, "float32") else 6e-2) * max(1.0, float(ref.abs().max()))


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def close(got, ref, dtype, what="", slack=0.5):
    err = float((got.double().cpu() - ref.double()).abs().max())
    assert err <= tol(dtype, ref) * slack, f"{what}: max error {err} > {tol(dtype, ref) * slack}"


def dev(x, dtype):
    return x.to(dtype).to(DEV)


# ------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(5, 48), (70, 256), (3, 1000)])
def test_norm_after_the_sum_with_a_weight_around_zero(dtype, rows, width):
    x, d, w = rnd(rows, width, seed=1, scale=2.0), rnd(rows, width, seed=2).to(dtype).double(), rnd(width, seed=3, scale=0.2)
    ref = plain.norm_one_plus(1.7 * x.float().double() + d, w.float().double(), 1e-5)
    norm = build_part(OnePlusRMSNormSpec(width, 1e-5), Runtime(DEV, dtype))
    norm.bind({"": w.float().to(DEV)})
    h = x.float().to(DEV)
    a = norm.scale_add_forward(h, 1.7, dev(d, dtype), torch.empty(rows, width, dtype=dtype, device=DEV))
    close(h, ref, torch.float32, "stream")
    close(a, ref, dtype, "copy")
    # the same norm as a final norm: gathered rows, the stream untouched
    rows_idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out = norm.add_forward(h, None, torch.empty(2, width, dtype=dtype, device=DEV), rows_idx)
    close(out, plain.norm_one_plus(ref.float().double(), w.float().double(), 1e-5)[[rows - 1, 0]], dtype, "final")


def prep_part(dtype, H, G, D, V, taps, rot, qk_norm=True, seed=0, **opts):
    spec = MaskedAttentionSpec(hidden_size=8, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=D ** -0.5,
                               unit_sink=True, conv_taps=taps if taps > 1 else None,
                               qk_norm=RMSNormSpec(D, 1e-5) if qk_norm else None,
                               position=RotaryPartSpec(rot[0], rot[1]) if rot else None, **opts)
    part = build_part(spec, Runtime(DEV, dtype))
    C = (H + G) * D + G * V
    p = {"q.conv": rnd(H * D, taps, seed=seed + 10, scale=0.6), "k.conv": rnd(G * D, taps, seed=seed + 11, scale=0.6),
         "v.conv": rnd(G * V, taps, seed=seed + 12, scale=0.6), "q.norm": 1 + rnd(D, seed=seed + 13, scale=0.2),
         "k.norm": 1 + rnd(D, seed=seed + 14, scale=0.2)}
    p = {k: v.to(dtype).double() for k, v in p.items()}
    if taps > 1:
        part.w_conv = dev(torch.cat([p["q.conv"], p["k.conv"], p["v.conv"]], 0), dtype).contiguous()
    if qk_norm:
        part.q_norm_w, part.k_norm_w = dev(p["q.norm"], torch.float32), dev(p["k.norm"], torch.float32)
    return part, p, C


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,taps,rot", [(4, 2, 32, 16, 4, (32, 10000.0)), (3, 3, 16, 48, 2, (8, 500.0)),
                                              (2, 1, 64, 64, 3, (32, 250000.0)), (3, 1, 20, 10, 3, (10, 100.0)),
                                              (2, 2, 16, 16, 1, None), (1, 1, 256, 8, 9, (256, 1e6))])
def test_convolution_head_norm_and_rotation_in_prompts_portions_and_single_tokens(dtype, H, G, D, V, taps, rot):
    """The projection rows of one sequence are cut into steps down to one and two tokens (the convolution's state
    carries over), with a second sequence beside it; positions run past 300, where a wrong angle shows."""
    part, p, C = prep_part(dtype, H, G, D, V, taps, rot)
    lens = [70, 2, 1, 1, 3, 130, 1, 2, 100]
    T = sum(lens)
    u = rnd(T, C, seed=5).to(dtype).double()
    q, k, v = u[:, :H * D], u[:, H * D:(H + G) * D], u[:, (H + G) * D:]
    if taps > 1:
        q, k, v = plain.short_conv(q, p["q.conv"]), plain.short_conv(k, p["k.conv"]), plain.short_conv(v, p["v.conv"])
    q = plain.rms(q.view(T, H, D), 1e-5) * p["q.norm"]
    k = plain.rms(k.view(T, G, D), 1e-5) * p["k.norm"]
    if rot:
        q, k = plain.rotate_partial(q, torch.arange(T), *rot), plain.rotate_partial(k, torch.arange(T), *rot)
    ref = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v], 1)
    cache = Cache([part.cache_requests()], 64 * 12, 4, DEV)
    other, slot = cache.begin(), cache.begin()
    part.prepare(T + 8)
    t0 = 0
    for n in lens:
        m = 1 if n == 1 else 2
        ctx = build_context(cache, [(other, [0] * m, []), (slot, [0] * n, [])], DEV, plans=part.step_plans())
        wide = torch.zeros(m + n, C + 8, dtype=dtype, device=DEV)
        wide[m:, :C] = dev(u[t0:t0 + n], dtype)
        out = part.prepared_rows(ctx, cache.views(0), wide[:, :C])
        close(out[m:], ref[t0:t0 + n], dtype, f"rows {t0}..{t0 + n}", slack=0.25)
        cache.commit(other, m), cache.commit(slot, n)
        t0 += n


def attention_case(dtype, H, G, D, V, size, keep, cap, lens_steps, plant=None, seed=0):
    """The part's ``mix`` without anything between projection and cache (cache write and whichever attention kernel
    the part picks) over one sequence cut into steps, a second sequence beside it, against the plain attention over
    the whole sequence. ``plant`` = (query position, key position, strength): that key is given the query's direction,
    so that its score stands out, and a value of 5."""
    T = sum(lens_steps)
    q, k, v = rnd(T, H, D, seed=seed), rnd(T, G, D, seed=seed + 1), rnd(T, G, V, seed=seed + 2)
    if plant:
        qi, kj, strength = plant
        k[kj] = strength * q[qi, 0] / q[qi, 0].norm()
        v[kj] = 5.0
    q, k, v = (x.to(dtype).double() for x in (q, k, v))
    scale = D ** -0.5
    ref = plain.attention_core(q, k, v, scale, size, keep, cap).reshape(T, H * V)
    spec = MaskedAttentionSpec(hidden_size=8, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=V, scale=scale, window=size,
                               keep_first=keep, softcap=cap, unit_sink=True)
    part = build_part(spec, Runtime(DEV, dtype))
    cache = Cache([part.cache_requests()], 64 * 40, 4, DEV)
    other, slot = cache.begin(), cache.begin()
    t0 = 0
    got = []
    for n in lens_steps:
        m = 1 if n == 1 else 3
        ctx = build_context(cache, [(other, [0] * m, []), (slot, [0] * n, [])], DEV, plans=part.step_plans())
        wide = torch.zeros(m + n, part.n_in + 8, dtype=dtype, device=DEV)
        wide[m:, :part.n_in] = dev(torch.cat([q[t0:t0 + n].reshape(n, -1), k[t0:t0 + n].reshape(n, -1),
                                              v[t0:t0 + n].reshape(n, -1)], 1), dtype)
        out = torch.empty(m + n, H * V + 8, dtype=dtype, device=DEV)
        part.mix(ctx, cache.views(0), wide[:, :part.n_in], out[:, :H * V], 1.0)
        got.append(out[m:, :H * V].double().cpu())
        cache.commit(other, m), cache.commit(slot, n)
        t0 += n
    return torch.cat(got, 0), ref, cache, slot


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,size,keep,cap", [(4, 2, 32, 16, 24, 3, 30.0), (3, 3, 16, 48, 64, 0, None), (2, 1, 64, 64, 100, 5, 20.0),
                                                   (6, 2, 16, 16, 7, 9, 4.0), (2, 2, 128, 128, None, 0, 50.0), (3, 1, 20, 10, 33, 2, 8.0),
                                                   (8, 1, 128, 128, 70, 70, 2.0)])
def test_attention_scores_window_kept_tokens_and_sink(dtype, H, G, D, V, size, keep, cap):
    got, ref, _, _ = attention_case(dtype, H, G, D, V, size, keep, cap, [131, 2, 1, 1, 40, 1, 1, 1, 90])
    close(got, ref, dtype, "attention")


@pytest.mark.parametrize("dtype,D", [(torch.float32, 32), (torch.bfloat16, 32), (torch.bfloat16, 64)])
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("edge", ["last inside the window", "first outside the window", "last kept token", "first token not kept",
                                  "far key among hundreds", "page border"])
def test_a_planted_key_shows_inside_and_is_hidden_outside(dtype, D, where, edge):
    """Head size 32 runs on the float32-arithmetic kernel, 64 in bfloat16 on the tensor-core kernels."""
    size, keep, qi = 70, 4, 300
    kj, seen = {"last inside the window": (qi - size + 1, True), "first outside the window": (qi - size, False),
                "last kept token": (keep - 1, True), "first token not kept": (keep, False),
                "far key among hundreds": (1, True), "page border": (256, True)}[edge]
    lens = [qi + 20] if where == "prompt" else [qi - 10] + [1] * 30
    got, ref, _, _ = attention_case(dtype, 4, 2, D, D, size, keep, 40.0, lens, plant=(qi, kj, 25.0), seed=3)
    close(got, ref, dtype, edge)
    # the planted key carries the head's output when it is seen, and leaves no trace when it is not
    head0 = got[qi, :D]
    assert (float(head0.min()) > 4.0) == seen, (edge, float(head0.min()), float(head0.max()))


def test_windowed_cache_keeps_the_first_pages_and_gives_the_others_back():
    _, _, cache, slot = attention_case(torch.float32, 2, 1, 16, 16, 30, 70, None, [400, 1, 1])
    pages = cache.groups[0].pages[slot]
    assert pages[0] >= 0 and pages[1] >= 0            # positions 0..69 are kept: two pages
    assert pages[2] == -1 and pages[4] == -1 and pages[-1] >= 0
    free = cache.pages_free()[0]
    cache.end(slot)
    assert cache.pages_free()[0] > free


def gla_case(dtype, H, D, V, rank, tau, lens_steps, bias_shift=0.0, seed=0, width=40):
    spec = GatedLinearAttentionSpec(hidden_size=width, num_heads=H, head_dim=D, v_head_dim=V, decay_rank=rank, tau=tau, norm_eps=1e-5)
    part = build_part(spec, Runtime(DEV, dtype))
    p = {"q": rnd(H * D, width, seed=seed, scale=0.2), "k": rnd(H * D, width, seed=seed + 1, scale=0.2),
         "v": rnd(H * V, width, seed=seed + 2, scale=0.2), "g": rnd(H * V, width, seed=seed + 3, scale=0.2),
         "o": rnd(width, H * V, seed=seed + 4, scale=0.2), "norm": 1 + rnd(V, seed=seed + 5, scale=0.2),
         "a1": rnd(rank, width, seed=seed + 6, scale=0.3), "a2": rnd(H * D, rank, seed=seed + 7, scale=0.5),
         "a2.b": rnd(H * D, seed=seed + 8) + bias_shift}
    p = {k: v.to(dtype).double() for k, v in p.items()}
    part.bind({k: dev(v, torch.float32 if k in ("norm", "a2.b") else dtype) for k, v in p.items()})
    T = sum(lens_steps)
    h = rnd(T, width, seed=seed + 9).to(dtype).double()
    ref = plain.gla_mixer(h, p, {"heads": H, "dim": D, "vdim": V, "tau": tau}, 1e-5)
    cache = Cache([part.cache_requests()], 64 * 16, 4, DEV)
    other, slot = cache.begin(), cache.begin()
    t0, got = 0, []
    for n in lens_steps:
        m = 1 if n == 1 else 2
        ctx = build_context(cache, [(other, [0] * m, []), (slot, [0] * n, [])], DEV)
        a = torch.zeros(m + n, width, dtype=dtype, device=DEV)
        a[m:] = dev(h[t0:t0 + n], dtype)
        out = part.forward(ctx, cache.views(0), a)
        out = out.sum(dtype) if isinstance(out, api.Partial) else out
        got.append(out[m:].double().cpu())
        cache.commit(other, m), cache.commit(slot, n)
        t0 += n
    return torch.cat(got, 0), ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V,rank,tau", [(2, 16, 24, 4, 4.0), (4, 32, 64, 16, 16.0), (1, 32, 8, 12, 1.0), (3, 16, 32, 8, 8.0),
                                            (2, 64, 64, 16, 16.0), (1, 24, 12, 5, 2.0), (2, 128, 128, 8, 32.0)])
def test_gated_linear_attention_in_prompts_portions_and_single_tokens(dtype, H, D, V, rank, tau):
    got, ref = gla_case(dtype, H, D, V, rank, tau, [70, 2, 1, 1, 33, 1, 2, 64, 1])
    close(got, ref, dtype, "gated linear attention")


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_linear_attention_keeps_far_tokens_under_a_slow_decay(dtype):
    """A bias of +6 and tau 64 give decays of about 0.99996 a token: after 900 tokens the first ones still weigh."""
    got, ref = gla_case(dtype, 2, 32, 32, 8, 64.0, [600, 1, 1, 298], bias_shift=6.0, seed=4)
    close(got, ref, dtype, "slow decay")


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (12, 3, 4, 3), (6, 3, 1, 1), (4, 1, 2, 1), (3, 2, 3, 2), (64, 6, 8, 3),
                                               (256, 8, 8, 4), (5, 5, 5, 5)])
def test_router_choice_and_weights(E, top, groups, keep):
    """Logits spread over several units and corrections that reach below minus one (so that choice scores are
    negative: an expert outside the kept groups must count as minus infinity, not as zero). Tokens whose choice
    hangs on a difference below 1e-5 are left out."""
    T, W = 150, 32
    x = rnd(T, W, seed=E)
    wr = rnd(E, W, seed=E + 1, scale=0.4)
    corr = rnd(E, seed=E + 2, scale=0.8) - 1.0
    wsg = rnd(W, seed=E + 3, scale=0.3)
    z = x.float().double() @ wr.float().double().T
    idx_ref, wt_ref = plain.route(z, corr.float().double(), top, groups, keep, 2.5)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(T, top, dtype=torch.float32, device=DEV)
    sg = torch.empty(T, dtype=torch.float32, device=DEV)
    api.moe_route(x.float().to(DEV), wr.float().to(DEV), corr.float().to(DEV), wsg.float().to(DEV), top, groups, keep, 2.5, idx, wt, sg)
    close(sg, torch.sigmoid(x.float().double() @ wsg.float().double()), torch.float32, "shared gate", slack=0.1)
    # a close call: the reference's own choice changes when the logits move by 1e-5
    moved, _ = plain.route(z + 1e-5 * rnd(T, E, seed=9), corr.float().double(), top, groups, keep, 2.5)
    checked = 0
    for t in range(T):
        if sorted(moved[t].tolist()) != sorted(idx_ref[t].tolist()):
            continue
        checked += 1
        got = dict(zip(idx[t].tolist(), wt[t].tolist()))
        want = dict(zip(idx_ref[t].tolist(), wt_ref[t].tolist()))
        assert set(got) == set(want), (t, got, want)
        assert all(abs(got[e] - want[e]) < 1e-5 for e in want), (t, got, want)
    assert checked > T * 0.8


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,ff,top,groups,keep,shared,W", [(8, 40, 2, 4, 2, 48, 64), (6, 24, 3, 1, 1, None, 96), (3, 20, 2, 3, 2, 20, 48),
                                                           (8, 64, 2, 2, 2, 64, 128)])
def test_routed_feed_forward_with_given_routes(dtype, E, ff, top, groups, keep, shared, W):
    """The experts' arithmetic: the corrections are set wide apart so that every token takes the same experts in
    both implementations whatever the rounding; the weights still come from the tokens' own scores."""
    spec = RoutedMLPSpec(hidden_size=W, expert_ff=ff, num_experts=E, top=top, groups=groups, keep_groups=keep, route_scale=1.7,
                         shared_ff=shared)
    part = build_part(spec, Runtime(DEV, dtype))
    p = {}
    for e in range(E):
        p[f"e{e}.gate"], p[f"e{e}.up"] = rnd(ff, W, seed=3 * e, scale=0.15), rnd(ff, W, seed=3 * e + 1, scale=0.15)
        p[f"e{e}.down"] = rnd(W, ff, seed=3 * e + 2, scale=0.15)
    p["router"] = rnd(E, W, seed=100, scale=0.2)
    p["correction"] = torch.tensor([((7 * e) % E) * 3.0 for e in range(E)], dtype=torch.float64)
    if shared:
        p["shared.gate"], p["shared.up"] = rnd(shared, W, seed=101, scale=0.15), rnd(shared, W, seed=102, scale=0.15)
        p["shared.down"], p["shared.sg"] = rnd(W, shared, seed=103, scale=0.15), rnd(1, W, seed=104, scale=0.3)
    p = {k: v.to(dtype).double() for k, v in p.items()}
    f32 = ("router", "correction", "shared.sg")
    part.bind({k: dev(v, torch.float32 if k in f32 else dtype) for k, v in p.items()})
    m = {"router": {"top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}}
    for T in (1, 5, 150):
        h = rnd(T, W, seed=T).to(dtype).double()
        ref = plain.moe_ff(h, p, m)
        out = part.forward(None, dev(h, dtype))
        close(out, ref, dtype, f"{T} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward_with_the_tanh_form_of_gelu(dtype):
    W, I = 64, 104
    part = build_part(GatedMLPSpec(W, I, "gelu_tanh", names=("gate", "up", "down")), Runtime(DEV, dtype))
    p = {"gate": rnd(I, W, seed=1, scale=0.3), "up": rnd(I, W, seed=2, scale=0.3), "down": rnd(W, I, seed=3, scale=0.3)}
    p = {k: v.to(dtype).double() for k, v in p.items()}
    part.bind({k: dev(v, dtype) for k, v in p.items()})
    for T in (1, 7, 200):
        h = rnd(T, W, seed=T, scale=1.5).to(dtype).double()
        out = part.forward(None, dev(h, dtype))
        out = out.sum(dtype) if isinstance(out, api.Partial) else out
        close(out, plain.dense_ff(h, p), dtype, f"{T} rows")


# ------------------------------------------------------------------------------------ whole models
def plain_logits(folder, tokens):
    cfg, t = plain.read_model(folder)
    return plain.forward(cfg, t, tokens)


class Errors:
    """float32 must hold everywhere. In bfloat16 a router's choice may flip where two choice scores lie within
    rounding of each other (the plain implementation routes on float64 activations), so a few positions may be
    off; a fault in a kernel would put most of them off."""

    def __init__(self, dtype):
        self.dtype, self.n, self.bad = dtype, 0, []

    def add(self, err, bound, what):
        self.n += 1
        if err > bound:
            self.bad.append((what, err))

    def verdict(self):
        allowed = 0 if self.dtype in (torch.float32, "float32") else self.n // 10
        assert len(self.bad) <= allowed, f"{len(self.bad)} of {self.n} positions off: {self.bad[:5]}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_portions_batches_and_reused_slots(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name)
    model = load_model(folder, dtype)
    runner = Runner(model, 64 * 24, 6)
    lens = [1, 23, 131, 200]
    seqs = [random_tokens(cfg.vocab, n, 40 + i) for i, n in enumerate(lens)]
    ref = [plain_logits(folder, s) for s in seqs]
    errs = Errors(dtype)

    def check(out, pairs, what):
        out = out.cpu().double()
        for row, (i, p) in enumerate(pairs):
            errs.add(float((out[row] - ref[i][p]).abs().max()), tol(dtype, ref[i]), f"{name} {what}: sequence {i} position {p}")

    for round_ in range(2):        # the second round runs on the slots and pages the first gave back
        for i, s in enumerate(seqs):
            slot = runner.begin()
            want = sorted({0, len(s) // 2, len(s) - 1})
            check(runner.step([(slot, s, want)]), [(i, p) for p in want], "alone")
            runner.end(slot)
        # a ragged batch of prompts cut short, then one token each, shorter ones ending earlier
        cut = [1, 17, 100, 130]
        slots = [runner.begin() for _ in seqs]
        check(runner.step([(sl, s[:c], [c - 1]) for sl, s, c in zip(slots, seqs, cut)]), [(i, c - 1) for i, c in enumerate(cut)],
              "batch of prompts")
        live = [i for i in range(4) if cut[i] < lens[i]]
        k = 0
        while live and k < 40:
            out = runner.step([(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live])
            check(out, [(i, cut[i] + k) for i in live], f"decode step {k}")
            k += 1
            for i in [i for i in live if cut[i] + k >= lens[i]]:
                runner.end(slots[i])
                slots[i] = None
            live = [i for i in live if cut[i] + k < lens[i]]
        for sl in slots:
            if sl is not None:
                runner.end(sl)
        # portions of several sizes, down to two tokens and one
        s, i = seqs[3], 3
        slot = runner.begin()
        at = 0
        for n in [64, 2, 31, 1, 2, 70, 30]:
            check(runner.step([(slot, s[at:at + n], [0, n - 1])]), [(i, at), (i, at + n - 1)], f"portion of {n} at {at}")
            at += n
        runner.end(slot)
    errs.verdict()
    assert runner.cache.slots.n_live == 0 and all(f == runner.cache.num_pages for f in runner.cache.pages_free())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_through_the_decode_state_and_its_graph(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name, seed=3)
    model = load_model(folder, dtype)
    seqs = [random_tokens(cfg.vocab, n, 60 + i) for i, n in enumerate([150, 90])]
    ref = [plain_logits(folder, s) for s in seqs]
    for use_graph in (False, True):
        errs = Errors(dtype)
        runner = Runner(model, 64 * 12, 4)
        loop = DecodeLoop(runner, use_graph=use_graph)
        slots = [runner.begin() for _ in seqs]
        cut = [30, 5]
        runner.step([(sl, s[:c], []) for sl, s, c in zip(slots, seqs, cut)])
        for k in range(85):                          # windows of 24, 64 and 7 positions pass over decoded tokens, pages fill
            out = loop.forced_step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().double()
            for i in range(2):
                errs.add(float((out[i] - ref[i][cut[i] + k]).abs().max()), tol(dtype, ref[i]), f"graph={use_graph} step {k} sequence {i}")
        errs.verdict()
        for sl in slots:
            runner.end(sl)
    api.gemm_tc_check()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    folder, cfg = make_model(tmp_path, name, seed=5)
    pcfg, t = plain.read_model(folder)
    prompts = [random_tokens(cfg.vocab, n, 80 + i) for i, n in enumerate([3, 40, 77])]
    n_new = 30
    for dtype in DTYPES:
        eng = dk.Engine(folder, dtype=dtype)
        steps = list(eng.generate(prompts, n_new))
        again = list(dk.Engine(folder, dtype=dtype, use_graph=False, max_prefill_tokens=16).generate(prompts, n_new))
        for i, p in enumerate(prompts):
            emitted = [s[i] for s in steps]
            logits = plain.forward(pcfg, t, p + emitted[:-1])[len(p) - 1:]
            gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
            assert gap <= (1e-4 if dtype == torch.float32 else 0.12 * max(1.0, float(logits.abs().max()))), (name, dtype, i, gap)
            if dtype == torch.float32:               # prompts cut into portions of 16, plain launches: the same tokens
                assert emitted == [s[i] for s in again]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_ragged_schedule(tmp_path, dtype):
    folder, cfg = make_model(tmp_path, "B", seed=7)
    seqs = {"a": random_tokens(cfg.vocab, 140, 1), "b": random_tokens(cfg.vocab, 9, 2), "c": random_tokens(cfg.vocab, 66, 3)}
    ref = {k: plain_logits(folder, s) for k, s in seqs.items()}
    start = {"a": 130, "b": 1, "c": 60}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seqs["a"][:130], "want": [0, 63, 64, 129]},
                                     {"id": "b", "tokens": seqs["b"][:1], "want": [0]},
                                     {"id": "c", "tokens": seqs["c"][:60], "want": []}], "end": []}]
    for k in range(10):
        ent = [{"id": i, "tokens": [seqs[i][start[i] + k]], "want": [0] if (i != "c" or k % 2) else []}
               for i in ("a", "b", "c") if start[i] + k < len(seqs[i])]
        steps.append({"step": k + 1, "entries": ent, "end": [e["id"] for e in ent if start[e["id"]] + k + 1 == len(seqs[e["id"]])]})
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", "512"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    at = {"a": 0, "b": 0, "c": 0}
    errs = Errors(dtype)
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [(e["id"], at[e["id"]] + w) for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        if rows:
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(len(rows), cfg.vocab))
            for r, (i, p) in enumerate(rows):
                errs.add(float((got[r].double() - ref[i][p]).abs().max()), tol(dtype, ref[i]), (s["step"], i, p))
    errs.verdict()


def test_command_line_generates_with_a_pibulix_model(tmp_path):
    """Random weights from a config.json of this design through the command line, the tokens it prints against the
    plain implementation's greedy tokens."""
    from dryft_challenge_htn_2026_b200.cli import random_prompts

    cfg = dk.config_from_dict(SHAPES["A"])
    cfg.save(str(tmp_path))
    model_dir = str(tmp_path / "model")
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "dryft_challenge_htn_2026_b200.cli", "--random-weights", str(tmp_path / "config.json"),
                        "--save-model", model_dir, "--seed", "3", "--dtype", "float32", "--shapes", "2,30,6", "--samples", "1",
                        "--print-tokens"], capture_output=True, text=True, env=env, cwd=str(ROOT), timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens 2,30,6 seq ")]
    assert len(lines) == 2
    pcfg, t = plain.read_model(model_dir)
    prompts = random_prompts(2, 30, 1, cfg.vocab, False)
    for i, line in enumerate(lines):
        emitted = [int(x) for x in line.split(":")[1].split()]
        logits = plain.forward(pcfg, t, prompts[i] + emitted[:-1])[len(prompts[i]) - 1:]
        gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
        assert gap <= 1e-4, (i, gap)
