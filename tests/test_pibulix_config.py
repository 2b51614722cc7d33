"""Pibulix without a GPU: config.json reading, layers that run on another layer's weights as schedule entries,
tensor names, cache requests, the page bookkeeping of a window that keeps its first tokens, and the plain
implementation's own consistency."""
import copy
import math

import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_pibulix as plain
from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest, StateRequest
from dryft_challenge_htn_2026_b200.config.specs import (GatedLinearAttentionSpec, GatedMLPSpec, MaskedAttentionSpec,
                                                        OnePlusRMSNormSpec, PostNormLayerSpec, RotaryPartSpec, RoutedMLPSpec)
from dryft_challenge_htn_2026_b200.engine.model import CausalLM

ATT = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 3, "scale": 0.3, "softcap": 25.0,
                                      "rot": {"dims": 8, "base": 1000.0}, "mask": {"size": 20, "keep_first": 2}},
       "mlp": {"kind": "dense", "ff": 48}}
GLA = {"type": "gla", "mixer": {"heads": 3, "dim": 8, "vdim": 16, "tau": 4.0},
       "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}},
               "shared": {"ff": 40}}}
BASE = dict(architecture="Pibulix", vocab=90, width=32, norm={"eps": 1e-6}, postln_alpha=2.5,
            layers=[ATT, GLA, dict(ATT, weights_of=0), dict(GLA, mlp=None), dict(GLA, weights_of=1)])


def test_config_round_trip_and_registry():
    cfg = dk.config_from_dict(BASE)
    assert isinstance(cfg, dk.PibulixConfig) and "Pibulix" in dk.architectures()
    assert dk.config_from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"][2]["weights_of"] == 0 and cfg.to_dict()["layers"][0]["mixer"]["mask"] == {"size": 20, "keep_first": 2}
    shaped = cfg.with_shapes({"l1.mix.a1": (5, 32), "l3.mix.a1": (7, 32)})
    assert shaped.decay_rank == (None, 5, None, 7, 5) and dk.config_from_dict(shaped.to_dict()) == shaped


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="conv"), "not implemented"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "not implemented"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "fit together"),
    (lambda d: d["layers"][2].update(weights_of=4), "tensors of its own"),
    (lambda d: d["layers"][2].update(mixer=dict(d["layers"][2]["mixer"], scale=0.5)), "described differently"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_config_errors(change, message):
    d = copy.deepcopy(BASE)
    change(d)
    with pytest.raises(dk.ConfigError, match=message):
        dk.config_from_dict(d)


def test_shared_weights_become_schedule_entries_with_a_cache_each():
    spec = dk.config_from_dict(BASE).to_spec()
    assert [ls.prefix for ls in spec.layers] == ["l0.", "l1.", "l3."]
    assert [(e.layer, e.cache, e.writes) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (0, 2, True), (2, 3, True), (1, 4, True)]
    model = CausalLM(spec, torch.float32, "cpu")
    reqs = model.entry_requests()
    assert reqs[0] == reqs[2] == [KVRequest(2, 16, 20, torch.float32, 8, None, 2), StateRequest((2, 4 * 16 + 2 * 16 + 2 * 8), torch.float32)]
    assert reqs[1] == reqs[3] == reqs[4] == [StateRequest((3, 8, 16), torch.float32)]
    cache = Cache(reqs, 64 * 8, 4, "cpu", allocate=False)
    assert sorted(len(g.entries) for g in cache.groups) == [2, 2, 3]


def test_spec_carries_every_constant():
    spec = dk.config_from_dict(BASE).to_spec()
    l0, l1, l3 = spec.layers
    assert isinstance(l0, PostNormLayerSpec) and l0.alpha == 2.5 and l0.norm_mix == OnePlusRMSNormSpec(32, 1e-6)
    m = l0.mixer
    assert isinstance(m, MaskedAttentionSpec) and (m.num_heads, m.num_kv_heads, m.head_dim, m.v_head_dim) == (4, 2, 16, 8)
    assert (m.window, m.keep_first, m.softcap, m.scale, m.conv_taps, m.unit_sink) == (20, 2, 25.0, 0.3, 3, True)
    assert m.position == RotaryPartSpec(8, 1000.0) and m.qk_norm.dim == 16 and not m.sink and not m.distance_bias
    assert l0.feed_forward == GatedMLPSpec(32, 48, "gelu_tanh", names=("gate", "up", "down"))
    assert l1.mixer == GatedLinearAttentionSpec(32, 3, 8, 16, 16, 4.0, 1e-6)
    assert l1.feed_forward == RoutedMLPSpec(32, 24, 6, 2, 3, 2, 1.5, 40, "silu")
    assert l3.feed_forward is None and l3.norm_ff is None
    assert spec.final_norm == OnePlusRMSNormSpec(32, 1e-6) and spec.tie_embeddings is False
    # options left out of config.json: no mask, no rotation, one tap, no cap
    d = copy.deepcopy(BASE)
    d["layers"] = [copy.deepcopy(ATT)]
    for k in ("mask", "rot", "conv", "softcap"):
        d["layers"][0]["mixer"].pop(k)
    m = dk.config_from_dict(d).to_spec().layers[0].mixer
    assert (m.window, m.keep_first, m.softcap, m.conv_taps, m.position) == (None, 0, None, None, None)


def test_what_an_entry_leaves_out():
    d = copy.deepcopy(BASE)
    d["layers"][2] = {"weights_of": 0}                       # only the pointer: the rest is layer 0's
    d["layers"][1] = dict(GLA, mixer={"heads": 3, "dim": 8, "tau": 4.0})
    d["layers"][4] = dict(d["layers"][1], weights_of=1)
    d["layers"][0] = dict(ATT, mixer={k: v for k, v in ATT["mixer"].items() if k not in ("kv_heads", "vdim")})
    cfg = dk.config_from_dict(d)
    l = cfg.layer_dicts()
    assert l[2]["mixer"] == l[0]["mixer"] and l[2]["weights_of"] == 0
    assert l[0]["mixer"]["kv_heads"] == 4 and l[0]["mixer"]["vdim"] == 16 and l[1]["mixer"]["vdim"] == 8


def test_tensor_names_and_shapes():
    cfg = dk.config_from_dict(BASE).with_shapes({"l3.mix.a1": (7, 32)})
    decls = CausalLM(cfg.to_spec(), torch.float32, "cpu").param_decls(False)
    shapes = {k: tuple(v.shape) for k, v in decls.items()}
    assert not any(k.startswith(("l2.", "l4.")) for k in shapes)
    want = {"embed": (90, 32), "head": (90, 32), "final.norm": (32,), "l0.norm1": (32,), "l0.norm2": (32,), "l0.mix.q": (64, 32),
            "l0.mix.k": (32, 32), "l0.mix.v": (16, 32), "l0.mix.o": (32, 32), "l0.mix.q.conv": (64, 3), "l0.mix.k.conv": (32, 3),
            "l0.mix.v.conv": (16, 3), "l0.mix.q.norm": (16,), "l0.mix.k.norm": (16,), "l0.mlp.gate": (48, 32), "l0.mlp.down": (32, 48),
            "l1.mix.q": (24, 32), "l1.mix.v": (48, 32), "l1.mix.g": (48, 32), "l1.mix.o": (32, 48), "l1.mix.norm": (16,),
            "l1.mix.a1": (16, 32), "l1.mix.a2": (24, 16), "l1.mix.a2.b": (24,), "l1.mlp.e5.up": (24, 32), "l1.mlp.e0.down": (32, 24),
            "l1.mlp.router": (6, 32), "l1.mlp.correction": (6,), "l1.mlp.shared.gate": (40, 32), "l1.mlp.shared.sg": (1, 32),
            "l3.mix.a1": (7, 32), "l3.mix.a2": (24, 7), "l3.norm1": (32,)}
    for k, v in want.items():
        assert shapes[k] == v, (k, shapes.get(k))
    assert "l3.norm2" not in shapes and "l3.mlp.router" not in shapes


def test_pages_of_a_window_that_keeps_its_first_tokens():
    cache = Cache([[KVRequest(1, 16, 30, torch.float32, 16, None, 70)], [KVRequest(1, 16, 30, torch.float32, 16, None, 0)]],
                  64 * 16, 2, "cpu", allocate=False)
    kept, plain_window = cache.groups
    s = cache.begin()
    cache.reserve(s, 400)
    cache.commit(s, 400)
    assert [p >= 0 for p in kept.pages[s]] == [True, True, False, False, False, True, True]
    assert [p >= 0 for p in plain_window.pages[s]] == [False, False, False, False, False, True, True]
    for _ in range(200):
        cache.reserve(s, 1)
        cache.commit(s, 1)
    assert [p >= 0 for p in kept.pages[s]] == [True, True] + [False] * 6 + [True, True]
    cache.end(s)
    assert cache.pages_free() == [16, 16]
    t = cache.begin()                           # the slot and the pages come again
    cache.reserve(t, 64 * 16)
    assert cache.pages_free() == [0, 0]


def test_plain_recurrence_against_its_closed_form():
    T, H, D, V = 9, 2, 3, 4
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(T, H, D, generator=g, dtype=plain.F), torch.randn(T, H, D, generator=g, dtype=plain.F)
    v = torch.randn(T, H, V, generator=g, dtype=plain.F)
    alpha = torch.rand(T, H, D, generator=g, dtype=plain.F) * 0.5 + 0.5
    o, S = plain.gla_recurrence(q, k, v, alpha)
    for t in range(T):
        want = torch.zeros(H, V, dtype=plain.F)
        for j in range(t + 1):      # key j reaches step t through the decays of steps j+1..t, channel by channel
            w = alpha[j + 1:t + 1].prod(0) if j < t else torch.ones(H, D, dtype=plain.F)
            want += torch.einsum("hd,hd,hv->hv", q[t], w * k[j], v[j])
        assert torch.allclose(o[t], want, atol=1e-12)
    # cut in two, the state carried over
    o1, S1 = plain.gla_recurrence(q[:4], k[:4], v[:4], alpha[:4])
    o2, S2 = plain.gla_recurrence(q[4:], k[4:], v[4:], alpha[4:], S1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(S2, S)


def test_plain_router_and_masks():
    z = torch.tensor([[2.0, 1.9, -3.0, -3.0, 0.5, 0.4, 1.0, -9.0]], dtype=plain.F)
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0], dtype=plain.F)
    idx, w = plain.route(z, corr, 3, 4, 2, 2.0)          # groups (0,1) (2,3) (4,5) (6,7): the best two are the first and the third
    assert sorted(idx[0].tolist()) == [0, 1, 4] and abs(float(w.sum()) - 2.0) < 1e-12
    idx, _ = plain.route(z, corr - 5.0, 3, 4, 2, 2.0)    # all choice scores negative: the others count as minus infinity, not 0
    assert sorted(idx[0].tolist()) == [0, 1, 4]
    corr[6] = 3.0                                         # a correction moves the choice but not the weight
    idx, w = plain.route(z, corr, 1, 4, 1, 1.0)
    assert idx[0].tolist() == [6] and abs(float(w[0, 0]) - 1.0) < 1e-12
    assert plain.visible(100, 31, 70, 4) and not plain.visible(100, 30, 70, 4) and plain.visible(100, 3, 70, 4)
    assert not plain.visible(100, 4, 70, 4) and not plain.visible(5, 6, 70, 4)
    x = torch.arange(8, dtype=plain.F).view(1, 1, 8)
    r = plain.rotate_partial(x, torch.tensor([3]), 4, 100.0)
    assert torch.equal(r[..., 4:], x[..., 4:]) and abs(float(r[0, 0, 0]) - (0 * math.cos(3) - 2 * math.sin(3))) < 1e-12
