"""Nilivik without a GPU: config.json reading, the schedule its loop becomes, cache requests and the
page bookkeeping of a chunked key/value group, and the plain implementation's own consistency."""
import copy

import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_nilivik as plain
from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest
from dryft_challenge_htn_2026_b200.config.specs import (DenseMLPSpec, LinearAttentionSpec, MaskedAttentionSpec,
                                                        ParallelMixerSpec, ScalarRMSNormSpec, SinusoidSpec)
from dryft_challenge_htn_2026_b200.engine.model import CausalLM


def layer(ff=48, chunk=20, kv=1):
    return {"type": "parallel",
            "mixer": {"left": {"heads": 2, "kv_heads": kv, "dim": 16, "vdim": 8, "mask": {"size": chunk}, "scale": 0.25},
                      "right": {"heads": 3, "dim": 8, "vdim": 16, "decay": [0.5, 0.9, 0.99]},
                      "left_scale": 0.75, "right_scale": 1.25},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


BASE = dict(architecture="Nilivik", vocab=90, width=32, embedding={"scale": 3.0}, norm={"eps": 1e-6}, logit_softcap=12.0,
            loop={"start": 1, "stop": 3, "times": 2}, layers=[layer(), layer(None), layer(40, 33, 2), layer()])


def test_config_round_trip_and_registry():
    cfg = dk.config_from_dict(BASE)
    assert isinstance(cfg, dk.NilivikConfig) and "Nilivik" in dk.architectures()
    assert dk.config_from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"][2]["mixer"]["left"]["mask"]["size"] == 33
    # a single decay number stands for every head
    d = copy.deepcopy(BASE)
    d["layers"][0]["mixer"]["right"]["decay"] = 0.8
    assert dk.config_from_dict(d).layer_dicts()[0]["mixer"]["right"]["decay"] == [0.8, 0.8, 0.8]


def test_loop_becomes_schedule_entries_with_a_cache_each():
    spec = dk.config_from_dict(BASE).to_spec()
    got = [(e.layer, e.cache, e.add_embedding, e.add_row) for e in spec.schedule]
    assert got == [(0, 0, False, None), (1, 1, False, ("loop.step", 0)), (2, 2, False, None),
                   (1, 3, True, ("loop.step", 1)), (2, 4, False, None), (3, 5, False, None)]
    assert spec.tables == (("loop.step", (2, 32)),)
    assert [(i, p) for i, p in plain.layer_runs(BASE)] == [(e.layer, e.add_row[1] if e.add_row else None) for e in spec.schedule]
    no_loop = {k: v for k, v in BASE.items() if k != "loop"}
    spec = dk.config_from_dict(no_loop).to_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and spec.tables == () and not any(e.add_row for e in spec.schedule)
    once = dict(BASE, loop={"start": 0, "stop": 4, "times": 1})
    spec = dk.config_from_dict(once).to_spec()
    assert [(e.layer, e.add_embedding, e.add_row) for e in spec.schedule][0] == (0, False, ("loop.step", 0))
    empty = dict(BASE, loop={"start": 2, "stop": 2, "times": 3})      # a span without layers: nothing loops, the table is still the model's
    cfg = dk.config_from_dict(empty)
    spec = cfg.to_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and not any(e.add_row or e.add_embedding for e in spec.schedule)
    assert spec.tables == (("loop.step", (3, 32)),) and dk.config_from_dict(cfg.to_dict()) == cfg


def test_spec_carries_every_constant():
    spec = dk.config_from_dict(BASE).to_spec()
    assert spec.embed_scale == 3.0 and spec.logit_cap == 12.0 and spec.embed_position == SinusoidSpec(32, 10000.0)
    assert spec.final_norm == ScalarRMSNormSpec(32, 1e-6) and spec.embed_name == "embed" and spec.head_name == "head"
    l2 = spec.layers[2]
    assert isinstance(l2.mixer, ParallelMixerSpec) and l2.feed_forward == DenseMLPSpec(32, 40, "xielu")
    (pl, left, sl), (pr, right, sr) = l2.mixer.branches
    assert (pl, sl, pr, sr) == ("left.", 0.75, "right.", 1.25)
    assert left == MaskedAttentionSpec(32, 2, 2, 16, 8, 0.25, chunk=33, distance_bias=True, sink=True, output_gate=True)
    assert isinstance(right, LinearAttentionSpec) and right.decay == (0.5, 0.9, 0.99) and right.out_norm.dim == 48
    assert spec.layers[1].feed_forward is None and spec.layers[1].norm_post is None


def test_tensor_names_and_shapes():
    model = CausalLM(dk.config_from_dict(BASE).to_spec(), torch.float32, "cpu")
    decls = model.param_decls(False)
    want = {"embed": (90, 32), "head": (90, 32), "final.norm": (), "loop.step": (2, 32), "l0.norm1": (), "l0.norm2": (),
            "l2.mix.left.q": (32, 32), "l2.mix.left.k": (32, 32), "l2.mix.left.v": (16, 32), "l2.mix.left.g": (16, 32),
            "l2.mix.left.o": (32, 16), "l2.mix.left.r1": (2,), "l2.mix.left.r2": (2,), "l2.mix.left.sink": (2,),
            "l2.mix.right.q": (24, 32), "l2.mix.right.k": (24, 32), "l2.mix.right.v": (48, 32), "l2.mix.right.g": (48, 32),
            "l2.mix.right.o": (32, 48), "l2.mix.right.norm": (48,), "l2.mlp.up": (40, 32), "l2.mlp.down": (32, 40),
            "l2.mlp.act": (2,)}
    for name, shape in want.items():
        assert tuple(decls[name].shape) == shape, name
    assert "l1.norm2" not in decls and not any(n.startswith("l1.mlp.") for n in decls)


@pytest.mark.parametrize("change,fragment", [
    (lambda d: d["layers"][0].update(type="serial"), "type"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "mlp"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d.update(architecture="Nobody"), "registered"),
])
def test_what_is_not_implemented_is_an_error(change, fragment):
    d = copy.deepcopy(BASE)
    change(d)
    with pytest.raises(dk.ConfigError, match=fragment):
        dk.config_from_dict(d).to_spec()


def test_chunked_group_gives_back_pages_before_the_current_chunk():
    req = KVRequest(1, 16, None, torch.float32, 8, 100)
    cache = Cache([[req], [req]], 64 * 12, 4, "cpu", allocate=False)
    g = cache.groups[0]
    s = cache.begin()
    cache.reserve(s, 330)
    cache.commit(s, 330)                                  # next position 330 sits in the chunk that starts at 300
    assert [p >= 0 for p in g.pages[s]] == [False] * 4 + [True] * 2       # pages 0..3 end before 300 = 4 * 64 + 44
    cache.reserve(s, 75)
    cache.commit(s, 75)                                   # 405: chunk starts at 400 = 6 * 64 + 16
    assert [p >= 0 for p in g.pages[s]] == [False] * 6 + [True]
    t = cache.begin()
    cache.reserve(t, 64 * 11)                             # the freed pages serve another sequence
    assert g.pool.n_free == 0
    cache.end(s), cache.end(t)
    assert g.pool.n_free == 12


def test_plain_recurrence_equals_its_closed_form_and_attention_masks_by_chunk():
    g = torch.Generator().manual_seed(0)
    T, H, D, Dv = 37, 2, 5, 3
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (D, D, Dv))
    decay = [0.8, 0.97]
    out, last = plain.decay_recurrence(q, k, v, decay)
    for h in range(H):
        w = torch.tensor([[decay[h] ** (i - j) if j <= i else 0.0 for j in range(T)] for i in range(T)], dtype=torch.float64)
        assert torch.allclose(out[:, h], ((q[:, h] @ k[:, h].T) * w) @ v[:, h], atol=1e-10)
    half, mid = plain.decay_recurrence(q[:20], k[:20], v[:20], decay)
    rest, last2 = plain.decay_recurrence(q[20:], k[20:], v[20:], decay, mid)
    assert torch.allclose(torch.cat([half, rest]), out, atol=1e-12) and torch.allclose(last, last2, atol=1e-12)
    # a value planted just before a chunk's first position is invisible to that chunk, one planted on it is seen
    kk, vv = k[:, :1].clone(), torch.zeros(T, 1, Dv, dtype=torch.float64)
    vv[9], vv[10] = 100.0, -100.0
    o = plain.attention_core(q, kk, vv, 0.3, chunk=10)
    assert float(o[10:20].max()) <= 0 and float(o[:10, :, 0].min()) >= 0 and float(o[20:].abs().max()) == 0
    z = torch.tensor([-1e-9, 0.0, 1e-9], dtype=torch.float64)
    f = plain.xielu(z, torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64))
    assert float(f[1]) == 0.0 and abs(float(f[2] - f[0]) / 2e-9 - 0.5) < 1e-6       # continuous, slope 1/2 at zero
