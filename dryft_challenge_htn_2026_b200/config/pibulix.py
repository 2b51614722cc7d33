"""Pibulix: a decoder with the norm after the sum, whose layers are either softmax attention (grouped
key/value heads, a short causal convolution on q, k and v, a norm per q and k head, a rotation of the heads'
first coordinates, capped scores, a sliding window that keeps the sequence's first tokens, one added to the
softmax's denominator) or gated linear attention (a decay per key channel and token from a two-step
projection), each followed by a gated feed-forward (dense with the tanh form of GELU, or a mixture of experts
with a sigmoid router, groups, a correction for the choice and a gated shared expert) or by none. A layer may
run on another layer's weights with a cache or state of its own.

config.json keys (every size, and every constant that differs between models of the design):
  architecture "Pibulix"; vocab, width; norm.eps; postln_alpha;
  layers[i] = {type: "attention", mixer: {heads, kv_heads, dim, vdim, conv, scale, softcap, rot: {dims, base},
                                          mask: {size, keep_first}}, mlp: ...}
            | {type: "gla", mixer: {heads, dim, vdim, tau}, mlp: ...}
     with mlp = {kind: "dense", ff} | {kind: "moe", expert: {ff}, router: {experts, top, scale, groups: {count, keep}},
                                       shared: {ff}} | null,
     and optionally weights_of: j (the layer has no tensors; it runs on layer j's; what its entry leaves out is layer j's).
  Left out: kv_heads = heads, vdim = dim, conv = 1, softcap = none, rot = none, mask = none, keep_first = 0, tau = 1,
  router.scale = 1, router.groups = one group, postln_alpha = 1.
Tensors: embed, head, final.norm, and per layer with tensors l<i>.norm1, l<i>.norm2,
  attention: l<i>.mix.{q,k,v,o}, .mix.{q,k,v}.conv [channels, taps], .mix.{q,k}.norm [dim];
  gla: l<i>.mix.{q,k,v,g,o}, .mix.norm [vdim], .mix.a1 [rank, width], .mix.a2 [heads*dim, rank], .mix.a2.b;
  dense: l<i>.mlp.{gate,up,down}; moe: l<i>.mlp.e<k>.{gate,up,down}, .mlp.router, .mlp.correction,
  .mlp.shared.{gate,up,down}, .mlp.shared.sg [1, width].
The inner size of the decay's two-step projection is not a config key: it is the shape of l<i>.mix.a1, so
``to_spec`` takes it from ``decay_rank`` (set by ``with_shapes`` from a checkpoint, or given).
"""
from dataclasses import dataclass, field, replace

from .base import ConfigError, ModelConfig, get
from .nilivik import _freeze, _section, _thaw
from .specs import (GatedLinearAttentionSpec, GatedMLPSpec, MaskedAttentionSpec, ModelSpec, OnePlusRMSNormSpec,
                    PostNormLayerSpec, RMSNormSpec, RotaryPartSpec, RoutedMLPSpec, ScheduleEntry)

DEFAULT_DECAY_RANK = 16


def _check_mlp(mlp, where):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}.mlp must be an object or null")
    kind = mlp.get("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": get(mlp, "ff", int, positive=True)}
    if kind == "moe":
        r = _section(mlp, "router", f"{where}.mlp")
        g = r.get("groups") or {"count": 1, "keep": 1}
        out = {"kind": "moe", "expert": {"ff": get(_section(mlp, "expert", f"{where}.mlp"), "ff", int, positive=True)},
               "router": {"experts": get(r, "experts", int, positive=True), "top": get(r, "top", int, positive=True),
                          "scale": get(r, "scale", float, 1.0),
                          "groups": {"count": get(g, "count", int, positive=True), "keep": get(g, "keep", int, positive=True)}}}
        E, gc, gk = out["router"]["experts"], out["router"]["groups"]["count"], out["router"]["groups"]["keep"]
        if E % gc or gk > gc or out["router"]["top"] > gk * (E // gc):
            raise ConfigError(f"config.json: {where}.mlp.router: {E} experts, {gc} groups, {gk} kept, "
                              f"{out['router']['top']} chosen do not fit together")
        if mlp.get("shared") is not None:
            out["shared"] = {"ff": get(_section(mlp, "shared", f"{where}.mlp"), "ff", int, positive=True)}
        return out
    raise ConfigError(f"config.json: {where}.mlp kind {kind!r} is not implemented (dense, moe or null)")


def _check_mixer(kind, m, where):
    if kind == "attention":
        H = get(m, "heads", int, positive=True)
        G = get(m, "kv_heads", int, H, positive=True)          # left out: as many key/value heads as query heads
        if H % G:
            raise ConfigError(f"config.json: {where}: {H} heads are not a multiple of {G} key/value heads")
        dim = get(m, "dim", int, positive=True)
        out = {"heads": H, "kv_heads": G, "dim": dim, "vdim": get(m, "vdim", int, dim, positive=True),
               "conv": get(m, "conv", int, 1, positive=True), "scale": get(m, "scale", float),
               "softcap": get(m, "softcap", float, 0.0)}
        rot = m.get("rot")
        if rot is not None:
            rot = _section(m, "rot", where)
            out["rot"] = {"dims": get(rot, "dims", int), "base": get(rot, "base", float, positive=True)}
            if out["rot"]["dims"] % 2 or not 0 <= out["rot"]["dims"] <= out["dim"]:
                raise ConfigError(f"config.json: {where}.rot.dims {out['rot']['dims']} must be even and at most dim")
        mask = m.get("mask")
        if mask is not None:
            mask = _section(m, "mask", where)
            out["mask"] = {"size": get(mask, "size", int, positive=True), "keep_first": get(mask, "keep_first", int, 0)}
            if out["mask"]["keep_first"] < 0:
                raise ConfigError(f"config.json: {where}.mask.keep_first must not be negative")
        return out
    if kind == "gla":
        dim = get(m, "dim", int, positive=True)
        return {"heads": get(m, "heads", int, positive=True), "dim": dim, "vdim": get(m, "vdim", int, dim, positive=True),
                "tau": get(m, "tau", float, 1.0, positive=True)}
    raise ConfigError(f"config.json: {where}.type {kind!r} is not implemented (attention, gla)")


@dataclass(frozen=True)
class PibulixConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    layers: tuple = field(default=())          # the config's layer entries, checked, frozen
    decay_rank: tuple = field(default=())      # per layer: inner size of a gla layer's decay projection (None elsewhere)

    architecture = "Pibulix"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        for i, lc in enumerate(layers):
            if not isinstance(lc, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            j = lc.get("weights_of")
            if isinstance(j, int) and not isinstance(j, bool) and 0 <= j < len(layers) and isinstance(layers[j], dict):
                # what an entry that runs on another layer's weights leaves out is that layer's
                lc = dict({k: v for k, v in layers[j].items() if k != "weights_of"}, **lc)
            kind = lc.get("type")
            entry = {"type": kind, "mixer": _check_mixer(kind, _section(lc, "mixer", f"layers[{i}]"), f"layers[{i}].mixer"),
                     "mlp": _check_mlp(lc.get("mlp"), f"layers[{i}]")}
            if lc.get("weights_of") is not None:
                entry["weights_of"] = get(lc, "weights_of", int)
            checked.append(entry)
        for i, lc in enumerate(checked):
            j = lc.get("weights_of")
            if j is None:
                continue
            if not 0 <= j < len(checked) or j == i or "weights_of" in checked[j]:
                raise ConfigError(f"config.json: layers[{i}].weights_of {j} must name another layer that has tensors of its own")
            if {k: v for k, v in lc.items() if k != "weights_of"} != checked[j]:
                raise ConfigError(f"config.json: layers[{i}] runs on the weights of layer {j} but is described differently")
        ranks = d.get("decay_rank")       # not a key of the design's config.json; kept when this library writes one
        if ranks is None:
            ranks = [DEFAULT_DECAY_RANK if lc["type"] == "gla" else None for lc in checked]
        if not isinstance(ranks, list) or len(ranks) != len(checked):
            raise ConfigError("config.json: 'decay_rank' must give one entry per layer")
        return cls(vocab=get(d, "vocab", int, positive=True), width=get(d, "width", int, positive=True),
                   norm_eps=get(_section(d, "norm", "the"), "eps", float, positive=True),
                   postln_alpha=get(d, "postln_alpha", float, 1.0), layers=tuple(_freeze(l) for l in checked),
                   decay_rank=tuple(ranks))

    def layer_dicts(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self):
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "postln_alpha": self.postln_alpha, "layers": self.layer_dicts()}
        if any(r not in (None, DEFAULT_DECAY_RANK) for r in self.decay_rank):
            d["decay_rank"] = list(self.decay_rank)
        return d

    def with_shapes(self, shapes):
        """The config with what only the checkpoint's tensor shapes say: the inner size of each gla layer's
        decay projection (rows of l<i>.mix.a1). ``shapes``: tensor name -> shape."""
        ranks = list(self.decay_rank)
        for i, lc in enumerate(self.layer_dicts()):
            name = f"l{lc.get('weights_of', i)}.mix.a1"
            if lc["type"] == "gla" and name in shapes and len(shapes[name]) == 2:
                ranks[i] = int(shapes[name][0])
        return replace(self, decay_rank=tuple(ranks))

    def owners(self):
        """Per layer the layer whose tensors it runs on (itself unless it says weights_of)."""
        return [lc.get("weights_of", i) for i, lc in enumerate(self.layer_dicts())]

    def to_spec(self):
        W, eps = self.width, self.norm_eps
        dicts, owners = self.layer_dicts(), self.owners()
        own = sorted(set(owners))                  # layers with tensors of their own, in order
        index = {i: k for k, i in enumerate(own)}
        layers = []
        for i in own:
            lc, m = dicts[i], dicts[i]["mixer"]
            if lc["type"] == "attention":
                mask, rot = m.get("mask"), m.get("rot")
                mixer = MaskedAttentionSpec(
                    hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                    scale=m["scale"], window=mask["size"] if mask else None, keep_first=mask["keep_first"] if mask else 0,
                    softcap=m["softcap"] or None, unit_sink=True, conv_taps=m["conv"] if m["conv"] > 1 else None,
                    qk_norm=RMSNormSpec(m["dim"], eps), position=RotaryPartSpec(rot["dims"], rot["base"]) if rot and rot["dims"] else None)
            else:
                mixer = GatedLinearAttentionSpec(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                 decay_rank=self.decay_rank[i] or DEFAULT_DECAY_RANK, tau=m["tau"], norm_eps=eps)
            mlp = lc["mlp"]
            if mlp is None:
                ff = None
            elif mlp["kind"] == "dense":
                ff = GatedMLPSpec(W, mlp["ff"], "gelu_tanh", names=("gate", "up", "down"))
            else:
                r = mlp["router"]
                ff = RoutedMLPSpec(hidden_size=W, expert_ff=mlp["expert"]["ff"], num_experts=r["experts"], top=r["top"],
                                   groups=r["groups"]["count"], keep_groups=r["groups"]["keep"], route_scale=r["scale"],
                                   shared_ff=mlp["shared"]["ff"] if mlp.get("shared") else None, activation="silu")
            names = (("mixer", "mix."), ("norm_mix", "norm1")) + ((("feed_forward", "mlp."), ("norm_ff", "norm2")) if ff else ())
            layers.append(PostNormLayerSpec(prefix=f"l{i}.", mixer=mixer, norm_mix=OnePlusRMSNormSpec(W, eps), feed_forward=ff,
                                            norm_ff=OnePlusRMSNormSpec(W, eps) if ff else None, alpha=self.postln_alpha,
                                            names=names))
        schedule = tuple(ScheduleEntry(layer=index[o], cache=k, writes=True) for k, o in enumerate(owners))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         schedule=schedule, final_norm=OnePlusRMSNormSpec(W, eps), tie_embeddings=False,
                         max_positions=1 << 20, embed_name="embed", final_norm_prefix="final.norm", head_name="head")
