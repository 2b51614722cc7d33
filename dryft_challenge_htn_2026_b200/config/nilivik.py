"""Nilivik: a decoder whose layers run two mixers side by side (chunked softmax attention with a
logarithmic distance bias, a sink and an output gate; linear attention with a constant decay per head),
with a scalar RMS norm, an xIELU feed-forward, a sinusoidal position vector on a scaled embedding, a
span of layers that runs several times with the same weights, and capped logits.

config.json keys (all sizes and all constants that differ between models of the design):
  architecture "Nilivik"; vocab, width; embedding.scale; norm.eps; logit_softcap;
  layers[i] = {type: "parallel", mixer: {left: {heads, kv_heads, dim, vdim, scale, mask: {size}},
               right: {heads, dim, vdim, decay}, left_scale, right_scale}, mlp: {kind: "dense", ff} | null};
  loop = {start, stop, times}: layers start .. stop-1 run ``times`` times, each pass with a cache of its own.
Tensors: embed, head, final.norm, loop.step [times, width], and per layer l<i>.norm1, l<i>.norm2,
l<i>.mix.left.{q,k,v,g,o,r1,r2,sink}, l<i>.mix.right.{q,k,v,g,o,norm}, l<i>.mlp.{up,down,act}.
"""
import copy
from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig, get
from .specs import (DenseMLPSpec, LayerSpec, LinearAttentionSpec, MaskedAttentionSpec, ModelSpec, ParallelMixerSpec,
                    RMSNormSpec, ScalarRMSNormSpec, ScheduleEntry, SinusoidSpec)

SINUSOID_BASE = 10000.0      # fixed by the design
LOOP_TABLE = "loop.step"


def _section(d, key, what):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {what} '{key}' must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class NilivikConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: float            # 0: logits are not capped
    loop_start: int
    loop_stop: int
    loop_times: int
    layers: tuple = field(default=())          # the config's layer entries, checked, as plain dicts
    loop_given: bool = True                    # config.json has a 'loop' section (then the model has its 'loop.step' table)

    architecture = "Nilivik"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        for i, lc in enumerate(layers):
            if not isinstance(lc, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = lc.get("type")
            if kind != "parallel":
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not implemented (parallel)")
            m = _section(lc, "mixer", f"layers[{i}]")
            left, right = _section(m, "left", f"layers[{i}].mixer"), _section(m, "right", f"layers[{i}].mixer")
            H, G = get(left, "heads", int, positive=True), get(left, "kv_heads", int, positive=True)
            if H % G:
                raise ConfigError(f"config.json: layers[{i}]: {H} heads are not a multiple of {G} key/value heads")
            mask = left.get("mask")
            size = None if mask is None else get(_section(left, "mask", f"layers[{i}].mixer.left"), "size", int, positive=True)
            Hr = get(right, "heads", int, positive=True)
            decay = right.get("decay")
            if isinstance(decay, (int, float)) and not isinstance(decay, bool):
                decay = [float(decay)] * Hr
            if not isinstance(decay, list) or len(decay) != Hr or not all(isinstance(x, (int, float)) for x in decay):
                raise ConfigError(f"config.json: layers[{i}].mixer.right.decay must give one number per head")
            mlp = lc.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp kind {mlp!r} is not implemented (dense or null)")
                mlp = {"kind": "dense", "ff": get(mlp, "ff", int, positive=True)}
            checked.append({
                "type": "parallel",
                "mixer": {
                    "left": {"heads": H, "kv_heads": G, "dim": get(left, "dim", int, positive=True),
                             "vdim": get(left, "vdim", int, positive=True), "scale": get(left, "scale", float),
                             "mask": None if size is None else {"size": size}},
                    "right": {"heads": Hr, "dim": get(right, "dim", int, positive=True),
                              "vdim": get(right, "vdim", int, positive=True), "decay": [float(x) for x in decay]},
                    "left_scale": get(m, "left_scale", float), "right_scale": get(m, "right_scale", float)},
                "mlp": mlp})
        n = len(checked)
        loop = d.get("loop")
        if loop is None:
            start, stop, times = 0, 0, 1
        else:
            loop = _section(d, "loop", "the")
            start, stop, times = get(loop, "start", int), get(loop, "stop", int), get(loop, "times", int, positive=True)
            if not 0 <= start <= stop <= n:
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {n} layers")
        emb = d.get("embedding") or {}
        return cls(vocab=get(d, "vocab", int, positive=True), width=get(d, "width", int, positive=True),
                   embedding_scale=get(emb, "scale", float, 1.0),
                   norm_eps=get(_section(d, "norm", "the"), "eps", float, positive=True),
                   logit_softcap=get(d, "logit_softcap", float, 0.0), loop_start=start, loop_stop=stop, loop_times=times,
                   layers=tuple(_freeze(l) for l in checked), loop_given=loop is not None)

    def layer_dicts(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self):
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": self.layer_dicts()}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.loop_given:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return d

    def runs(self):
        """[(layer, pass number or None)] in running order; the number is set on the first layer of a
        pass of the loop."""
        n = len(self.layers)
        a, b = self.loop_start, self.loop_stop
        out = [(i, None) for i in range(a)]
        for p in range(self.loop_times if b > a else 0):
            out += [(i, p if i == a else None) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]

    def to_spec(self):
        W, eps = self.width, self.norm_eps
        layers = []
        for i, lc in enumerate(self.layer_dicts()):
            m = lc["mixer"]
            l, r = m["left"], m["right"]
            left = MaskedAttentionSpec(hidden_size=W, num_heads=l["heads"], num_kv_heads=l["kv_heads"], head_dim=l["dim"],
                                       v_head_dim=l["vdim"], scale=l["scale"],
                                       chunk=l["mask"]["size"] if l["mask"] else None, distance_bias=True, sink=True,
                                       output_gate=True)
            right = LinearAttentionSpec(hidden_size=W, num_heads=r["heads"], head_dim=r["dim"], v_head_dim=r["vdim"],
                                        decay=tuple(r["decay"]), out_norm=RMSNormSpec(r["heads"] * r["vdim"], eps),
                                        output_gate=True)
            mixer = ParallelMixerSpec(W, (("left.", left, m["left_scale"]), ("right.", right, m["right_scale"])))
            ff = DenseMLPSpec(W, lc["mlp"]["ff"], "xielu") if lc["mlp"] else None
            names = (("norm_in", "norm1"), ("mixer", "mix.")) + ((("norm_post", "norm2"), ("feed_forward", "mlp.")) if ff else ())
            layers.append(LayerSpec(prefix=f"l{i}.", norm_in=ScalarRMSNormSpec(W, eps), mixer=mixer,
                                    norm_post=ScalarRMSNormSpec(W, eps) if ff else None, feed_forward=ff, names=names))
        schedule = tuple(ScheduleEntry(layer=i, cache=k, writes=True, add_embedding=p is not None and p > 0,
                                       add_row=(LOOP_TABLE, p) if p is not None else None)
                         for k, (i, p) in enumerate(self.runs()))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         schedule=schedule, final_norm=ScalarRMSNormSpec(W, eps), tie_embeddings=False,
                         max_positions=1 << 20, embed_name="embed", final_norm_prefix="final.norm", head_name="head",
                         embed_scale=self.embedding_scale, embed_position=SinusoidSpec(W, SINUSOID_BASE),
                         logit_cap=self.logit_softcap or None,
                         tables=((LOOP_TABLE, (self.loop_times, W)),) if self.loop_given else ())


def _freeze(x):
    if isinstance(x, dict):
        return tuple((k, _freeze(v)) for k, v in x.items())
    if isinstance(x, list):
        return ("__list__",) + tuple(_freeze(v) for v in x)
    return x


def _thaw(x):
    if isinstance(x, tuple) and x and x[0] == "__list__":
        return [_thaw(v) for v in x[1:]]
    if isinstance(x, tuple):
        return {k: _thaw(v) for k, v in x}
    return copy.copy(x)
