"""Typed configuration of the Bizetar decoder, read from its config.json.

The file names every size and every constant that differs between models of the design:

    {"architecture": "Bizetar", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "attention" | "attention_2", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F},
                         "router": {"experts": E, "top": k, "identity": n}}
                      | null}, ...]}

* Both mixers: ``heads``, ``kv_heads``, ``dim`` (of a query or key head), ``vdim``, ``scale``,
  ``v_mix`` (whether the layer takes part in the mixing of values: the first such layer gives its
  values, the later ones mix theirs with them).
* ``attention``: q and k are normed over their whole projections; no rotation; optional ``q_temp``
  (``coef``, ``every``): the query grows with the logarithm of its position; a distance bias with
  slopes that the design fixes; one output gate a head.
* ``attention_2``: biases on q, k, v; optional ``conv`` (taps of a short causal convolution on
  their channels); norms per head; optional ``rot`` (``base``, ``dims``, optional ``scaling`` with
  ``factor``, ``original``, ``fast``, ``slow``) on adjacent pairs; one output gate a feature.
* Every mixer's softmax has a sink per head.  A layer is x + norm1(g1 * mixer(x)), then
  x + norm2(g2 * mlp(x)) with gates g = sigmoid(W x + b) of the sublayer's own input, and what goes
  on to the next layer is a learned mix of the embedding rows and all layers' results so far.
* ``dense``: down(P(up x)) with a learned cubic of normed powers.  ``moe``: ``experts`` gated
  experts (silu), ``identity`` further router outputs that hand the input on, ``top`` a token; the
  scores are the softmax over all router outputs, the choice goes by score + correction.

Layer i's tensors are named ``l<i>.*``.  A model of this design has no position limit of its own.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Mapping

from .model import (ConfigError, LayerSpec, ModelConfig, PartSpec, positive, require,
                    number as _number, positive_int as _int, section as _section)

NAME = "Bizetar"
MAX_POSITIONS = 1 << 20          # the design names none
KINDS = ("attention", "attention_2")


def _freeze(value):
    if isinstance(value, dict):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    return value


def _flag(m: Mapping[str, Any], key: str, where: str) -> bool:
    value = m.get(key, False)
    if value is None:
        return False
    if not isinstance(value, bool):
        raise ConfigError(f"config.json: '{where}{key}' must be true or false, got {value!r}")
    return value


def _rotation(m: Mapping[str, Any], where: str, dim: int) -> "dict | None":
    if m.get("rot") is None:
        return None
    rot = _section(m, "rot", where)
    dims = rot.get("dims")
    if type(dims) is not int or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: '{where}rot.dims' ({dims!r}) must be an even number from "
                          f"0 to '{where}dim' ({dim})")
    base = _number(rot, "base", where + "rot.")
    if base <= 1.0:
        raise ConfigError(f"config.json: '{where}rot.base' must be above 1")
    scaling = None
    if rot.get("scaling") is not None:
        sc = _section(rot, "scaling", where + "rot.")
        w = where + "rot.scaling."
        scaling = (_number(sc, "factor", w), _number(sc, "original", w), _number(sc, "fast", w),
                   _number(sc, "slow", w))
        if min(scaling) <= 0:
            raise ConfigError(f"config.json: '{where}rot.scaling' needs positive factor, "
                              f"original, fast and slow")
    return {"base": base, "dims": dims, "scaling": scaling}


def _mixer(kind: str, m: Mapping[str, Any], where: str) -> dict:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: '{where}heads' ({heads}) must be a multiple of "
                          f"'{where}kv_heads' ({kv_heads})")
    out = {"heads": heads, "kv_heads": kv_heads, "dim": _int(m, "dim", where),
           "vdim": _int(m, "vdim", where), "scale": _number(m, "scale", where),
           "v_mix": _flag(m, "v_mix", where)}
    if kind == "attention":
        out["q_temp"] = None
        if m.get("q_temp") is not None:
            t = _section(m, "q_temp", where)
            out["q_temp"] = (_number(t, "coef", where + "q_temp."),
                             _int(t, "every", where + "q_temp."))
        allowed = {"q_temp"}
    else:
        taps = m.get("conv")
        if taps is not None and (type(taps) is not int or taps <= 0):
            raise ConfigError(f"config.json: '{where}conv' must be a positive number of taps or "
                              f"null, got {taps!r}")
        out["conv"] = taps or 0
        out["rot"] = _rotation(m, where, out["dim"])
        allowed = {"conv", "rot"}
    # a key of the other form may stand with null or false (nothing of it is there)
    unknown = {k for k in set(m) - allowed - {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix"}
               if m[k] is not None and m[k] is not False}
    if unknown:
        raise ConfigError(f"config.json: '{where}' has keys this design does not know for "
                          f"'{kind}': {sorted(unknown)}")
    return out


def _feed_forward(mlp: Any, where: str) -> "dict | None":
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping):
        raise ConfigError(f"config.json: '{where}mlp' must be an object or null")
    kind = mlp.get("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": _int(mlp, "ff", where + "mlp.")}
    if kind == "moe":
        router = _section(mlp, "router", where + "mlp.")
        experts = _int(router, "experts", where + "mlp.router.")
        top = _int(router, "top", where + "mlp.router.")
        identity = router.get("identity") or 0
        if type(identity) is not int or identity < 0:
            raise ConfigError(f"config.json: '{where}mlp.router.identity' must be a number >= 0")
        if top > experts + identity:
            raise ConfigError(f"config.json: '{where}mlp.router.top' ({top}) is more than the "
                              f"{experts + identity} router outputs")
        return {"kind": "moe", "experts": experts, "top": top, "identity": identity,
                "ff": _int(_section(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")}
    raise ConfigError(f"config.json: '{where}mlp.kind' is {kind!r}; this design has 'dense' and "
                      f"'moe'")


@dataclass(frozen=True)
class BizetarConfig(ModelConfig):
    vocab: int
    model_width: int
    eps: float
    # per layer: (type, the mixer's parsed keys, the feed-forward's parsed keys or None), frozen
    layers: tuple

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_json(data: Mapping[str, Any]) -> "BizetarConfig":
        width = positive("width", require(data, "width", int))
        eps = _number(_section(data, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        entries = data.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a nonempty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            kind = entry.get("type")
            if kind not in KINDS:
                raise ConfigError(f"config.json: '{where}type' is {kind!r}; this design has "
                                  f"{' and '.join(repr(k) for k in KINDS)}")
            mixer = _mixer(kind, _section(entry, "mixer", where), where + "mixer.")
            layers.append((kind, _freeze(mixer), _freeze(_feed_forward(entry.get("mlp"), where))))
        sizes = {dict(m)["kv_heads"] * dict(m)["vdim"] for _, m, _ in layers if dict(m)["v_mix"]}
        if len(sizes) > 1:
            raise ConfigError("config.json: the layers with 'v_mix' must have values of one size "
                              f"(kv_heads * vdim numbers a token), got {sorted(sizes)}")
        return BizetarConfig(architecture=NAME,
                             vocab=positive("vocab", require(data, "vocab", int)),
                             model_width=width, eps=eps, layers=tuple(layers))

    def to_json(self) -> dict[str, Any]:
        layers = []
        for kind, mixer, mlp in self.layers:
            m = dict(mixer)
            out_mixer: dict[str, Any] = {k: m[k] for k in ("heads", "kv_heads", "dim", "vdim",
                                                           "scale", "v_mix")}
            if kind == "attention":
                if m["q_temp"] is not None:
                    out_mixer["q_temp"] = {"coef": m["q_temp"][0], "every": m["q_temp"][1]}
            else:
                if m["conv"]:
                    out_mixer["conv"] = m["conv"]
                if m["rot"] is not None:
                    r = dict(m["rot"])
                    rot: dict[str, Any] = {"base": r["base"], "dims": r["dims"]}
                    if r["scaling"] is not None:
                        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"),
                                                  r["scaling"]))
                    out_mixer["rot"] = rot
            out_mlp = None
            if mlp is not None:
                f = dict(mlp)
                out_mlp = ({"kind": "dense", "ff": f["ff"]} if f["kind"] == "dense" else
                           {"kind": "moe", "expert": {"ff": f["ff"]},
                            "router": {"experts": f["experts"], "top": f["top"],
                                       "identity": f["identity"]}})
            layers.append({"type": kind, "mixer": out_mixer, "mlp": out_mlp})
        out = {"architecture": NAME, "vocab": self.vocab, "width": self.model_width,
               "norm": {"eps": self.eps}, "layers": layers}
        return json.loads(json.dumps(out))

    # ------------------------------------------------------------------ the model as data
    @property
    def width(self) -> int:
        return self.model_width

    @property
    def vocabulary(self) -> int:
        return self.vocab

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    @property
    def tied_output(self) -> bool:
        return False

    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec.of("rmsnorm", width=self.model_width, eps=self.eps, tensor=tensor)

    def embedding_norm(self) -> PartSpec:
        return self._norm("norm")

    def layer_specs(self) -> list[LayerSpec]:
        specs, d = [], self.model_width
        gives = True                 # the first layer that mixes values gives them
        for i, (kind, mixer, mlp) in enumerate(self.layers):
            m, base = dict(mixer), f"l{i}."
            value_mix = None
            if m["v_mix"]:
                value_mix, gives = ("give" if gives else "take"), False
            common = dict(width=d, heads=m["heads"], kv_heads=m["kv_heads"], key_dim=m["dim"],
                          value_dim=m["vdim"], scale=m["scale"], eps=self.eps,
                          value_mix=value_mix)
            if kind == "attention":
                part = PartSpec.of("sink_attention", norm="whole", slopes=True, gate="head",
                                   temperature=m["q_temp"], **common)
            else:
                rot = dict(m["rot"]) if m["rot"] is not None else None
                part = PartSpec.of("sink_attention", biased=True, taps=m["conv"], norm="head",
                                   gate="feature", adjacent=True,
                                   rotary_dim=rot["dims"] if rot else 0,
                                   theta=rot["base"] if rot else 10000.0,
                                   stretch=rot["scaling"] if rot else None, **common)
            feed_forward = None
            if mlp is not None:
                f = dict(mlp)
                if f["kind"] == "dense":
                    feed_forward = PartSpec.of("polynorm_mlp", width=d, inner=f["ff"],
                                               eps=self.eps)
                else:
                    feed_forward = PartSpec.of("routed_experts", width=d, inner=f["ff"],
                                               experts=f["experts"], top=f["top"],
                                               activation="silu", gated=True,
                                               scoring="corrected_scores",
                                               identity=f["identity"], bias_name="correction")
            specs.append(LayerSpec(
                block="sublayer_norm", mixer=part, feed_forward=feed_forward,
                norm=self._norm("norm1"), feed_forward_norm=self._norm("norm2"),
                block_params=(("depth", i + 2), ("gated", True)),
                prefixes=(("mixer", base + "mix."), ("feed_forward", base + "mlp."),
                          ("mixer_norm", base), ("feed_forward_norm", base),
                          ("mixer_gate", base + "rg1"), ("feed_forward_gate", base + "rg2"),
                          ("depth_mix", base))))
        return specs

    def final_norm(self) -> PartSpec:
        return self._norm("norm")

    def unused_tensors(self) -> set[str]:
        """Tensors that a weight file of this design may hold for parts that a layer does not
        have: the mixing weight of a layer outside the mixing of values, and the second
        sublayer's norm and gate of a layer without a feed-forward."""
        names = set()
        for i, (_, mixer, mlp) in enumerate(self.layers):
            if not dict(mixer)["v_mix"]:
                names.add(f"l{i}.mix.vmix")
            if mlp is None:
                names |= {f"l{i}.norm2", f"l{i}.rg2", f"l{i}.rg2.b"}
        return names

    def tensor_names(self) -> dict[str, str]:
        return {"embedding": "embed", "embedding_norm": "embed.", "final_norm": "final.",
                "output": "head"}
