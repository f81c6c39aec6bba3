"""Typed configuration of the Vapelix decoder, read from its config.json.

The file names every size and every constant that differs between models of the design:

    {"architecture": "Vapelix", "vocab": V, "width": D, "norm": {"eps": e},
     "token_side": {"dim": s} (optional),
     "loop": {"start": a, "stop": b, "times": t} (optional),
     "layers": [{"type": "latent_attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}}
                      | null}, ...]}

* ``latent_attention`` mixer: ``heads``, ``dim`` (features of a head's query and key that are not
  rotated), ``rot_dim`` (rotated features; one rotated key part serves all heads), ``vdim``,
  ``q_rank`` and ``kv_rank`` (the sizes of the two latents), ``scale``, and ``rot`` (``base``,
  ``dims`` = ``rot_dim``, optional ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``).
* A layer is x + mixer(norm1 x) + mlp(norm2 x), both branches of the same x, followed (with
  ``token_side``) by what a table row of the token adds.  All norms are RMS norms with a weight.
* ``loop``: layers a .. b-1 run t times in a row with the same weights, every pass with a cache of
  its own; before every pass but the first the embedding rows are added to the stream again.

Layer i's tensors are named ``l<i>.*``; the output matrix is the embedding table.  A model of this
design has no position limit of its own.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Mapping

from .model import (ConfigError, LayerSpec, ModelConfig, PartSpec, PlanEntry, positive, require,
                    number as _number, positive_int as _int, section as _section)

NAME = "Vapelix"
MAX_POSITIONS = 1 << 20          # the design names none; positions are exact in float32 far beyond


def _rotation(m: Mapping[str, Any], where: str, rot_dim: int) -> tuple:
    """(base, scaling or None) of a mixer's ``rot`` section; scaling = (factor, original, fast,
    slow)."""
    rot = _section(m, "rot", where)
    dims = rot.get("dims", rot_dim)
    if type(dims) is not int or dims != rot_dim:
        raise ConfigError(f"config.json: '{where}rot.dims' ({dims!r}) must equal '{where}rot_dim' "
                          f"({rot_dim})")
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
    return base, scaling


def _latent_attention(m: Mapping[str, Any], where: str) -> dict:
    rot_dim = m.get("rot_dim")
    if type(rot_dim) is not int or rot_dim < 0 or rot_dim % 2:
        raise ConfigError(f"config.json: '{where}rot_dim' ({rot_dim!r}) must be an even number "
                          f">= 0")
    base, scaling = (1.0e4, None) if rot_dim == 0 and m.get("rot") is None else \
        _rotation(m, where, rot_dim)
    return {"heads": _int(m, "heads", where), "dim": _int(m, "dim", where), "rot_dim": rot_dim,
            "vdim": _int(m, "vdim", where), "q_rank": _int(m, "q_rank", where),
            "kv_rank": _int(m, "kv_rank", where), "scale": _number(m, "scale", where),
            "base": base, "scaling": scaling}


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
        if top > experts:
            raise ConfigError(f"config.json: '{where}mlp.router.top' ({top}) is more than the "
                              f"{experts} experts")
        return {"kind": "moe", "experts": experts, "top": top,
                "ff": _int(_section(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")}
    raise ConfigError(f"config.json: '{where}mlp.kind' is {kind!r}; this design has 'dense' and "
                      f"'moe'")


def _freeze(value):
    if isinstance(value, dict):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    return value


@dataclass(frozen=True)
class VapelixConfig(ModelConfig):
    vocab: int
    model_width: int
    eps: float
    side_dim: int                    # 0: no per-layer token input
    loop: "tuple[int, int, int] | None"      # (start, stop, times)
    # per layer: (the mixer's parsed keys, the feed-forward's parsed keys or None), frozen
    layers: tuple

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_json(data: Mapping[str, Any]) -> "VapelixConfig":
        width = positive("width", require(data, "width", int))
        eps = _number(_section(data, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        side_dim = 0
        if data.get("token_side") is not None:
            side_dim = _int(_section(data, "token_side", ""), "dim", "token_side.")
        entries = data.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a nonempty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            if entry.get("type") != "latent_attention":
                raise ConfigError(f"config.json: '{where}type' is {entry.get('type')!r}; this "
                                  f"design has 'latent_attention'")
            mixer = _latent_attention(_section(entry, "mixer", where), where + "mixer.")
            layers.append((_freeze(mixer), _freeze(_feed_forward(entry.get("mlp"), where))))
        loop = None
        if data.get("loop") is not None:
            section = _section(data, "loop", "")
            start, stop, times = (section.get(k) for k in ("start", "stop", "times"))
            if (any(type(x) is not int for x in (start, stop, times))
                    or not 0 <= start <= stop <= len(layers) or times < 1):
                raise ConfigError("config.json: 'loop' needs integers 0 <= start <= stop <= the "
                                  "number of layers and times >= 1")
            if start < stop and times > 1:
                loop = (start, stop, times)
        return VapelixConfig(architecture=NAME,
                             vocab=positive("vocab", require(data, "vocab", int)),
                             model_width=width, eps=eps, side_dim=side_dim, loop=loop,
                             layers=tuple(layers))

    def to_json(self) -> dict[str, Any]:
        layers = []
        for mixer, mlp in self.layers:
            m = dict(mixer)
            rot: dict[str, Any] = {"base": m["base"], "dims": m["rot_dim"]}
            if m["scaling"] is not None:
                rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), m["scaling"]))
            out_mixer = {k: m[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank",
                                           "scale")}
            out_mixer["rot"] = rot
            out_mlp = None
            if mlp is not None:
                f = dict(mlp)
                out_mlp = ({"kind": "dense", "ff": f["ff"]} if f["kind"] == "dense" else
                           {"kind": "moe", "expert": {"ff": f["ff"]},
                            "router": {"experts": f["experts"], "top": f["top"]}})
            layers.append({"type": "latent_attention", "mixer": out_mixer, "mlp": out_mlp})
        out: dict[str, Any] = {"architecture": NAME, "vocab": self.vocab,
                               "width": self.model_width, "norm": {"eps": self.eps},
                               "layers": layers}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
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
        return True

    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec.of("rmsnorm", width=self.model_width, eps=self.eps, tensor=tensor)

    def layer_specs(self) -> list[LayerSpec]:
        """A block of two parallel branches per layer: latent attention beside a gated dense
        feed-forward or routed experts, then the token's side input."""
        specs, d = [], self.model_width
        for i, (mixer, mlp) in enumerate(self.layers):
            m, base = dict(mixer), f"l{i}."
            part = PartSpec.of("latent_attention", width=d, heads=m["heads"], key_dim=m["dim"],
                               rotary_dim=m["rot_dim"], value_dim=m["vdim"], q_rank=m["q_rank"],
                               kv_rank=m["kv_rank"], scale=m["scale"], theta=m["base"],
                               scaling=m["scaling"], eps=self.eps)
            feed_forward = None
            if mlp is not None:
                f = dict(mlp)
                if f["kind"] == "dense":
                    feed_forward = PartSpec.of("gated_mlp", width=d, inner=f["ff"],
                                               activation="gelu_tanh",
                                               names=("gate", "up", "down"))
                else:
                    feed_forward = PartSpec.of("routed_experts", width=d, inner=f["ff"],
                                               experts=f["experts"], top=f["top"],
                                               activation="gelu_erf")
            side = None
            if self.side_dim:
                side = PartSpec.of("token_side", width=d, dim=self.side_dim, index=i,
                                   layers=len(self.layers), vocabulary=self.vocab, eps=self.eps,
                                   table="/side.embed")
            specs.append(LayerSpec(
                block="parallel_norms", mixer=part, feed_forward=feed_forward,
                norm=self._norm("norm1"), feed_forward_norm=self._norm("norm2"), side_input=side,
                prefixes=(("mixer", base + "mix."), ("feed_forward", base + "mlp."),
                          ("mixer_norm", base), ("feed_forward_norm", base),
                          ("side_input", base + "side."))))
        return specs

    def plan(self) -> list[PlanEntry]:
        """Layers in order, the looped ones ``times`` times in a row; every pass but the first
        starts with the embedding rows added to the stream."""
        n = len(self.layers)
        if self.loop is None:
            return [PlanEntry(i) for i in range(n)]
        start, stop, times = self.loop
        plan = [PlanEntry(i) for i in range(start)]
        for t in range(times):
            plan += [PlanEntry(i, adds_embedding=(t > 0 and i == start))
                     for i in range(start, stop)]
        return plan + [PlanEntry(i) for i in range(stop, n)]

    def final_norm(self) -> PartSpec:
        return self._norm("norm")

    def tensor_names(self) -> dict[str, str]:
        return {"embedding": "embed", "final_norm": "final.", "output": "embed"}
