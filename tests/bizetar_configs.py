"""Small Bizetar configurations for the tests, their random weights and model folders."""

from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_bizetar as pb


def first(heads, kv_heads, dim, vdim, scale, v_mix=True, q_temp=None):
    """A mixer of type ``attention``."""
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
           "v_mix": v_mix}
    if q_temp is not None:
        out["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return out


def second(heads, kv_heads, dim, vdim, scale, v_mix=True, conv=None, rot=None):
    """A mixer of type ``attention_2``; rot = (base, dims) or (base, dims, (factor, original, fast,
    slow))."""
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
           "v_mix": v_mix}
    if conv is not None:
        out["conv"] = conv
    if rot is not None:
        out["rot"] = {"base": rot[0], "dims": rot[1]}
        if len(rot) > 2:
            out["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "identity": identity}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# odd sizes (nothing a multiple of 4), the mixer without rotation first (it gives the values), two
# kv heads, a layer without a feed-forward, a layer outside the mixing of values, 2 and 4 taps
BIZ_A = {
    "architecture": "Bizetar", "vocab": 61, "width": 42, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", first(6, 2, 5, 3, 0.4, q_temp=(0.7, 4)), moe(5, 2, 11, identity=2)),
        layer("attention_2", second(6, 2, 10, 3, 0.3, conv=2, rot=(100.0, 6, (4.0, 16, 8.0, 1.0))),
              dense(30)),
        layer("attention_2", second(3, 1, 6, 7, 0.5, v_mix=False, conv=4, rot=(500.0, 6)), None),
        layer("attention", first(4, 2, 7, 3, 0.35), moe(3, 1, 8)),
    ],
}

# rows of whole 16-byte pieces; ten query heads a kv head (single tokens then go through the
# kernels with work items); a layer outside the mixing of values between the giver and a taker; every router output chosen; no convolution in one layer, one tap
# in another; a query that grows at every position
BIZ_B = {
    "architecture": "Bizetar", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention_2", second(20, 2, 16, 8, 0.2, rot=(70000.0, 8, (8.0, 32, 16.0, 1.0))),
              moe(4, 6, 16, identity=2)),
        layer("attention", first(8, 4, 16, 8, 0.25, v_mix=False, q_temp=(0.3, 1)), dense(96)),
        layer("attention_2", second(4, 2, 32, 8, 0.15, conv=1, rot=(1000.0, 32)),
              moe(9, 3, 24, identity=1)),
    ],
}

# up to 8 heads a kv head and whole pieces (the kernel for single tokens), five taps, rotation of
# nothing, only the second layer and the last mix values, only identity outputs beside one expert
BIZ_C = {
    "architecture": "Bizetar", "vocab": 128, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention_2", second(4, 4, 8, 8, 0.3, v_mix=False, conv=5, rot=(10000.0, 0)),
              moe(1, 2, 32, identity=3)),
        layer("attention_2", second(8, 1, 16, 12, 0.22, conv=3,
                                    rot=(1000000.0, 16, (16.0, 48, 32.0, 1.0))), dense(64)),
        layer("attention", first(8, 1, 8, 12, 0.3, q_temp=(1.5, 64)), dense(20)),
    ],
}

# wide: a prompt of a thousand tokens has so many rows that attention takes tiles of 64 rows and
# the products a thousand rows and more; more than 128 pairs an expert (the tensor-core experts)
BIZ_WIDE = {
    "architecture": "Bizetar", "vocab": 300, "width": 256, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention_2", second(12, 2, 64, 40, 0.12, conv=2,
                                    rot=(40000.0, 48, (6.0, 256, 16.0, 2.0))),
              moe(6, 2, 128, identity=3)),
        layer("attention", first(8, 2, 56, 40, 0.14, q_temp=(0.4, 96)), dense(512)),
    ],
}

ALL = {"biz_a": BIZ_A, "biz_b": BIZ_B, "biz_c": BIZ_C, "biz_wide": BIZ_WIDE}
SEEDS = {"biz_a": 31, "biz_b": 32, "biz_c": 33, "biz_wide": 34}
PAGES = {"biz_a": 16, "biz_b": 8, "biz_c": 4, "biz_wide": 16}


def write_folder(config: dict, folder: str, weights: dict) -> str:
    from distengine_b200.weights import save_tensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config, handle)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return folder


def make_folder(name: str, root: str, weights: "dict | None" = None) -> "tuple[str, dict]":
    """Write the model folder (bfloat16 tensors); returns (folder, weights)."""
    config = ALL[name]
    if weights is None:
        weights = pb.random_weights(config, SEEDS[name], spread=1.5)
    return write_folder(config, os.path.join(root, name), weights), weights


def tokens(name: str, length: int, index: int = 0) -> list[int]:
    rng = np.random.default_rng(100 * SEEDS[name] + 7 * index + length)
    return [int(t) for t in rng.integers(0, ALL[name]["vocab"], size=length)]


class RoutingTap:
    """While it is open, notes which router outputs the engine's router kernel chose for every
    token, by request and layer.  In bfloat16 the engine's router sees slightly different inputs
    than the plain implementation's, and two nearly tied scores may fall the other way; the plain
    implementation is then run with the engine's choice (``routing``).  Steps that are replayed as
    CUDA graphs do not pass here."""

    def __init__(self, runner, config: dict) -> None:
        self.runner = runner
        self.layers = [i for i, entry in enumerate(config["layers"])
                       if (entry.get("mlp") or {}).get("kind") == "moe"]
        self.parts: dict = {}

    def __enter__(self):
        from distengine_b200.kernels import latent as lk
        self._module, self._route, self._step = lk, lk.experts_route, self.runner.step
        calls: list = []

        def route(h, router, bias, top, chosen, weight, *more):
            self._route(h, router, bias, top, chosen, weight, *more)
            calls.append(chosen.clone())

        def step(entries, extra=None):
            calls.clear()
            out = self._step(entries, extra)
            assert len(calls) == len(self.layers), "one router call for every routed layer"
            at = 0
            for entry in entries:
                n = len(entry.tokens)
                for index, chosen in zip(self.layers, calls):
                    self.parts.setdefault(entry.request_id, {}).setdefault(index, []).append(
                        chosen[at: at + n].cpu().long())
                at += n
            return out

        lk.experts_route, self.runner.step = route, step
        return self

    def __exit__(self, *exc):
        self._module.experts_route = self._route
        del self.runner.step
        return False

    def routing(self, request_id: str) -> dict:
        return {i: torch.cat(parts) for i, parts in self.parts.get(request_id, {}).items()}
