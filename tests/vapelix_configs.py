"""Small Vapelix configurations for the tests, their random weights and model folders."""

from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_vapelix as pv


def _rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def _mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
            "kv_rank": kv_rank, "scale": scale, "rot": _rot(base, rot_dim, scaling)}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# odd sizes (nothing a multiple of 4), every kind of feed-forward, a loop of two layers run three
# times, layers of different head counts
VAP_A = {
    "architecture": "Vapelix", "vocab": 61, "width": 42, "norm": {"eps": 1e-5},
    "token_side": {"dim": 5},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer(_mixer(3, 6, 2, 5, 9, 7, 0.4, 100.0), _moe(5, 2, 11)),
        _layer(_mixer(2, 10, 6, 3, 14, 18, 0.3, 10000.0, (4.0, 64, 8.0, 1.0)), _dense(30)),
        _layer(_mixer(5, 3, 4, 7, 6, 5, 0.5, 500.0, (2.0, 32, 4.0, 2.0)), None),
        _layer(_mixer(3, 6, 2, 5, 9, 7, 0.4, 100.0), _moe(3, 1, 8)),
    ],
}

# sizes of whole 16-byte rows, more than 8 heads (single tokens then take the kernels with work
# items), no side input, no loop, every token through all experts of one layer
VAP_B = {
    "architecture": "Vapelix", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mixer(12, 16, 8, 16, 24, 24, 0.2, 50000.0, (8.0, 128, 16.0, 1.0)), _moe(4, 4, 16)),
        _layer(_mixer(12, 16, 8, 16, 24, 24, 0.2, 50000.0, (8.0, 128, 16.0, 1.0)), _dense(96)),
        _layer(_mixer(4, 8, 8, 32, 16, 40, 0.25, 1000.0), _moe(9, 3, 24)),
    ],
}

# the loop covers the whole model and starts at layer 0; up to 8 heads (the kernel for single
# tokens); a rotated part as large as the plain one; one expert out of two
VAP_C = {
    "architecture": "Vapelix", "vocab": 128, "width": 48, "norm": {"eps": 1e-6},
    "token_side": {"dim": 8},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _layer(_mixer(8, 8, 8, 8, 16, 24, 0.3, 1000000.0, (16.0, 48, 32.0, 1.0)), _moe(2, 1, 32)),
        _layer(_mixer(4, 16, 4, 12, 32, 12, 0.22, 10000.0), _dense(64)),
    ],
}

# wide: a prompt of a thousand tokens has so many rows that attention takes tiles of 64 rows and
# the products a thousand rows and more; a latent beyond 256 features with its rotated part
VAP_WIDE = {
    "architecture": "Vapelix", "vocab": 300, "width": 256, "norm": {"eps": 1e-6},
    "token_side": {"dim": 16},
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        _layer(_mixer(12, 32, 32, 48, 96, 128, 0.12, 1000000.0, (8.0, 256, 32.0, 1.0)),
               _moe(8, 2, 128)),
        _layer(_mixer(6, 64, 64, 32, 64, 256, 0.1, 10000.0), _dense(512)),
    ],
}

# cached rows of 64 and of 128 features (in bfloat16 their prompt portions take the tcgen05
# attention kernel), layers that differ in every size, a loop over the last two layers
VAP_D = {
    "architecture": "Vapelix", "vocab": 200, "width": 96, "norm": {"eps": 1e-6},
    "token_side": {"dim": 12},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(_mixer(6, 24, 16, 20, 32, 48, 0.2, 10000.0, (8.0, 64, 32.0, 1.0)), _moe(6, 2, 40)),
        _layer(_mixer(4, 32, 32, 16, 24, 96, 0.15, 1000000.0, (4.0, 128, 16.0, 2.0)), _dense(128)),
        _layer(_mixer(10, 16, 16, 24, 40, 48, 0.2, 500.0), _moe(8, 3, 32)),
    ],
}

ALL = {"vap_a": VAP_A, "vap_b": VAP_B, "vap_c": VAP_C, "vap_wide": VAP_WIDE, "vap_d": VAP_D}
SEEDS = {"vap_a": 21, "vap_b": 22, "vap_c": 23, "vap_wide": 24, "vap_d": 25}
PAGES = {"vap_a": 16, "vap_b": 8, "vap_c": 4, "vap_wide": 16, "vap_d": 16}


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
        weights = pv.random_weights(config, SEEDS[name], spread=1.5)
    return write_folder(config, os.path.join(root, name), weights), weights


def tokens(name: str, length: int, index: int = 0) -> list[int]:
    rng = np.random.default_rng(100 * SEEDS[name] + 7 * index + length)
    return [int(t) for t in rng.integers(0, ALL[name]["vocab"], size=length)]


class RoutingTap:
    """While it is open, notes which experts the engine's router kernel chose for every token, by
    request and layer run.  In bfloat16 the engine's router sees slightly different inputs than
    the plain implementation's, and two nearly tied logits may fall the other way; the plain
    implementation is then run with the engine's choice (``routing``) and tells how far that
    choice is from its own (``plain_vapelix.routed_feed_forward``).  Steps that are replayed as
    CUDA graphs do not pass here."""

    def __init__(self, runner, config: dict) -> None:
        self.runner = runner
        self.runs = [run for run, (layer, _) in enumerate(pv.run_order(config))
                     if (config["layers"][layer].get("mlp") or {}).get("kind") == "moe"]
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
            assert len(calls) == len(self.runs), "one router call for every routed layer run"
            at = 0
            for entry in entries:
                n = len(entry.tokens)
                for run, chosen in zip(self.runs, calls):
                    self.parts.setdefault(entry.request_id, {}).setdefault(run, []).append(
                        chosen[at: at + n].cpu())
                at += n
            return out

        lk.experts_route, self.runner.step = route, step
        return self

    def __exit__(self, *exc):
        self._module.experts_route = self._route
        del self.runner.step
        return False

    def routing(self, request_id: str) -> dict:
        return {run: torch.cat(parts) for run, parts in self.parts.get(request_id, {}).items()}
