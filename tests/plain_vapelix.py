"""A plain, slow implementation of the Vapelix decoder, one function per mechanism, whole sequences
only, in float64 (or float32) on the CPU.  It shares no code with the engine: the engine's parts
and kernels are compared with it.

``act`` (None or torch.bfloat16) models the engine's bfloat16 mode: the results of matrix products
and the norms' outputs are rounded to it (``rnd``); the residual stream, scores, softmax weights,
angles, router logits and norm statistics are not.

Notation: T tokens, width D.  A weight matrix is stored [out, in]; ``lin`` applies it.  ``w`` maps
tensor names to tensors, ``config`` is the parsed config.json.
"""

from __future__ import annotations

import math

import torch


def rnd(x: torch.Tensor, act) -> torch.Tensor:
    return x if act is None else x.to(act).to(x.dtype)


def lin(x: torch.Tensor, weight: torch.Tensor, act=None) -> torch.Tensor:
    return rnd(x @ weight.to(x.dtype).t(), act)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, act=None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return rnd(x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype), act)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


# ----------------------------------------------------------------------------- rotation
def stretched_frequencies(base: float, dims: int, scaling=None):
    """(f [dims / 2], magnitude).  f_i = base^(-2i / dims).  ``scaling`` {factor, original, fast,
    slow} stretches the slow frequencies: with d(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and the ramp
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- f_i / factor * r_i + f_i (1 - r_i);
    cosines and sines are multiplied by magnitude = 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling is None:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def d(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, magnitude: float = 1.0):
    """x [T, ..., d] with d = 2 len(freq): feature i is paired with feature i + d / 2 and the pair
    (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i, with cosine and
    sine multiplied by ``magnitude``."""
    half = freq.shape[0]
    angle = positions.to(x.dtype)[:, None] * freq.to(x.dtype)[None, :]
    angle = angle.reshape(x.shape[0], *([1] * (x.dim() - 2)), half)
    c, s = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    u, v = x[..., :half], x[..., half: 2 * half]
    return torch.cat((u * c - v * s, v * c + u * s), dim=-1)


# ----------------------------------------------------------------------------- mixer
def latent_attention(h, w, prefix, m, eps, positions=None, act=None):
    """Attention whose keys and values are read from a small latent per token.

        cq = rms_norm(W_dq h) ; q = W_uq cq, per head [dim plain | rot_dim rotated]
        [c | kr] = W_dkv h ; c = rms_norm(c) (kv_rank) ; kr rotated (rot_dim), one for all heads
        k_h = W_uk c (dim per head) ; v_h = W_uv c (vdim per head)
        score = (q_plain . k_h + q_rot . kr) * scale ; causal softmax ; sum of v_h
        out = W_o (heads * sigmoid(W_g h))
    """
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T) if positions is None else positions
    cq = rms_norm(lin(h, w[prefix + "dq"], act), w[prefix + "dq.norm"], eps, act)
    q = lin(cq, w[prefix + "uq"], act).reshape(T, H, dim + rot_dim)
    kv = lin(h, w[prefix + "dkv"], act)
    c = rms_norm(kv[:, :rank], w[prefix + "dkv.norm"], eps, act)
    rot = m["rot"]
    freq, magnitude = stretched_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
    q_rot = rotate(q[..., dim:], positions, freq, magnitude)
    k_rot = rotate(kv[:, rank:], positions, freq, magnitude)
    k = lin(c, w[prefix + "uk"], act).reshape(T, H, dim)
    v = lin(c, w[prefix + "uv"], act).reshape(T, H, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :dim], k)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    seen = positions[:, None] >= positions[None, :]
    scores = scores.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    heads = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * vdim)
    gate = torch.sigmoid(lin(h, w[prefix + "g"], act))
    return lin(rnd(heads * gate, act), w[prefix + "o"], act)


# ----------------------------------------------------------------------------- feed-forwards
def gated_feed_forward(h, w, prefix, act=None):
    """W_down (gelu_tanh(W_gate h) * (W_up h))."""
    inner = rnd(gelu_tanh(lin(h, w[prefix + "gate"], act)) * lin(h, w[prefix + "up"], act), act)
    return lin(inner, w[prefix + "down"], act)


def route(h, w, prefix, top):
    """(chosen experts [T, top], their weights [T, top]): the ``top`` largest router logits
    W_router h + b, and the softmax over those logits alone."""
    z = h @ w[prefix + "router"].to(h.dtype).t() + w[prefix + "router.b"].to(h.dtype)
    best, chosen = torch.topk(z, top, dim=-1)
    return chosen, torch.softmax(best, dim=-1)


def routed_feed_forward(h, w, prefix, experts, top, act=None, chosen=None, slack=None):
    """sum over the chosen experts e of weight_e * W_down_e gelu_erf(W_up_e h).

    ``chosen`` [T, top] takes the place of the router's choice (an implementation in bfloat16 sees
    slightly different logits, and where two are nearly tied it may pick the other): the weights
    are then the softmax over the logits of those experts, and ``slack`` (a list) receives by how
    much the smallest of them lies below the ``top``-th largest logit, as a share of the logits'
    spread, which is 0 where the choice is the router's."""
    if chosen is None:
        chosen, weights = route(h, w, prefix, top)
    else:
        z = h @ w[prefix + "router"].to(h.dtype).t() + w[prefix + "router.b"].to(h.dtype)
        mine = torch.gather(z, 1, chosen.long())
        assert all(len(set(row)) == top for row in chosen.tolist()), "an expert chosen twice"
        weights = torch.softmax(mine, dim=-1)
        if slack is not None:
            kth = torch.topk(z, top, dim=-1).values[:, -1]
            spread = (z.max(dim=-1).values - z.min(dim=-1).values).clamp_min(1e-9)
            slack.append(float(((kth - mine.min(dim=-1).values) / spread).max()))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            inner = rnd(gelu_erf(lin(h[t: t + 1], w[f"{prefix}e{e}.up"], act)), act)
            out[t] += weight * lin(inner, w[f"{prefix}e{e}.down"], act)[0]
    return out


def token_side(x, tokens, w, prefix, index, dim, eps, act=None):
    """What a token's own table row adds after a layer: with e = side.embed[token][index * dim :
    (index + 1) * dim], y = W_proj (gelu_tanh(W_gate x) * e) and x + rms_norm(y) * side.norm."""
    e = w["side.embed"][tokens][:, index * dim: (index + 1) * dim].to(x.dtype)
    g = rnd(gelu_tanh(lin(rnd(x, act), w[prefix + "gate"], act)) * e, act)
    y = lin(g, w[prefix + "proj"], act)
    return rms_norm(y, w[prefix + "norm"], eps)


# ----------------------------------------------------------------------------- the model
def run_order(config) -> list[tuple[int, bool]]:
    """(layer, whether the embedding output is added before it) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for t in range(times):
        order += [(i, t > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def layer(x, tokens, w, config, index, act=None, chosen=None, slack=None):
    """x + mixer(norm1 x) + ff(norm2 x), both branches of the same x; then the token's side input.
    ``chosen``, ``slack``: see ``routed_feed_forward``."""
    entry, eps, prefix = config["layers"][index], config["norm"]["eps"], f"l{index}."
    h = rms_norm(x, w[prefix + "norm1"], eps, act)
    branch = latent_attention(h, w, prefix + "mix.", entry["mixer"], eps, act=act)
    mlp = entry.get("mlp")
    if mlp is not None:
        h2 = rms_norm(x, w[prefix + "norm2"], eps, act)
        if mlp["kind"] == "dense":
            branch = branch + gated_feed_forward(h2, w, prefix + "mlp.", act)
        else:
            branch = branch + routed_feed_forward(h2, w, prefix + "mlp.", mlp["router"]["experts"],
                                                  mlp["router"]["top"], act, chosen, slack)
    x = x + branch
    side = config.get("token_side")
    if side:
        x = x + token_side(x, tokens, w, prefix + "side.", index, side["dim"], eps, act)
    return x


def forward(tokens, w, config, act=None, dtype=torch.float64, trace=None, routing=None,
            slack=None):
    """Logits [T, vocab] of one whole sequence.  ``trace``: a list that receives the residual
    stream after every layer run.  ``routing``: layer run -> chosen experts [T, top], in place of
    the router's choice in that run (see ``routed_feed_forward``, also for ``slack``)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    first = w["embed"][tokens]
    x = first.clone()
    for run, (index, add_first) in enumerate(run_order(config)):
        if add_first:
            x = x + first
        x = layer(x, tokens, w, config, index, act, None if routing is None else routing.get(run),
                  slack)
        if trace is not None:
            trace.append(x.clone())
    last = rms_norm(x, w["final.norm"], config["norm"]["eps"], act)
    return last @ w["embed"].t()


# ----------------------------------------------------------------------------- weights
def tensor_shapes(config) -> dict[str, tuple[int, ...]]:
    D, V = config["width"], config["vocab"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (V, D), "final.norm": (D,)}
    side = config.get("token_side")
    if side:
        shapes["side.embed"] = (V, len(config["layers"]) * side["dim"])
    for i, entry in enumerate(config["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        H, per = m["heads"], m["dim"] + m["rot_dim"]
        shapes.update({
            p + "norm1": (D,), p + "mix.dq": (m["q_rank"], D), p + "mix.dq.norm": (m["q_rank"],),
            p + "mix.uq": (H * per, m["q_rank"]), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], D),
            p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
            p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.g": (H * m["vdim"], D),
            p + "mix.o": (D, H * m["vdim"])})
        mlp = entry.get("mlp")
        if mlp is not None:
            shapes[p + "norm2"] = (D,)
            if mlp["kind"] == "dense":
                shapes.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D),
                               p + "mlp.down": (D, mlp["ff"])})
            else:
                E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
                shapes.update({p + "mlp.router": (E, D), p + "mlp.router.b": (E,)})
                for e in range(E):
                    shapes[f"{p}mlp.e{e}.up"] = (F, D)
                    shapes[f"{p}mlp.e{e}.down"] = (D, F)
        if side:
            shapes.update({p + "side.gate": (side["dim"], D), p + "side.proj": (D, side["dim"]),
                           p + "side.norm": (D,)})
    return shapes


def random_weights(config, seed: int, spread: float = 1.0) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, spread^2 / fan-in), norm weights near 1, router biases and
    table rows of order 1."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("router.b"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * spread / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
