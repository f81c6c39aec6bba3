"""A plain, slow implementation of the Bizetar decoder, one function per mechanism, whole sequences
only, in float64 (or float32) on the CPU.  It shares no code with the engine: the engine's parts
and kernels are compared with it.

``act`` (None or torch.bfloat16) models the engine's bfloat16 mode: the results of matrix products
are rounded to it (``rnd``); the residual stream, scores, softmax weights, angles, router scores
and norm statistics are not.

Notation: T tokens, width D.  A weight matrix is stored [out, in]; ``lin`` applies it.  ``w`` maps
tensor names to tensors, ``config`` is the parsed config.json.
"""

from __future__ import annotations

import math

import torch


def rnd(x: torch.Tensor, act) -> torch.Tensor:
    return x if act is None else x.to(act).to(x.dtype)


def lin(x: torch.Tensor, weight: torch.Tensor, act=None, bias=None) -> torch.Tensor:
    y = x @ weight.to(x.dtype).t()
    if bias is not None:
        y = rnd(y, act) + bias.to(x.dtype)
    return rnd(y, act)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight.to(x.dtype)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


# ----------------------------------------------------------------------------- rotation
def stretched_frequencies(base: float, dims: int, scaling=None):
    """(f [dims / 2], magnitude).  f_i = base^(-2i / dims).  ``scaling`` {factor, original, fast,
    slow} stretches the slow frequencies: with d(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and the ramp
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- f_i / factor * r_i + f_i (1 - r_i);
    cosines and sines are multiplied by magnitude = 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / max(dims, 1))
    if scaling is None:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def d(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_adjacent(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor,
                    magnitude: float = 1.0) -> torch.Tensor:
    """x [T, heads, d]: features 2i and 2i + 1 (i < len(freq)) are a pair (u, v) that becomes
    (u cos a - v sin a, v cos a + u sin a) with a = p f_i, cosine and sine times ``magnitude``;
    features from 2 len(freq) on pass."""
    n = freq.shape[0]
    if n == 0:
        return x
    angle = positions.to(x.dtype)[:, None, None] * freq.to(x.dtype)[None, None, :]
    c, s = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    u, v = x[..., 0: 2 * n: 2], x[..., 1: 2 * n: 2]
    out = x.clone()
    out[..., 0: 2 * n: 2] = u * c - v * s
    out[..., 1: 2 * n: 2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- pieces of a mixer
def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] u_(t - K + 1 + j), zeros before the start."""
    t, k = u.shape[0], taps.shape[1]
    padded = torch.cat((u.new_zeros(k - 1, u.shape[1]), u), dim=0)
    y = torch.zeros_like(u)
    for j in range(k):
        y = y + taps.to(u.dtype)[None, :, j] * padded[j: j + t]
    return y


def head_slopes(heads: int) -> torch.Tensor:
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return 2.0 ** (-8.0 * h / heads)


def sink_attention(q, k, v, scale, sink, slopes=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv].  Causal; head h reads key/value head
    h // (H / G); score = q . k * scale - slope_h (i - j); the softmax's denominator also holds
    exp(sink_h)."""
    t, heads = q.shape[0], q.shape[1]
    group = heads // k.shape[1]
    pos = torch.arange(t)
    dist = (pos[:, None] - pos[None, :]).to(q.dtype)
    seen = pos[None, :] <= pos[:, None]
    out = q.new_zeros(t, heads, v.shape[2])
    for h in range(heads):
        s = (q[:, h] @ k[:, h // group].t()) * scale
        if slopes is not None:
            s = s - slopes[h].to(q.dtype) * dist
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(dim=1, keepdim=True).values, sink[h].to(q.dtype))
        e = torch.exp(s - top)
        p = e / (e.sum(dim=1, keepdim=True) + torch.exp(sink[h].to(q.dtype) - top))
        out[:, h] = p @ v[:, h // group]
    return out


def mix_values(v, lam, v_first):
    """v <- (1 - lambda) v + lambda v_first; ``v_first`` None: this layer is the one that gives."""
    if v_first is None:
        return v
    lam = lam.to(v.dtype)
    return (1.0 - lam) * v + lam * v_first.reshape(v.shape)       # number by number


# ----------------------------------------------------------------------------- mixers
def attention(h, w, p, m, eps, v_first, act=None):
    """The mixer without rotation: q and k normed over their whole projections, the query grown
    with its position, a distance bias per head, a sink, mixed values, one gate a head.
    Returns (output [T, D], the values as cached [T, G, dv])."""
    t = h.shape[0]
    heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    q = rms_norm(lin(h, w[p + "q"], act), w[p + "q.norm"], eps)
    k = rms_norm(lin(h, w[p + "k"], act), w[p + "k.norm"], eps)
    v = lin(h, w[p + "v"], act).view(t, groups, dv)
    if m.get("q_temp"):
        every, coef = m["q_temp"]["every"], m["q_temp"]["coef"]
        steps = torch.div(pos + 1, every, rounding_mode="floor").to(h.dtype)
        q = q * (1.0 + coef * torch.log(steps + 1.0))[:, None]
    q, k = rnd(q, act).view(t, heads, dk), rnd(k, act).view(t, groups, dk)
    if m.get("v_mix"):
        v = rnd(mix_values(v, w[p + "vmix"], v_first), act)
    o = sink_attention(q, k, v, m["scale"], w[p + "sink"], head_slopes(heads))
    gate = sigmoid(lin(h, w[p + "g"], act))                       # [T, H]
    o = rnd(o * gate[:, :, None], act).reshape(t, heads * dv)
    return lin(o, w[p + "o"], act), v


def attention_2(h, w, p, m, eps, v_first, act=None):
    """The mixer with biases, a short convolution over time on q, k and v, norms per head, rotation
    of adjacent pairs with stretched frequencies, a sink, mixed values, a gate per feature."""
    t = h.shape[0]
    heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(t)
    q = lin(h, w[p + "q"], act, w[p + "q.b"])
    k = lin(h, w[p + "k"], act, w[p + "k.b"])
    v = lin(h, w[p + "v"], act, w[p + "v.b"])
    if m.get("conv"):
        q, k, v = (causal_conv(x, w[p + n + ".conv"]) for x, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_norm(q.view(t, heads, dk), w[p + "q.norm"], eps)
    k = rms_norm(k.view(t, groups, dk), w[p + "k.norm"], eps)
    v = v.view(t, groups, dv)
    rot = m.get("rot")
    if rot:
        freq, magnitude = stretched_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q = rotate_adjacent(q, pos, freq, magnitude)
        k = rotate_adjacent(k, pos, freq, magnitude)
    q, k = rnd(q, act), rnd(k, act)
    if m.get("v_mix"):
        v = mix_values(v, w[p + "vmix"], v_first)
    v = rnd(v, act)
    o = sink_attention(q, k, v, m["scale"], w[p + "sink"])
    gate = sigmoid(lin(h, w[p + "g"], act))                       # [T, H dv]
    o = rnd(o.reshape(t, heads * dv) * gate, act)
    return lin(o, w[p + "o"], act), v


# ----------------------------------------------------------------------------- feed-forwards
def poly_norm(z, coefficients, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N dividing a row by its root mean square."""
    a, b, c, e = (x.to(z.dtype) for x in coefficients)
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def dense_feed_forward(h, w, p, eps, act=None):
    z = lin(h, w[p + "up"], act)
    return lin(rnd(poly_norm(z, w[p + "act"], eps), act), w[p + "down"], act)


def route(h, w, p, top):
    """(chosen [T, top], their weights): scores are the softmax over all router outputs; the choice
    goes by score + correction, the weights are the scores themselves."""
    z = h @ w[p + "router"].to(h.dtype).t()
    s = torch.softmax(z, dim=-1)
    chosen = torch.topk(s + w[p + "correction"].to(h.dtype), top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def routed_feed_forward(h, w, p, router, act=None, chosen=None):
    """Experts e < experts are gated layers down(silu(gate h) * up h); the router's last
    ``identity`` outputs stand for experts that hand their input on."""
    experts, top = router["experts"], router["top"]
    picked, weight = route(h, w, p, top)
    if chosen is not None:                       # the engine's choice, where two scores nearly tie
        z = torch.softmax(h @ w[p + "router"].to(h.dtype).t(), dim=-1)
        picked, weight = chosen, torch.gather(z, 1, chosen)
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for e, a in zip(picked[n].tolist(), weight[n]):
            if e >= experts:
                out[n] += a * h[n]
                continue
            x = h[n: n + 1]
            gate = lin(x, w[f"{p}e{e}.gate"], act)
            inner = rnd(gate * sigmoid(gate) * lin(x, w[f"{p}e{e}.up"], act), act)
            out[n] += a * lin(inner, w[f"{p}e{e}.down"], act)[0]
    return out


# ----------------------------------------------------------------------------- the model
def layer(x, w, config, index, v_first, act=None, chosen=None):
    """x <- x + norm1(gate1 * mixer(x)); x <- x + norm2(gate2 * ff(x)); both sublayers read x
    itself, the gates are sigmoid(W x + b) of the same x.  Returns (x, v_first)."""
    entry, eps, p = config["layers"][index], config["norm"]["eps"], f"l{index}."
    m = entry["mixer"]
    h = rnd(x, act)
    mixer = attention if entry["type"] == "attention" else attention_2
    first = v_first if m.get("v_mix") else None
    y, v = mixer(h, w, p + "mix.", m, eps, first, act)
    if m.get("v_mix") and v_first is None:
        v_first = v
    y = y * sigmoid(lin(h, w[p + "rg1"], act, w[p + "rg1.b"]))
    x = x + rms_norm(y, w[p + "norm1"], eps)
    mlp = entry.get("mlp")
    if mlp is not None:
        h = rnd(x, act)
        if mlp["kind"] == "dense":
            y = dense_feed_forward(h, w, p + "mlp.", eps, act)
        else:
            y = routed_feed_forward(h, w, p + "mlp.", mlp["router"], act, chosen)
        y = y * sigmoid(lin(h, w[p + "rg2"], act, w[p + "rg2.b"]))
        x = x + rms_norm(y, w[p + "norm2"], eps)
    return x, v_first


def forward(tokens, w, config, act=None, dtype=torch.float64, trace=None, routing=None):
    """Logits [T, vocab].  ``trace``: a list that receives the stream after every layer (after the
    average over the depth).  ``routing``: {layer: chosen [T, top]} to force the experts."""
    eps = config["norm"]["eps"]
    if act is not None:
        w = {k: (v.to(act) if v.is_floating_point() and v.dim() >= 2 else v) for k, v in w.items()}
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    x = rms_norm(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], eps)
    outputs, v_first = [x], None
    for i in range(len(config["layers"])):
        y, v_first = layer(x, w, config, i, v_first, act,
                           None if routing is None else routing.get(i))
        outputs.append(y)
        mix = w[f"l{i}.dwa"]
        x = sum(mix[j] * outputs[j] for j in range(i + 2))
        if trace is not None:
            trace.append(x)
    x = rms_norm(x, w["final.norm"], eps)
    return lin(rnd(x, act), w["head"]).to(dtype)


# ----------------------------------------------------------------------------- random models
def tensor_shapes(config) -> dict[str, tuple[int, ...]]:
    d, v = config["width"], config["vocab"]
    out: dict[str, tuple[int, ...]] = {"embed": (v, d), "embed.norm": (d,), "final.norm": (d,),
                                       "head": (v, d)}
    for i, entry in enumerate(config["layers"]):
        m, p = entry["mixer"], f"l{i}.mix."
        heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        second = entry["type"] == "attention_2"
        out.update({p + "q": (heads * dk, d), p + "k": (groups * dk, d), p + "v": (groups * dv, d),
                    p + "sink": (heads,), p + "o": (d, heads * dv),
                    p + "g": ((heads * dv if second else heads), d),
                    p + "q.norm": ((dk,) if second else (heads * dk,)),
                    p + "k.norm": ((dk,) if second else (groups * dk,))})
        if m.get("v_mix"):
            out[p + "vmix"] = ()
        if second:
            out.update({p + "q.b": (heads * dk,), p + "k.b": (groups * dk,),
                        p + "v.b": (groups * dv,)})
            if m.get("conv"):
                out.update({p + "q.conv": (heads * dk, m["conv"]),
                            p + "k.conv": (groups * dk, m["conv"]),
                            p + "v.conv": (groups * dv, m["conv"])})
        q = f"l{i}."
        out.update({q + "norm1": (d,), q + "rg1": (d, d), q + "rg1.b": (d,), q + "dwa": (i + 2,)})
        mlp = entry.get("mlp")
        if mlp is None:
            continue
        out.update({q + "norm2": (d,), q + "rg2": (d, d), q + "rg2.b": (d,)})
        if mlp["kind"] == "dense":
            out.update({q + "mlp.up": (mlp["ff"], d), q + "mlp.down": (d, mlp["ff"]),
                        q + "mlp.act": (4,)})
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            total = r["experts"] + r.get("identity", 0)
            out.update({q + "mlp.router": (total, d), q + "mlp.correction": (total,)})
            for e in range(r["experts"]):
                out.update({f"{q}mlp.e{e}.gate": (ff, d), f"{q}mlp.e{e}.up": (ff, d),
                            f"{q}mlp.e{e}.down": (d, ff)})
    return out


def random_weights(config, seed: int, spread: float = 1.0) -> dict[str, torch.Tensor]:
    """bfloat16-representable random weights: matrices N(0, spread / sqrt(in)), norm weights near
    1, biases, sinks and corrections of a visible size, depth weights that sum to about 1."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2") or name in ("embed.norm", "final.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "vmix":
            t = torch.rand(shape, generator=g) * 0.6 + 0.2
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last == "dwa":
            t = torch.full(shape, 1.0 / shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.tensor([0.8, 0.5, 0.3, 0.1]) + 0.1 * torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.05 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (spread / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
