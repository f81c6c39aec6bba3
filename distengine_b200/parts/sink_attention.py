"""Grouped-query causal softmax attention over the paged cache whose softmax has a *sink* - a
learned number per head that joins the denominator without a key or a value - with 32-bit scores
and weights, and with a choice of what happens to q, k and v between their projections and the
scores.  Every one of these is a parameter:

    q, k, v = W x (+ b)                             ``biased``
    a causal convolution over time on every channel ``taps`` (K > 0 taps, no bias; the last K - 1
        projected rows of a sequence are kept in its state slot)
    q, k / root mean square * weight                ``norm`` "head" (over a head's features, one
        weight [dk] for all heads) or "whole" (over the whole projection, weights [H dk], [G dk])
    q, k turned by position                         ``rotary_dim`` features of every head, pairs
        (2i, 2i + 1) (``adjacent``) or (i, i + rotary_dim / 2), frequencies theta^(-2i / rotary_dim),
        optionally stretched (``stretch`` = (factor, original, fast, slow): a ramp between two
        wavelengths blends f and f / factor; cosine and sine grow by 0.1 ln(factor) + 1)
    q * (1 + coef ln(floor((p + 1) / every) + 1))   ``temperature`` = (coef, every)
    v <- (1 - lambda) v + lambda v_first            ``value_mix`` "take"; the layer with "give"
        leaves its values of the step's tokens for the layers that take; the mixed v is cached
    score(i, j) = q_i . k_j * scale - slope_h (i - j),  slope_h = 2^(-8 (h + 1) / H)  (``slopes``)
    weights = exp(score) / (sum over j <= i of exp(score) + exp(sink_h))
    out = W_o [heads' results * sigmoid(W_g x)]     ``gate`` "feature" ([H dv] numbers a token) or
        "head" ([H])

The input product stacks [q; k; v; g].  The scores, the weights and the weighted sums of the
values are float32 (``csrc/attention_chunk.cu``); so are the convolution's sums, the norms, the
angles and the mixing of the values.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import recurrent as rk
from ..kernels.attention_plan import build_plan
from .base import PagedKVSpec, StateSpec, compute_matrix, register_mixer
from .context import StepPrep
from .recurrent import ProjectedMixer, stack_segments, vector32

MAX_DIM = 256


def stretched_frequencies(theta: float, dims: int, stretch=None) -> "tuple[torch.Tensor, float]":
    """(float32 [dims / 2] formed in float64, the factor on cosine and sine)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(theta) ** (-2.0 * i / max(dims, 1))
    if stretch is None:
        return f.to(torch.float32), 1.0
    factor, original, fast, slow = (float(x) for x in stretch)

    def place(turns: float) -> float:       # the (fractional) pair whose wavelength fits `turns`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(place(fast)), 0)
    hi = min(math.ceil(place(slow)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


class SinkAttention(ProjectedMixer):
    kind = "sink_attention"

    def __init__(self, width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, eps: float, dtype: torch.dtype, device: torch.device,
                 biased: bool = False, taps: int = 0, norm: "str | None" = None,
                 rotary_dim: int = 0, theta: float = 10000.0, stretch=None,
                 adjacent: bool = True, temperature=None, slopes: bool = False,
                 value_mix: "str | None" = None, gate: "str | None" = None,
                 mix_key: str = "value_mix.first") -> None:
        super().__init__(dtype, device)
        name = "sink_attention"
        if heads % kv_heads:
            raise ValueError(f"{name}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        if not (0 < key_dim <= MAX_DIM and 0 < value_dim <= MAX_DIM):
            raise ValueError(f"{name}: key and value sizes up to {MAX_DIM}, got {key_dim} and "
                             f"{value_dim}")
        if rotary_dim % 2 or not 0 <= rotary_dim <= key_dim:
            raise ValueError(f"{name}: rotary_dim ({rotary_dim}) must be even and at most the key "
                             f"size ({key_dim})")
        if norm not in (None, "head", "whole") or gate not in (None, "head", "feature") \
                or value_mix not in (None, "give", "take") or taps < 0:
            raise ValueError(f"{name}: norm is None, 'head' or 'whole'; gate None, 'head' or "
                             f"'feature'; value_mix None, 'give' or 'take'; taps >= 0")
        if temperature is not None and (len(temperature) != 2 or int(temperature[1]) <= 0):
            raise ValueError(f"{name}: temperature is (coef, every) with every > 0")
        self.width, self.heads, self.kv_heads = width, heads, kv_heads
        self.dk, self.dv, self.scale, self.eps = key_dim, value_dim, float(scale), float(eps)
        self.biased, self.taps, self.norm, self.gate = biased, taps, norm, gate
        self.rotary_dim, self.adjacent, self.temperature = rotary_dim, adjacent, temperature
        self.value_mix, self.mix_key, self.with_slopes = value_mix, mix_key, slopes
        self.channels = (heads + kv_heads) * key_dim + kv_heads * value_dim
        freq, self.magnitude = stretched_frequencies(theta, rotary_dim, stretch)
        self.freq = freq.to(device)
        h = torch.arange(1, heads + 1, dtype=torch.float64)
        self.slopes = (2.0 ** (-8.0 * h / heads)).to(torch.float32).to(device) if slopes else None
        self.key = f"sink_attention/{heads // kv_heads}/{kv_heads}/{key_dim}/{value_dim}"

    # ------------------------------------------------------------------ weights
    def _gate_rows(self) -> int:
        return {None: 0, "head": self.heads, "feature": self.heads * self.dv}[self.gate]

    def tensors(self):
        d, h, g, dk, dv = self.width, self.heads, self.kv_heads, self.dk, self.dv
        out = {"q": ((h * dk, d), "matrix"), "k": ((g * dk, d), "matrix"),
               "v": ((g * dv, d), "matrix"), "o": ((d, h * dv), "matrix"),
               "sink": ((h,), "bias")}
        if self.biased:
            out.update({"q.b": ((h * dk,), "bias"), "k.b": ((g * dk,), "bias"),
                        "v.b": ((g * dv,), "bias")})
        if self.taps:
            out.update({"q.conv": ((h * dk, self.taps), "bias"),
                        "k.conv": ((g * dk, self.taps), "bias"),
                        "v.conv": ((g * dv, self.taps), "bias")})
        if self.norm is not None:
            whole = self.norm == "whole"
            out.update({"q.norm": (((h * dk) if whole else dk,), "vector"),
                        "k.norm": (((g * dk) if whole else dk,), "vector")})
        if self.value_mix is not None:
            out["vmix"] = ((), "bias")
        if self.gate is not None:
            out["g"] = ((self._gate_rows(), d), "matrix")
        return out

    def load(self, tensors):
        mats = [torch.cat((tensors["q"], tensors["k"], tensors["v"]), dim=0)]
        if self.gate is not None:
            mats.append(tensors["g"])
        self._host_in, offsets = stack_segments(mats)
        self.g_col = offsets[1] if self.gate is not None else 0
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.w_in = None
        dev = self.device
        self.sink = vector32(tensors["sink"], dev)
        self.bias = vector32(torch.cat([tensors[n + ".b"].reshape(-1) for n in "qkv"]), dev) \
            if self.biased else None
        self.conv = vector32(torch.cat([tensors[n + ".conv"] for n in "qkv"], dim=0), dev) \
            if self.taps else None
        self.q_norm = vector32(tensors["q.norm"], dev) if self.norm else None
        self.k_norm = vector32(tensors["k.norm"], dev) if self.norm else None
        self.lam = vector32(tensors["vmix"].reshape(1), dev) if self.value_mix else None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def kernel_modules(self):
        return ("attention_chunk",)

    # the norms of a block that reads the stream itself never ride on this mixer's products
    def takes_unscaled(self, n_rows: int) -> bool:
        return False

    def ahead_parts(self, n_rows: int) -> int:
        return 0

    # ------------------------------------------------------------------ cache
    def cache_spec(self):
        pages = PagedKVSpec(self.kv_heads, self.dk, None, value_dim=self.dv)
        if self.taps > 1:
            return (pages, StateSpec(((self.taps - 1) * self.channels,), torch.float32))
        return pages

    @property
    def prepare_key(self) -> str:
        return self.key

    def prepare(self, prep: StepPrep) -> None:
        """The step's tiles of rows (work items of ``kernels.attention_plan``, unsplit).  Their
        number depends on the sequences' token counts only."""
        name = self.key + "/items"
        if prep.has(name):
            return
        host = prep.host
        prep.notes["sink_attention/single_tokens"] = int(host.seq_qlen.max()) == 1
        if int(host.seq_qlen.max()) == 1 and rk.chunk_decode_ok(self.dtype, self.heads,
                                                               self.kv_heads, self.dk, self.dv):
            # single tokens only: the kernel that takes a (sequence, kv head) a block, no items
            prep.add(name, np.zeros((0, 8), dtype=np.int32))
            prep.notes[self.key] = 0
            return
        rows = rk.chunk_rows_per_tile(self.dtype, self.dk, self.dv,
                                      int(host.seq_qlen.max()) > 1,
                                      rk.long_portion_rows(host.seq_qlen, self.heads, self.kv_heads))
        plan = build_plan(host.seq_qlen, host.seq_pos0, self.heads // self.kv_heads,
                          self.kv_heads, rows, 0, chunk=0)
        prep.add(name, plan.items)
        prep.notes[self.key] = rows

    # ------------------------------------------------------------------ step
    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        pages, state = cache, None
        if cache is not None and cache.kind == "parts":
            pages, state = cache.parts
        if pages is None or pages.kind != "paged" or (self.taps > 1) != (state is not None):
            raise ValueError("sink attention needs a paged key/value cache and, with a "
                             "convolution, a state slot")
        n, H, G, dk, dv = proj.shape[0], self.heads, self.kv_heads, self.dk, self.dv
        mix = None
        if self.value_mix == "give":
            first = ctx.buffer(self.mix_key, (n, G * dv), torch.float32)
            ctx.extras[self.mix_key] = first
            mix = ("give", first)
        elif self.value_mix == "take":
            first = ctx.extras.get(self.mix_key)
            if first is None or tuple(first.shape) != (n, G * dv):
                raise ValueError("sink attention: a layer that takes mixed values needs an "
                                 "earlier layer of the step that gives values of the same size")
            mix = ("take", first, self.lam)
        q = ctx.buffer("sink_attention.q", (n, H * dk))
        # in a step of single tokens a slot is read by one block only, which then moves the
        # slot's kept rows on itself
        keep_here = state is not None and bool(ctx.notes.get("sink_attention/single_tokens"))
        rk.qkv_prepare(
            proj, q, H, G, dk, dv, pages.k_pages, pages.v_pages, pages.block_table, ctx,
            bias=self.bias, taps=self.conv, kept=(state.state, 0) if state is not None else None,
            norm=(self.norm, self.q_norm, self.k_norm, self.eps) if self.norm else None,
            rotation=(self.freq, self.magnitude, self.adjacent), temperature=self.temperature,
            mix=mix, keep_here=keep_here)
        if state is not None and not keep_here:
            rk.conv_keep(proj, state.state, 0, self.channels, self.taps, ctx)
        # the gate rides in the attention kernels' last step: the heads' results are multiplied
        # in float32 and rounded once
        context = ctx.buffer("sink_attention.context", (n, H * dv))
        gate = proj[:, self.g_col: self.g_col + self._gate_rows()] if self.gate else None
        extras = dict(slopes=self.slopes, sink=self.sink, gate=gate,
                      gate_per_head=self.gate == "head")
        if ctx.notes[self.key] == 0:
            rk.chunk_attention_decode(q, context, pages.k_pages, pages.v_pages,
                                      pages.block_table, None, None, H, G, dk, dv, self.scale, 0,
                                      ctx, **extras)
        else:
            rk.chunk_attention(q, context, pages.k_pages, pages.v_pages, pages.block_table,
                               ctx.arrays[self.key + "/items"], None, None, H, G, dk, dv,
                               self.scale, 0, ctx, tile_rows=ctx.notes[self.key], **extras)
        return self.project_out(context, "sink_attention.out", ctx, ahead, out_dtype=out_dtype)


register_mixer("sink_attention", SinkAttention)
