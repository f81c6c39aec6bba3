"""Latent attention: causal softmax attention whose keys and values of all heads are read from one
small latent per token, the only thing that is cached (with one rotated key part that all heads
share).

    cq = rms_norm(W_dq x) * n_q ;  q = W_uq cq            per head [key_dim plain | rotary_dim turned]
    [c' | kr] = W_dkv x ;  c = rms_norm(c') * n_kv         c [kv_rank], kr [rotary_dim]
    k_h = W_uk[h] c ;  v_h = W_uv[h] c
    score_h(i, j) = (q_h,plain(i) . k_h(j) + turn(q_h,rot(i)) . turn(kr(j))) * scale ;  j <= i
    out = W_o [ heads' weighted sums of v_h * sigmoid(W_g x) ]

Run in the folded form, which reads nothing but [c | turn(kr)] of a key:
q'_h = W_uk[h]^T q_h,plain, score = (q'_h . c + turn(q_h,rot) . turn(kr)) * scale, the weighted sum
is taken over c and W_uv[h] is applied to it afterwards.  That is attention with one key/value head
of size kv_rank + rotary_dim whose values are the first kv_rank features of its keys, which the
kernels of ``csrc/attention_chunk.cu`` run; the per-head products are ``kernels.latent``.

Turning: the pair (i, i + rotary_dim / 2) of the rotated part by the angle position * f_i, with
f_i = theta^(-2i / rotary_dim).  ``scaling`` = (factor, original, fast, slow) stretches the slow
frequencies: with d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta),
lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and the ramp
r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- f_i / factor * r_i + f_i * (1 - r_i), and
cosines and sines are multiplied by 0.1 ln(factor) + 1.  ``scale`` is used as it is given.

Steps with prompt portions in bfloat16, when the cached row is a multiple of 16 features up to the
tensor-core attention's largest head: the kernels of ``kernels.attention`` (mma.sync, or tcgen05
at rows of 64 and 128 features) run it as one key/value head whose value pages are its key pages;
the weighted sums then cover the whole row, and the per-head value product reads their first
kv_rank features.  Other steps: the CUDA-core kernels of ``csrc/attention_chunk.cu``.

Scores, softmax weights, angles and norm statistics are float32; so is the weighted sum over the
latent on the CUDA-core kernels (the tensor-core kernels round the softmax weights and the sums
to bfloat16, as they do for every model).
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import latent as lk
from ..kernels import ops
from ..kernels import recurrent as rk
from ..kernels.attention import MAX_HEAD_DIM, AttentionLauncher, uses_tensor_cores
from ..kernels.attention_plan import build_plan
from .base import Mixer, PagedKVSpec, compute_matrix, register_mixer, stored_vector
from .context import CacheBinding, StepContext, StepPrep
from .recurrent import stack_segments

MAX_RANK, MAX_ROW = 256, 576    # of kv_rank and of kv_rank + rotary_dim: what the attention
                                # kernels take as value and key sizes


def stretched_frequencies(theta: float, dims: int, scaling=None) -> "tuple[torch.Tensor, float]":
    """(float64 [dims / 2], magnitude of cosine and sine); see the module's text."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(theta) ** (-2.0 * i / max(dims, 1))
    if scaling is None:
        return f, 1.0
    factor, original, fast, slow = (float(x) for x in scaling)

    def turns_at(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))

    lo = max(math.floor(turns_at(fast)), 0)
    hi = min(math.ceil(turns_at(slow)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class LatentAttention(Mixer):
    kind = "latent_attention"

    def __init__(self, width: int, heads: int, key_dim: int, rotary_dim: int, value_dim: int,
                 q_rank: int, kv_rank: int, scale: float, theta: float, eps: float,
                 dtype: torch.dtype, device: torch.device, scaling=None) -> None:
        super().__init__(dtype, device)
        if rotary_dim % 2 or rotary_dim < 0:
            raise ValueError(f"latent_attention: rotary_dim ({rotary_dim}) must be even")
        if kv_rank > MAX_RANK or kv_rank + rotary_dim > MAX_ROW:
            raise ValueError(f"latent_attention: kv_rank up to {MAX_RANK} and kv_rank + "
                             f"rotary_dim up to {MAX_ROW}, got {kv_rank} and "
                             f"{kv_rank + rotary_dim}")
        self.width, self.heads, self.dim, self.rot, self.dv = width, heads, key_dim, rotary_dim, value_dim
        self.q_rank, self.rank, self.scale, self.eps = q_rank, kv_rank, float(scale), float(eps)
        freq, self.magnitude = stretched_frequencies(theta, rotary_dim, scaling)
        self.freq = freq.to(device)
        self.row = kv_rank + rotary_dim              # what a key's row in the pages holds
        self.key = f"latent_attention/{heads}/{kv_rank}/{rotary_dim}"
        # prompt portions on the tensor cores: one key/value head of `row` features
        self.launcher = None
        if uses_tensor_cores(dtype, self.row) and self.row <= MAX_HEAD_DIM:
            self.launcher = AttentionLauncher(dtype, heads, 1, self.row, self.scale, None, device)

    def tensors(self):
        d, h = self.width, self.heads
        return {"dq": ((self.q_rank, d), "matrix"), "dq.norm": ((self.q_rank,), "vector"),
                "uq": ((h * (self.dim + self.rot), self.q_rank), "matrix"),
                "dkv": ((self.row, d), "matrix"), "dkv.norm": ((self.rank,), "vector"),
                "uk": ((h * self.dim, self.rank), "matrix"),
                "uv": ((h * self.dv, self.rank), "matrix"),
                "g": ((h * self.dv, d), "matrix"), "o": ((d, h * self.dv), "matrix")}

    def load(self, tensors):
        stacked, offsets = stack_segments([tensors["dq"], tensors["dkv"], tensors["g"]])
        self.kv_col, self.g_col = offsets[1], offsets[2]
        self.w_in = compute_matrix(stacked, self.dtype, self.device)
        self.w_uq = compute_matrix(tensors["uq"], self.dtype, self.device)
        h = self.heads
        # W_uk[h]^T as the matrix of a product: [H, kv_rank, key_dim]
        self.w_uk_t = compute_matrix(tensors["uk"].reshape(h, self.dim, self.rank).transpose(1, 2),
                                     self.dtype, self.device)
        self.w_uv = compute_matrix(tensors["uv"].reshape(h, self.dv, self.rank), self.dtype,
                                   self.device)
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.n_q = stored_vector(tensors["dq.norm"], self.dtype, self.device)
        self.n_kv = stored_vector(tensors["dkv.norm"], self.dtype, self.device)

    def kernel_modules(self):
        mine = ("attention_chunk", "latent")
        if self.launcher is None:
            return mine
        # the launcher's kernels for work items (not its single-token one, which is not used here)
        wide = (self.launcher.tcgen05_module,) if self.launcher.shapes[0].code == 2 else ()
        return mine + (self.launcher.module, ("attention_simt", ())) + wide

    def cache_spec(self):
        return PagedKVSpec(1, self.row, value_dim=self.rank, values_in_keys=True)

    @property
    def prepare_key(self) -> str:
        return self.key

    def _decode_kernel(self) -> bool:
        return rk.chunk_decode_ok(self.dtype, self.heads, 1, self.row, self.rank, True)

    def prepare(self, prep: StepPrep) -> None:
        """The step's tiles of rows (work items of ``kernels.attention_plan``, unsplit): all heads
        of a token are rows of the one key/value head."""
        name = self.key + "/items"
        if prep.has(name):
            return
        host = prep.host
        longest = int(host.seq_qlen.max())
        if longest == 1 and self._decode_kernel():
            prep.add(name, np.zeros((0, 8), dtype=np.int32))
            prep.notes[self.key] = 0
            return
        if self.launcher is not None:
            self.launcher.prepare(prep, allow_decode=False)
            prep.add(name, np.zeros((0, 8), dtype=np.int32))
            prep.notes[self.key] = -1
            return
        rows = rk.chunk_rows_per_tile(self.dtype, self.row, self.rank, longest > 1,
                                      rk.long_portion_rows(host.seq_qlen, self.heads, 1))
        plan = build_plan(host.seq_qlen, host.seq_pos0, self.heads, 1, rows, 0, chunk=0)
        prep.add(name, plan.items)
        prep.notes[self.key] = rows

    def forward(self, x: torch.Tensor, ctx: StepContext,
                cache: "CacheBinding | None") -> torch.Tensor:
        if cache is None or cache.kind != "paged" or not cache.writes:
            raise ValueError("latent attention needs a paged cache of its own")
        n, H = x.shape[0], self.heads
        proj = ctx.buffer("latent_attention.proj", (n, self.w_in.shape[0]))
        ops.linear(x, self.w_in, out=proj, status=ctx.status)
        cq = ctx.buffer("latent_attention.cq", (n, self.q_rank))
        ops.rmsnorm_cols(proj[:, : self.q_rank], self.n_q, self.eps, cq)
        q = ctx.buffer("latent_attention.q", (n, H * (self.dim + self.rot)))
        ops.linear(cq, self.w_uq, out=q, status=ctx.status)
        folded = ctx.buffer("latent_attention.folded", (n, H * self.row))
        lk.latent_write(q, proj[:, self.kv_col: self.kv_col + self.row], folded, self.freq,
                        self.magnitude, self.n_kv, self.eps, H, self.dim, self.rot, self.rank,
                        cache.k_pages, cache.block_table, ctx)
        lk.heads_product(q, self.dim + self.rot, self.w_uk_t, folded, self.row)
        if ctx.notes[self.key] == -1:
            sums = ctx.buffer("latent_attention.sums", (n, H * self.row))
            self.launcher.run(folded, sums, cache.k_pages, cache.k_pages, cache.block_table, ctx)
            return self._finish(sums, self.row, proj, ctx)
        mixed = ctx.buffer("latent_attention.mixed", (n, H * self.rank), torch.float32)
        if ctx.notes[self.key] == 0:
            rk.chunk_attention_decode(folded, mixed, cache.k_pages, cache.k_pages,
                                      cache.block_table, None, None, H, 1, self.row, self.rank,
                                      self.scale, 0, ctx, v_stride=self.row)
        else:
            rk.chunk_attention(folded, mixed, cache.k_pages, cache.k_pages, cache.block_table,
                               ctx.arrays[self.key + "/items"], None, None, H, 1, self.row,
                               self.rank, self.scale, 0, ctx, tile_rows=ctx.notes[self.key],
                               v_stride=self.row)
        return self._finish(mixed, self.rank, proj, ctx)

    def _finish(self, sums: torch.Tensor, stride: int, proj: torch.Tensor,
                ctx: StepContext) -> torch.Tensor:
        """The heads' weighted sums over the latent (head h's at columns h * stride) through
        W_uv[h], the gate and W_o."""
        n, H = sums.shape[0], self.heads
        context = ctx.buffer("latent_attention.context", (n, H * self.dv))
        lk.heads_product(sums, stride, self.w_uv, context, self.dv,
                         gate=proj[:, self.g_col: self.g_col + H * self.dv])
        out = ctx.buffer("latent_attention.out", (n, self.width))
        ops.linear(context, self.w_o, out=out, status=ctx.status)
        return out


register_mixer("latent_attention", LatentAttention)
