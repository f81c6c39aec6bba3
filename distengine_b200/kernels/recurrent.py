"""The kernels of the mixers that carry a state from token to token (``csrc/recurrent.cu``) and of
the chunk-masked attention (``csrc/attention_chunk.cu``) as functions of torch tensors.  Like
``ops``: every function launches on the current stream and checks what it passes on.
"""

from __future__ import annotations

import torch

from . import library
from .ops import _check, _i32, _need, _ptr, _stream, _tag


def _f32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.float32 and t.is_cuda and t.stride(-1) == 1,
          f"{name} must be a float32 CUDA tensor with contiguous rows")


def max_key_dim() -> int:
    return 256


def delta_prep(proj: torch.Tensor, a: torch.Tensor, taps: torch.Tensor, dt_bias: torch.Tensor,
               a_log: torch.Tensor, state: torch.Tensor, conv_offset: int, ctx, qn: torch.Tensor,
               kn: torch.Tensor, vv: torch.Tensor, beta: torch.Tensor, gdec: torch.Tensor,
               heads: int, kv_heads: int, key_dim: int, value_dim: int, b_col: int) -> None:
    """What the delta rule needs of every token, from the stacked projection ``proj``
    = [q (G dk) | k (G dk) | v (H dv) | ...] with b (H) from column ``b_col`` on, and ``a`` float32 [N, H dk] (the low-rank
    decay projection): convolution over time with silu (its earlier inputs from ``state``
    [slots, n] at ``conv_offset``), unit q and k (float32 [N, G dk]; q also times dk^-1/2), values
    float32 [N, H dv], beta float32 [N, H], decays float32 [N, H dk]."""
    n, taps_k = proj.shape[0], taps.shape[1]
    qk, c = 2 * kv_heads * key_dim, 2 * kv_heads * key_dim + heads * value_dim
    _need(proj.stride(1) == 1 and b_col >= c and proj.shape[1] >= b_col + heads,
          "delta_prep: proj is too narrow")
    for t, name, shape in ((a, "a", (n, heads * key_dim)), (taps, "taps", (c, taps_k)),
                           (dt_bias, "dt_bias", (heads * key_dim,)), (a_log, "a_log", (heads,)),
                           (qn, "qn", (n, qk // 2)), (kn, "kn", (n, qk // 2)),
                           (vv, "vv", (n, heads * value_dim)), (beta, "beta", (n, heads)),
                           (gdec, "gdec", (n, heads * key_dim))):
        _f32(t, name)
        _need(tuple(t.shape) == shape and t.is_contiguous(), f"delta_prep: {name} must be "
              f"contiguous {list(shape)}")
    _f32(state, "state")
    _need(state.dim() == 2 and conv_offset + (taps_k - 1) * c <= state.shape[1],
          "delta_prep: the state rows are too short for the convolution's inputs")
    lib = library.load("recurrent")
    _check(lib.de_delta_prep(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), a.data_ptr(),
                             taps.data_ptr(), dt_bias.data_ptr(), a_log.data_ptr(),
                             state.data_ptr(), state.stride(0), conv_offset,
                             ctx.token_seq.data_ptr(), ctx.token_slot.data_ptr(),
                             ctx.positions.data_ptr(), ctx.seq_pos0.data_ptr(), qn.data_ptr(),
                             kn.data_ptr(), vv.data_ptr(), beta.data_ptr(), gdec.data_ptr(), n,
                             heads, kv_heads, key_dim, value_dim, taps_k, b_col, _stream()),
           "delta_prep")


def conv_state(proj: torch.Tensor, state: torch.Tensor, conv_offset: int, channels: int,
               taps: int, ctx) -> None:
    """The slots keep the last ``taps - 1`` inputs of the convolution (the first ``channels``
    columns of ``proj``) of every sequence of the step."""
    _f32(state, "state")
    lib = library.load("recurrent")
    _check(lib.de_conv_state(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), state.data_ptr(),
                             state.stride(0), conv_offset, ctx.seq_slot.data_ptr(),
                             ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.n_seqs,
                             channels, taps, _stream()), "conv_state")


def retention_prep(proj: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, heads: int,
                   key_dim: int, qr: torch.Tensor, kr: torch.Tensor, ctx) -> None:
    """q and k ([q (H dk) | k (H dk) | ...] in ``proj``) rotated by position into float32
    [N, H dk]; k also times dk^-1/2."""
    n = proj.shape[0]
    _need(proj.stride(1) == 1 and proj.shape[1] >= 2 * heads * key_dim,
          "retention_prep: proj is too narrow")
    _f32(inv_freq, "inv_freq")
    _need(inv_freq.shape == (rotary_dim // 2,) and rotary_dim % 2 == 0 and rotary_dim <= key_dim,
          "retention_prep: inv_freq must be [rotary_dim / 2], rotary_dim even and <= key_dim")
    for t in (qr, kr):
        _f32(t, "rotated rows")
        _need(tuple(t.shape) == (n, heads * key_dim) and t.is_contiguous(),
              "retention_prep: outputs must be contiguous [N, H dk]")
    lib = library.load("recurrent")
    _check(lib.de_retention_prep(_tag(proj.dtype), proj.data_ptr(), proj.stride(0),
                                 ctx.positions.data_ptr(), inv_freq.data_ptr(), rotary_dim, heads,
                                 key_dim, qr.data_ptr(), kr.data_ptr(), n, _stream()),
           "retention_prep")


def state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor,
               out: torch.Tensor, heads: int, qk_heads: int, key_dim: int, value_dim: int, ctx,
               g: "torch.Tensor | None" = None, beta: "torch.Tensor | None" = None,
               decay: "torch.Tensor | None" = None, keep: "tuple | None" = None,
               z: "torch.Tensor | None" = None, dots: "torch.Tensor | None" = None) -> None:
    """Walk every sequence's tokens of the step through its state ``state`` [slots, >= H dk dv]
    (float32, rows [h][key channel][value channel] at the front) and write the read-outs, float32
    [N, H dv].  With ``g`` [N, H dk] and ``beta`` [N, H]: the delta rule with a decay per key
    channel.  With ``g`` and ``z`` [N, H dk] and ``dots`` [N, 2 H] (every head's z . q and
    k . q): the generalized delta rule, S <- diag(g) S - z (k^T S) + k v^T with both first terms
    reading the old S.  With ``decay`` [H]: retention.
    q, k float32 [N, qk_heads dk]; v [N, H dv] in
    float32 or the activation dtype (any row stride).  ``keep`` = (proj, offset, channels, taps):
    the slots also keep, at ``offset`` of their rows, the last ``taps - 1`` rows of the first
    ``channels`` columns of ``proj`` of every sequence (a convolution's inputs, as ``conv_state``
    does; the kernel before this one has read the old ones)."""
    n = q.shape[0]
    general = z is not None
    delta = g is not None and not general
    _need((g is not None) != (decay is not None) and (beta is not None) == delta
          and (not general or g is not None), "state_scan: give g and beta, g and z, or decay")
    _need(key_dim <= max_key_dim(), f"state_scan: key size {key_dim} is beyond {max_key_dim()}")
    for t, name in ((q, "q"), (k, "k"), (state, "state"), (out, "out")):
        _f32(t, name)
    _need(q.shape == k.shape == (n, qk_heads * key_dim) and heads % qk_heads == 0,
          "state_scan: q and k must be [N, qk_heads dk]")
    _need(v.stride(1) == 1 and v.shape == (n, heads * value_dim), "state_scan: v [N, H dv]")
    _need(out.is_contiguous() and tuple(out.shape) == (n, heads * value_dim),
          "state_scan: out must be contiguous [N, H dv]")
    _need(state.dim() == 2 and state.shape[1] >= heads * key_dim * value_dim,
          "state_scan: the state rows are too short")
    if delta:
        _f32(g, "g"), _f32(beta, "beta")
        _need(g.shape == (n, heads * key_dim) and beta.shape == (n, heads)
              and v.dtype == torch.float32, "state_scan: g [N, H dk], beta [N, H], v float32")
    elif general:
        _f32(g, "g"), _f32(z, "z"), _f32(dots, "dots")
        _need(g.shape == z.shape == (n, heads * key_dim) and qk_heads == heads
              and dots.shape == (n, 2 * heads),
              "state_scan: g and z [N, H dk], dots [N, 2 H], one query/key head a head")
        beta = dots
    else:
        _f32(decay, "decay")
        _need(decay.shape == (heads,) and decay.is_contiguous(), "state_scan: decay [H]")
    conv = (None, 0, 0, 0, 0, 0)
    if keep is not None:
        proj, offset, channels, taps = keep
        _need(proj.stride(1) == 1 and proj.shape == (n, proj.shape[1]) and proj.shape[1] >= channels
              and offset + (taps - 1) * channels <= state.shape[1],
              "state_scan: the kept convolution inputs do not fit")
        conv = (proj.data_ptr(), proj.stride(0), _tag(proj.dtype), offset, channels, taps)
    lib = library.load("recurrent")
    _check(lib.de_state_scan(2 if general else int(delta), _tag(v.dtype), q.data_ptr(),
                             q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                             _ptr(g), g.stride(0) if g is not None else 0, _ptr(beta),
                             beta.stride(0) if beta is not None else 0, _ptr(z),
                             z.stride(0) if general else 0, _ptr(decay), state.data_ptr(),
                             state.stride(0), out.data_ptr(), ctx.seq_slot.data_ptr(),
                             ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.n_seqs, heads,
                             heads // qk_heads, key_dim, value_dim, *conv, _stream()),
           "state_scan")


def gdelta_prep(proj: torch.Tensor, r_col: int, k_col: int, a_col: int, wl: torch.Tensor,
                w0: torch.Tensor, a_bias: torch.Tensor, rr: torch.Tensor, kk: torch.Tensor,
                ww: torch.Tensor, zz: torch.Tensor, dots: torch.Tensor, heads: int,
                key_dim: int) -> None:
    """What the generalized delta rule needs of every token besides its values, all float32
    [N, H dk]: r and k as they stand in ``proj`` (from columns ``r_col`` and ``k_col``), the
    decays w = exp(-exp(-1/2) sigmoid(wl + w0)) from the low-rank projection ``wl`` (float32), and
    z = sigmoid(a + a_bias) k / (|k|^2 + 1e-6) per head with a from column ``a_col``; and
    ``dots`` float32 [N, 2 H]: every head's (z . r, k . r), which ``state_scan`` takes as
    ``dots``."""
    n, hk = proj.shape[0], heads * key_dim
    _need(proj.stride(1) == 1 and proj.shape[1] >= max(r_col, k_col, a_col) + hk,
          "gdelta_prep: proj is too narrow")
    for t, name in ((wl, "wl"), (rr, "rr"), (kk, "kk"), (ww, "ww"), (zz, "zz")):
        _f32(t, name)
        _need(tuple(t.shape) == (n, hk) and t.is_contiguous(),
              f"gdelta_prep: {name} must be contiguous [N, H dk]")
    for t, name in ((w0, "w0"), (a_bias, "a_bias")):
        _f32(t, name)
        _need(tuple(t.shape) == (hk,) and t.is_contiguous(), f"gdelta_prep: {name} [H dk]")
    _f32(dots, "dots")
    _need(tuple(dots.shape) == (n, 2 * heads) and dots.is_contiguous(),
          "gdelta_prep: dots must be contiguous [N, 2 H]")
    lib = library.load("recurrent")
    _check(lib.de_gdelta_prep(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), r_col, k_col,
                              a_col, wl.data_ptr(), w0.data_ptr(), a_bias.data_ptr(),
                              rr.data_ptr(), kk.data_ptr(), ww.data_ptr(), zz.data_ptr(),
                              dots.data_ptr(), n, heads, key_dim, _stream()), "gdelta_prep")


def silu_rows(proj: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(proj) as float32; proj [N, cols] with a free row stride, out contiguous."""
    _f32(out, "out")
    _need(proj.dim() == 2 and proj.stride(1) == 1 and out.is_contiguous()
          and out.shape == proj.shape, "silu_rows: proj [N, cols], out contiguous of that shape")
    lib = library.load("recurrent")
    _check(lib.de_silu_rows(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), out.data_ptr(),
                            proj.shape[0], proj.shape[1], _stream()), "silu_rows")


def head_gate(o: torch.Tensor, gate: torch.Tensor, weight: "torch.Tensor | None",
              out: torch.Tensor, heads: int, value_dim: int, eps: float,
              spanning: bool = False) -> None:
    """out = o / rms(o over each head) * weight * sigmoid(gate) with a float32 ``gate`` and a
    ``weight`` [dv]; or, without a weight, o / rms * silu(gate) with a gate of out's dtype; or
    (``spanning``) o / rms * weight * sigmoid(gate) with a ``weight`` [H dv] that spans the heads
    and a gate of out's dtype (``heads`` 1 and ``value_dim`` the whole row: the root mean square
    is the row's)."""
    n = o.shape[0]
    _f32(o, "o")
    _need(o.is_contiguous() and o.shape == (n, heads * value_dim) and out.is_contiguous()
          and out.shape == o.shape and gate.stride(1) == 1 and gate.shape == o.shape,
          "head_gate: o, gate and out must be [N, H dv]")
    if spanning:
        _f32(weight, "weight")
        _need(weight.shape == (heads * value_dim,) and gate.dtype == out.dtype,
              "head_gate: a spanning weight is [H dv] and its gate has the output's dtype")
    elif weight is not None:
        _f32(weight, "weight"), _f32(gate, "gate")
        _need(weight.shape == (value_dim,), "head_gate: weight [dv]")
    else:
        _need(gate.dtype == out.dtype, "head_gate: a silu gate has the output's dtype")
    lib = library.load("recurrent")
    _check(lib.de_head_gate(_tag(out.dtype), o.data_ptr(), gate.data_ptr(), gate.stride(0),
                            _ptr(weight), out.data_ptr(), n, heads, value_dim, float(eps),
                            2 if spanning else (0 if weight is not None else 1), _stream()),
           "head_gate")


def mean_of_normed(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor,
                   out: torch.Tensor, eps: float) -> None:
    """out = (a / rms(a) * wa + b / rms(b) * wb) / 2, rows over the width, float32 arithmetic."""
    n, width = a.shape
    _need(a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
          and a.shape == b.shape == out.shape and a.dtype == b.dtype == out.dtype,
          "mean_of_normed: a, b and out must be contiguous, of one shape and dtype")
    _f32(wa, "wa"), _f32(wb, "wb")
    _need(wa.shape == wb.shape == (width,), "mean_of_normed: weights [width]")
    lib = library.load("recurrent")
    _check(lib.de_mean_of_normed(_tag(out.dtype), a.data_ptr(), b.data_ptr(), wa.data_ptr(),
                                 wb.data_ptr(), out.data_ptr(), n, width, float(eps), _stream()),
           "mean_of_normed")


# ------------------------------------------------------------------------------- chunk attention
def _penalty(r1, r2, heads: int, slopes=None, sink=None, gate=None, gate_per_head=False,
             like=None, value_dim=0):
    """The penalty's two pointers and the kernels' last arguments (linear, sink, gate, its row
    stride, whether it is one number a head): either r1 log(1 + r2 distance) or ``slopes``
    [heads] times the distance; ``sink`` [heads]: the softmax's denominator also holds exp(sink);
    ``gate`` [N, heads dv] (or [N, heads] with ``gate_per_head``) of the queries' dtype ``like``:
    a row's result is multiplied by sigmoid(gate) before it is stored."""
    gated = (None, 0, 0)
    if gate is not None:
        _need(gate.dtype == like and gate.stride(1) == 1 and gate.dim() == 2
              and gate.shape[1] == (heads if gate_per_head else heads * value_dim),
              "attention: gate [N, heads dv] or [N, heads] of the queries' dtype")
        gated = (gate.data_ptr(), gate.stride(0), int(bool(gate_per_head)))
    _need((r1 is None) == (r2 is None), "attention: r1 and r2 come together")
    _need(r1 is None or slopes is None, "attention: one distance penalty, not two")
    if r1 is not None:
        _f32(r1, "r1"), _f32(r2, "r2")
        _need(r1.shape == r2.shape == (heads,), "attention: r1, r2 [heads]")
    for t, name in ((slopes, "slopes"), (sink, "sink")):
        if t is not None:
            _f32(t, name)
            _need(t.shape == (heads,) and t.is_contiguous(), f"attention: {name} [heads]")
    if slopes is not None:
        return slopes, slopes, (1, _ptr(sink), *gated)
    return r1, r2, (0, _ptr(sink), *gated)


def chunk_rows_per_tile(dtype: torch.dtype, key_dim: int, value_dim: int, wide: bool,
                        longest_rows: int = 0) -> int:
    """Rows of a tile of the chunk attention: 8, or 32 for steps with prompt portions (``wide``)
    at sizes whose rows are whole 16-byte pieces, or 64 where the longest portion has at least 48
    rows (``longest_rows``: its tokens times the query heads a kv head)."""
    hint = max(int(wide), int(longest_rows)) if wide else 0
    return int(library.load("attention_chunk").de_attn_chunk_rows(_tag(dtype), key_dim, value_dim,
                                                                  hint))


_sm_count: dict[int, int] = {}


def long_portion_rows(seq_qlen, heads: int, kv_heads: int) -> int:
    """The rows of a step's longest portion (tokens times query heads a kv head) if tiles of 64
    rows would still give every SM two blocks, else 0: what ``chunk_rows_per_tile`` takes as
    ``longest_rows``.  (Measured on B200, 16 heads on 4 kv heads of 128: a prompt of 512 tokens
    takes 274 us in 128 blocks of 64 rows against 221 us in 256 blocks of 32; one of 2,048 tokens
    739 against 1,362 us.)"""
    group = heads // kv_heads
    device = torch.cuda.current_device()
    if device not in _sm_count:
        _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    blocks = int(((seq_qlen.astype("int64") * group + 63) // 64).sum()) * kv_heads
    return int(seq_qlen.max()) * group if blocks >= 2 * _sm_count[device] else 0


def chunk_decode_ok(dtype: torch.dtype, heads: int, kv_heads: int, key_dim: int,
                    value_dim: int, values_in_keys: bool = False) -> bool:
    """Whether steps of single tokens can go to ``chunk_attention_decode``.  ``values_in_keys``:
    the values are the first ``value_dim`` features of the keys (one set of pages)."""
    return bool(library.load("attention_chunk").de_attn_chunk_decode_ok(
        _tag(dtype), heads, kv_heads, key_dim, value_dim, 1 if values_in_keys else 0))


def chunk_attention_decode(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, block_table: torch.Tensor, r1: torch.Tensor,
                           r2: torch.Tensor, heads: int, kv_heads: int, key_dim: int,
                           value_dim: int, scale: float, chunk: int, ctx, window: int = 0,
                           keep_first: int = 0, softcap: float = 0.0,
                           fused: "dict | None" = None, v_stride: int = 0,
                           slopes: "torch.Tensor | None" = None,
                           sink: "torch.Tensor | None" = None,
                           gate: "torch.Tensor | None" = None,
                           gate_per_head: bool = False) -> None:
    """``chunk_attention`` for a step in which every sequence brings one token: a block a
    (sequence, kv head), its warps share the key tiles out; no work items.

    ``fused`` = {fk, rotary_dim, fv, write_kv, gate}: the kernel also does what
    ``kv_write_rotated`` and ``attention_finish`` do around the other kernels - it turns the
    queries (in its own memory: ``q`` stays as it is), turns and stores the token's key and value
    (``q``'s rows are then [q (H dk) | k (G dk) | v (G dv) | ...]), turns every head's result back
    and gates it; ``out`` has the activation dtype.

    ``v_stride`` not 0: the values of consecutive keys lie that many elements apart in
    ``v_pages`` (values that are the first features of the key rows: ``v_pages`` is ``k_pages``
    and the stride the key size)."""
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == k_pages.dtype
          and out.dtype in (q.dtype, torch.float32)
          and out.shape[1] == heads * value_dim and q.shape[0] == ctx.n_seqs,
          "chunk_attention_decode: q, out and pages; one token a sequence")
    _i32(block_table, "block_table")
    r1, r2, last = _penalty(r1, r2, heads, slopes, sink, gate, gate_per_head, q.dtype, value_dim)
    extra = (0, None, 0, None, 0, None, 0)
    if fused is not None:
        fk, rot, fv, gate = fused["fk"], fused["rotary_dim"], fused["fv"], fused["gate"]
        write_kv = bool(fused["write_kv"])
        need = heads * key_dim + (kv_heads * (key_dim + value_dim) if write_kv else 0)
        _need(out.dtype == q.dtype and q.shape[1] >= need, "chunk_attention_decode: fused steps "
              "write the activation dtype and find k and v behind q")
        _f32(fk, "fk")
        _need(rot % 2 == 0 and 0 <= rot <= key_dim and fk.shape == (rot // 2,),
              "chunk_attention_decode: fk [rotary_dim / 2]")
        if fv is not None:
            _f32(fv, "fv")
            _need(value_dim % 2 == 0 and fv.shape == (value_dim // 2,),
                  "chunk_attention_decode: fv [dv / 2]")
        if gate is not None:
            _need(gate.dtype == out.dtype and gate.stride(1) == 1
                  and gate.shape == (q.shape[0], heads * value_dim),
                  "chunk_attention_decode: gate [N, H dv] of out's dtype")
        extra = (1, fk.data_ptr(), rot, _ptr(fv), int(write_kv), _ptr(gate),
                 gate.stride(0) if gate is not None else 0)
    lib = library.load("attention_chunk")
    _check(lib.de_attn_chunk_decode(_tag(q.dtype), q.data_ptr(), q.stride(0), out.data_ptr(),
                                    out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                                    block_table.data_ptr(), block_table.stride(0),
                                    k_pages.shape[0], ctx.seq_slot.data_ptr(),
                                    ctx.seq_qstart.data_ptr(), ctx.seq_pos0.data_ptr(),
                                    ctx.n_seqs, _ptr(r1), _ptr(r2), heads, kv_heads,
                                    key_dim, value_dim, k_pages.shape[2], float(scale),
                                    int(chunk), int(window), int(keep_first), float(softcap),
                                    int(out.dtype == torch.float32 and q.dtype != torch.float32),
                                    *extra, int(v_stride), *last, ctx.status.data_ptr(),
                                    _stream()),
           "chunk_attention_decode")


def kv_write_normed(proj: torch.Tensor, k_col: int, kv_heads: int, key_dim: int, value_dim: int,
                    eps: float, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    block_table: torch.Tensor, ctx) -> None:
    """Store every token's keys ([k (G dk) | v (G dv)] from column ``k_col`` of ``proj``) and its
    values, each head's divided by its root mean square, in the pages."""
    _need(proj.stride(1) == 1 and proj.shape[1] >= k_col + kv_heads * (key_dim + value_dim)
          and proj.dtype == k_pages.dtype == v_pages.dtype, "kv_write_normed: proj and pages")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and tuple(k_pages.shape[1:]) == (kv_heads, k_pages.shape[2], key_dim)
          and tuple(v_pages.shape) == (*k_pages.shape[:3], value_dim),
          "kv_write_normed: pages must be [pages, kv_heads, page, dk] and [..., dv]")
    _i32(block_table, "block_table")
    lib = library.load("attention_chunk")
    _check(lib.de_kv_write_normed(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), k_col,
                                  ctx.positions.data_ptr(), ctx.token_slot.data_ptr(), kv_heads,
                                  key_dim, value_dim, float(eps), k_pages.data_ptr(),
                                  v_pages.data_ptr(), block_table.data_ptr(),
                                  block_table.stride(0), k_pages.shape[2], k_pages.shape[0],
                                  proj.shape[0], ctx.status.data_ptr(), _stream()),
           "kv_write_normed")


def chunk_attention(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor,
                    v_pages: torch.Tensor, block_table: torch.Tensor, items: torch.Tensor,
                    r1: torch.Tensor, r2: torch.Tensor, heads: int, kv_heads: int, key_dim: int,
                    value_dim: int, scale: float, chunk: int, ctx, tile_rows: int = 8,
                    window: int = 0, keep_first: int = 0, softcap: float = 0.0,
                    v_stride: int = 0, slopes: "torch.Tensor | None" = None,
                    sink: "torch.Tensor | None" = None, gate: "torch.Tensor | None" = None,
                    gate_per_head: bool = False) -> None:
    """Attention of the step's rows over the pages: q rows of [heads dk] at the front of ``q``
    (row stride free), out [N, heads dv]; ``tile_rows``: the rows of a tile that ``items`` were
    cut for (``chunk_rows_per_tile``); ``v_stride`` as in ``chunk_attention_decode``; see
    ``csrc/attention_chunk.cu``."""
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == k_pages.dtype
          and out.dtype in (q.dtype, torch.float32)
          and out.shape[1] == heads * value_dim, "chunk_attention: q, out and pages")
    _i32(block_table, "block_table"), _i32(items, "items")
    r1, r2, last = _penalty(r1, r2, heads, slopes, sink, gate, gate_per_head, q.dtype, value_dim)
    lib = library.load("attention_chunk")
    _check(lib.de_attn_chunk(_tag(q.dtype), q.data_ptr(), q.stride(0), out.data_ptr(),
                             out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                             block_table.data_ptr(), block_table.stride(0), k_pages.shape[0],
                             ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(),
                             ctx.seq_qlen.data_ptr(), ctx.seq_pos0.data_ptr(), items.data_ptr(),
                             items.shape[0], _ptr(r1), _ptr(r2), heads, kv_heads,
                             key_dim, value_dim, k_pages.shape[2], float(scale), int(chunk),
                             int(window), int(keep_first), float(softcap),
                             int(out.dtype == torch.float32 and q.dtype != torch.float32),
                             int(tile_rows), int(v_stride), *last, ctx.status.data_ptr(),
                             _stream()),
           "chunk_attention")


def kv_write_rotated(proj: torch.Tensor, fk: torch.Tensor, rotary_dim: int,
                     fv: "torch.Tensor | None", heads: int, kv_heads: int, key_dim: int,
                     value_dim: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, write_kv: bool, ctx) -> None:
    """Turn the queries at the front of ``proj`` ([q (H dk) | k (G dk) | v (G dv) | ...]) by their
    tokens' positions in place and store the turned keys and the values in the pages; ``fk``
    [rotary_dim / 2] are the frequencies of the first ``rotary_dim`` features of queries and
    keys, ``fv`` [dv / 2] (or None: values as they are) those of all features of the values.
    ``write_kv`` false: a run that reads another run's cache turns its queries only."""
    need = heads * key_dim + (kv_heads * (key_dim + value_dim) if write_kv else 0)
    _need(proj.stride(1) == 1 and proj.shape[1] >= need and proj.dtype == k_pages.dtype
          == v_pages.dtype, "kv_write_rotated: proj and pages")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and tuple(k_pages.shape[1:]) == (kv_heads, k_pages.shape[2], key_dim)
          and tuple(v_pages.shape) == (*k_pages.shape[:3], value_dim),
          "kv_write_rotated: pages must be [pages, kv_heads, page, dk] and [..., dv]")
    _i32(block_table, "block_table")
    _f32(fk, "fk")
    _need(rotary_dim % 2 == 0 and 0 <= rotary_dim <= key_dim and fk.shape == (rotary_dim // 2,),
          "kv_write_rotated: fk [rotary_dim / 2], rotary_dim even and at most the key size")
    if fv is not None:
        _f32(fv, "fv")
        _need(value_dim % 2 == 0 and fv.shape == (value_dim // 2,),
              "kv_write_rotated: fv [dv / 2], dv even")
    lib = library.load("attention_chunk")
    _check(lib.de_kv_write_rotated(_tag(proj.dtype), proj.data_ptr(), proj.stride(0),
                                   ctx.positions.data_ptr(), ctx.token_slot.data_ptr(),
                                   fk.data_ptr(), rotary_dim, _ptr(fv), heads, kv_heads, key_dim,
                                   value_dim, k_pages.data_ptr(), v_pages.data_ptr(),
                                   block_table.data_ptr(), block_table.stride(0),
                                   k_pages.shape[2], k_pages.shape[0], int(write_kv),
                                   proj.shape[0], ctx.status.data_ptr(), _stream()),
           "kv_write_rotated")


def attention_finish(o: torch.Tensor, fv: "torch.Tensor | None", gate: "torch.Tensor | None",
                     out: torch.Tensor, heads: int, value_dim: int, ctx,
                     gate_per_head: bool = False) -> None:
    """out = the heads' results ``o`` (float32 [N, H dv]) turned back by their tokens' positions
    (``fv`` as in ``kv_write_rotated``) and multiplied by sigmoid(``gate``) (of out's dtype, free
    row stride; [N, H dv], or [N, H] with ``gate_per_head``), where given."""
    n = o.shape[0]
    _f32(o, "o")
    _need(o.is_contiguous() and o.shape == (n, heads * value_dim) and out.is_contiguous()
          and out.shape == o.shape, "attention_finish: o and out [N, H dv]")
    if fv is not None:
        _f32(fv, "fv")
        _need(value_dim % 2 == 0 and fv.shape == (value_dim // 2,), "attention_finish: fv [dv / 2]")
    if gate is not None:
        _need(gate.dtype == out.dtype and gate.stride(1) == 1
              and gate.shape == ((n, heads) if gate_per_head else o.shape),
              "attention_finish: gate [N, H dv] (or [N, H]) of out's dtype")
    lib = library.load("attention_chunk")
    _check(lib.de_attn_finish(_tag(out.dtype), o.data_ptr(), ctx.positions.data_ptr(), _ptr(fv),
                              _ptr(gate), gate.stride(0) if gate is not None else 0,
                              out.data_ptr(), n, heads, value_dim, int(gate_per_head), _stream()),
           "attention_finish")


def conv_keep(proj: torch.Tensor, state: torch.Tensor, conv_offset: int, channels: int, taps: int,
              ctx) -> None:
    """What ``conv_state`` does, from the attention kernels' library: the slots keep the last
    ``taps - 1`` rows of the first ``channels`` columns of ``proj`` of every sequence of the
    step, for ``qkv_prepare`` of the next step."""
    _f32(state, "state")
    _need(proj.stride(1) == 1 and proj.shape[1] >= channels and state.dim() == 2
          and conv_offset + (taps - 1) * channels <= state.shape[1],
          "conv_keep: the kept rows do not fit")
    lib = library.load("attention_chunk")
    _check(lib.de_conv_keep(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), state.data_ptr(),
                            state.stride(0), conv_offset, ctx.seq_slot.data_ptr(),
                            ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.n_seqs,
                            channels, taps, _stream()), "conv_keep")


def qkv_prepare(proj: torch.Tensor, q_out: torch.Tensor, heads: int, kv_heads: int, key_dim: int,
                value_dim: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                block_table: torch.Tensor, ctx, bias: "torch.Tensor | None" = None,
                taps: "torch.Tensor | None" = None, kept: "tuple | None" = None,
                norm: "tuple | None" = None, rotation: "tuple | None" = None,
                temperature: "tuple | None" = None, mix: "tuple | None" = None,
                keep_here: bool = False) -> None:
    """From the stacked projection ``proj`` = [q (H dk) | k (G dk) | v (G dv) | ...] to the
    queries ``q_out`` [N, H dk] and the keys and values in the pages, through (each optional, in
    this order): ``bias`` float32 [C] (C = (H + G) dk + G dv); ``taps`` float32 [C, K], a causal
    convolution over time whose inputs before the step come from ``kept`` = (state [slots, n],
    offset), laid out as ``conv_keep`` leaves them; ``norm`` = (mode, q weight, k weight, eps),
    mode "head" (weights [dk]) or "whole" (weights [H dk], [G dk]); ``rotation`` = (freq
    [rot / 2], magnitude, adjacent); ``temperature`` = (coef, every) on q; ``mix`` = ("give",
    v_first) or ("take", v_first, lambda [1]) with v_first float32 [N, G dv].  ``keep_here``:
    only for a step in which every sequence brings one token - the kernel then also moves the
    slots' kept rows on, and no ``conv_keep`` follows."""
    n = proj.shape[0]
    channels = (heads + kv_heads) * key_dim + kv_heads * value_dim
    _need(proj.stride(1) == 1 and proj.shape[1] >= channels and proj.dtype == k_pages.dtype
          == v_pages.dtype == q_out.dtype and q_out.is_contiguous()
          and q_out.shape == (n, heads * key_dim), "qkv_prepare: proj, q_out [N, H dk] and pages")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and tuple(k_pages.shape[1:]) == (kv_heads, k_pages.shape[2], key_dim)
          and tuple(v_pages.shape) == (*k_pages.shape[:3], value_dim),
          "qkv_prepare: pages must be [pages, kv_heads, page, dk] and [..., dv]")
    _i32(block_table, "block_table")
    if bias is not None:
        _f32(bias, "bias")
        _need(bias.shape == (channels,) and bias.is_contiguous(), "qkv_prepare: bias [C]")
    conv = (None, 0, None, 0, 0)
    if taps is not None:
        _f32(taps, "taps")
        _need(taps.dim() == 2 and taps.shape[0] == channels and taps.is_contiguous(),
              "qkv_prepare: taps [C, K]")
        k = taps.shape[1]
        conv = (taps.data_ptr(), k, None, 0, 0)
        if k > 1:
            state, offset = kept
            _f32(state, "state")
            _need(state.dim() == 2 and offset + (k - 1) * channels <= state.shape[1],
                  "qkv_prepare: the state rows are too short for the convolution's inputs")
            conv = (taps.data_ptr(), k, state.data_ptr(), state.stride(0), offset)
    normed = (0, None, None, 0.0)
    if norm is not None:
        mode, qw, kw, eps = norm
        _need(mode in ("head", "whole"), "qkv_prepare: norm over a head or the whole projection")
        _f32(qw, "q weight"), _f32(kw, "k weight")
        shapes = ((key_dim,), (key_dim,)) if mode == "head" else ((heads * key_dim,),
                                                                   (kv_heads * key_dim,))
        _need((tuple(qw.shape), tuple(kw.shape)) == shapes and qw.is_contiguous()
              and kw.is_contiguous(), "qkv_prepare: the norm's weights do not fit its mode")
        normed = (1 if mode == "head" else 2, qw.data_ptr(), kw.data_ptr(), float(eps))
    turned = (None, 0, 1.0, 0)
    if rotation is not None and rotation[0].numel() > 0:
        freq, magnitude, adjacent = rotation
        _f32(freq, "freq")
        _need(freq.dim() == 1 and 2 * freq.shape[0] <= key_dim and freq.is_contiguous(),
              "qkv_prepare: freq [rot / 2], rot at most the key size")
        turned = (freq.data_ptr(), 2 * freq.shape[0], float(magnitude), int(bool(adjacent)))
    temp = (0.0, 0) if temperature is None else (float(temperature[0]), int(temperature[1]))
    mixed = (0, None, None)
    if mix is not None:
        v_first = mix[1]
        _f32(v_first, "v_first")
        _need(v_first.is_contiguous() and v_first.shape == (n, kv_heads * value_dim),
              "qkv_prepare: v_first [N, G dv]")
        if mix[0] == "take":
            _f32(mix[2], "lambda")
            mixed = (2, mix[2].data_ptr(), v_first.data_ptr())
        else:
            _need(mix[0] == "give", "qkv_prepare: mix gives or takes")
            mixed = (1, None, v_first.data_ptr())
    lib = library.load("attention_chunk")
    _check(lib.de_qkv_prepare(_tag(proj.dtype), proj.data_ptr(), proj.stride(0), q_out.data_ptr(),
                              ctx.positions.data_ptr(), ctx.token_seq.data_ptr(),
                              ctx.token_slot.data_ptr(), ctx.seq_pos0.data_ptr(), _ptr(bias),
                              *conv, *normed, *turned, *temp, *mixed, int(bool(keep_here)), heads,
                              kv_heads, key_dim, value_dim, k_pages.data_ptr(), v_pages.data_ptr(),
                              block_table.data_ptr(), block_table.stride(0), k_pages.shape[2],
                              k_pages.shape[0], n, ctx.status.data_ptr(), _stream()),
           "qkv_prepare")
