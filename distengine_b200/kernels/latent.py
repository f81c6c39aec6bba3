"""Tensor-level wrappers of the latent-attention kernels (``csrc/latent.cu``) and of the routed
experts (``csrc/experts.cu``)."""

from __future__ import annotations

import torch

from . import library
from .ops import ACTIVATIONS, _check, _i32, _need, _ptr, _stream, _tag


def latent_write(q: torch.Tensor, kv: torch.Tensor, qa: torch.Tensor, freq: torch.Tensor,
                 magnitude: float, norm_weight: torch.Tensor, eps: float, heads: int, dim: int,
                 rot: int, rank: int, pages: torch.Tensor, block_table: torch.Tensor, ctx) -> None:
    """Per token: the latent c = rms_norm(kv[:, :rank]) * norm_weight and the key part kv[:, rank:]
    turned by the token's position go to the pages ([pages, 1, page, rank + rot]); every head's
    rotated query part (q rows are heads of [dim | rot]) goes, turned, to columns rank.. of its
    head in ``qa`` (rows of heads of [rank | rot]).  ``freq`` float64 [rot / 2]; cosine and sine
    are multiplied by ``magnitude``."""
    n = q.shape[0]
    _need(q.stride(1) == 1 and kv.stride(1) == 1 and qa.stride(1) == 1
          and q.shape[1] >= heads * (dim + rot) and kv.shape == (n, rank + rot)
          and qa.shape == (n, heads * (rank + rot)) and q.dtype == kv.dtype == qa.dtype
          == pages.dtype, "latent_write: q [N, H (dim + rot)], kv [N, rank + rot], qa "
          "[N, H (rank + rot)] of the pages' dtype")
    _need(pages.is_contiguous() and pages.dim() == 4 and pages.shape[1] == 1
          and pages.shape[3] == rank + rot, "latent_write: pages [pages, 1, page, rank + rot]")
    _need(freq.dtype == torch.float64 and freq.is_contiguous() and freq.shape == (rot // 2,)
          and rot % 2 == 0, "latent_write: freq float64 [rot / 2]")
    _need(norm_weight.is_contiguous() and norm_weight.shape == (rank,), "latent_write: weight")
    _i32(block_table, "block_table")
    lib = library.load("latent")
    _check(lib.de_latent_write(_tag(q.dtype), _tag(norm_weight.dtype), q.data_ptr(), q.stride(0),
                               kv.data_ptr(), kv.stride(0), qa.data_ptr(), qa.stride(0),
                               ctx.positions.data_ptr(), ctx.token_slot.data_ptr(),
                               freq.data_ptr(), float(magnitude), norm_weight.data_ptr(),
                               float(eps), heads, dim, rot, rank, pages.data_ptr(),
                               block_table.data_ptr(), block_table.stride(0), pages.shape[2],
                               pages.shape[0], n, ctx.status.data_ptr(), _stream()),
           "latent_write")


def heads_product(a: torch.Tensor, a_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int,
                  gate: "torch.Tensor | None" = None) -> None:
    """out[n, h * out_head + j] = sum_i a[n, h * a_head + i] * w[h, j, i], float32 sums on the CUDA
    cores; w [H, cols, depth] contiguous.  ``gate`` [N, H cols] (w's dtype, free row stride): the
    results are multiplied by its sigmoid.  a may be float32 beside bfloat16 weights."""
    heads, cols, depth = w.shape
    n = a.shape[0]
    _need(w.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == n
          and a.shape[1] >= (heads - 1) * a_head + depth
          and out.shape[1] >= (heads - 1) * out_head + cols,
          "heads_product: a [N, >= H a_head], w [H, cols, depth], out [N, >= H out_head]")
    if gate is not None:
        _need(gate.dtype == w.dtype and gate.stride(1) == 1 and gate.shape == (n, heads * cols),
              "heads_product: gate [N, H cols] of w's dtype")
    lib = library.load("latent")
    _check(lib.de_heads_product(_tag(a.dtype), _tag(w.dtype), _tag(out.dtype), a.data_ptr(),
                                a.stride(0), a_head, w.data_ptr(), out.data_ptr(), out.stride(0),
                                out_head, _ptr(gate), gate.stride(0) if gate is not None else 0,
                                n, heads, cols, depth, _stream()), "heads_product")


# ------------------------------------------------------------------------------- routed experts
SEGMENT, SEGMENT_TENSOR = 64, 128      # slots of a tile: CUDA-core products, tensor-core products


def experts_tiles(n: int, top: int, experts: int, segment: int = SEGMENT) -> int:
    """The most tiles of ``segment`` slots that the grouped (token, choice) pairs of n tokens
    take."""
    return int(library.load("experts").de_experts_tiles(n, top, experts, segment))


def experts_route(h: torch.Tensor, router: torch.Tensor, bias: torch.Tensor, top: int,
                  chosen: torch.Tensor, weight: torch.Tensor,
                  scoring: str = "chosen_logits") -> None:
    """chosen [N, top] (int32): the experts with the largest logits router h + bias (float32);
    weight [N, top] (float32): the softmax over those logits alone.  ``scoring``
    "corrected_scores": the scores are the softmax of router h over all outputs, the choice goes
    by score + bias, and the weights are the chosen scores as they are."""
    n, experts = h.shape[0], router.shape[0]
    _need(scoring in ("chosen_logits", "corrected_scores"), "experts_route: unknown scoring")
    _i32(chosen, "chosen")
    _need(h.stride(1) == 1 and router.dtype == bias.dtype == weight.dtype == torch.float32
          and router.is_contiguous() and router.shape[1] == h.shape[1] and bias.is_contiguous()
          and bias.shape == (experts,) and chosen.shape == weight.shape == (n, top)
          and weight.is_contiguous(), "experts_route: h [N, D], router float32 [E, D], bias [E]")
    lib = library.load("experts")
    _check(lib.de_experts_route(_tag(h.dtype), h.data_ptr(), h.stride(0), router.data_ptr(),
                                bias.data_ptr(), n, h.shape[1], experts, top,
                                int(scoring == "corrected_scores"), chosen.data_ptr(),
                                weight.data_ptr(), _stream()), "experts_route")


def experts_group(chosen: torch.Tensor, experts: int, pair_of: torch.Tensor,
                  tile_expert: torch.Tensor, slot_of: torch.Tensor,
                  segment: int = SEGMENT) -> None:
    """Sort the pairs by expert: pair_of [tiles * segment] (the pair in a slot, or -1),
    tile_expert [tiles] (or -1), slot_of [pairs]."""
    for t, name in ((chosen, "chosen"), (pair_of, "pair_of"), (tile_expert, "tile_expert"),
                    (slot_of, "slot_of")):
        _i32(t, name)
    tiles = tile_expert.shape[0]
    _need(pair_of.shape == (tiles * segment,) and slot_of.numel() == chosen.numel(),
          "experts_group: pair_of [tiles * segment], slot_of [pairs]")
    lib = library.load("experts")
    _check(lib.de_experts_group(chosen.data_ptr(), chosen.numel(), experts, tiles, segment,
                                pair_of.data_ptr(), tile_expert.data_ptr(), slot_of.data_ptr(),
                                _stream()), "experts_group")


def experts_up(h: torch.Tensor, up: torch.Tensor, pair_of: torch.Tensor,
               tile_expert: torch.Tensor, top: int, inner: torch.Tensor,
               act: "str | None") -> None:
    """inner[slot] = act(up[e] h[token of the slot's pair]); up [E, ff, D], inner [slots, ff];
    ``act`` None: the product as it is."""
    experts, ff, width = up.shape
    tiles = tile_expert.shape[0]
    _need(up.is_contiguous() and h.stride(1) == 1 and h.shape[1] == width and inner.is_contiguous()
          and inner.shape == (tiles * 64, ff) and h.dtype == up.dtype == inner.dtype
          and (act is None or act in ACTIVATIONS),
          "experts_up: h [N, D], up [E, ff, D], inner [slots, ff]")
    lib = library.load("experts")
    _check(lib.de_experts_up(_tag(h.dtype), h.data_ptr(), h.stride(0), up.data_ptr(),
                             pair_of.data_ptr(), tile_expert.data_ptr(), tiles, top, width, ff,
                             inner.data_ptr(), 5 if act is None else ACTIVATIONS[act],
                             _stream()), "experts_up")


def experts_down(inner: torch.Tensor, down: torch.Tensor, pair_of: torch.Tensor,
                 tile_expert: torch.Tensor, y: torch.Tensor) -> None:
    """y[pair] = down[e] inner[slot of the pair]; down [E, D, ff], y [pairs, D]."""
    experts, width, ff = down.shape
    tiles = tile_expert.shape[0]
    _need(down.is_contiguous() and inner.is_contiguous() and inner.shape == (tiles * 64, ff)
          and y.is_contiguous() and y.shape[1] == width and inner.dtype == down.dtype == y.dtype,
          "experts_down: inner [slots, ff], down [E, D, ff], y [pairs, D]")
    lib = library.load("experts")
    _check(lib.de_experts_down(_tag(inner.dtype), inner.data_ptr(), down.data_ptr(),
                               pair_of.data_ptr(), tile_expert.data_ptr(), tiles, width, ff,
                               y.data_ptr(), _stream()), "experts_down")


def experts_tensor_ok(h: torch.Tensor, up: torch.Tensor, pairs: int,
                      down: "torch.Tensor | None" = None) -> bool:
    """Whether the experts' products of this step go to the tensor cores (``experts_product``):
    bfloat16 and rows of whole 16-byte pieces.  Steps of few pairs go there too: their tiles of
    128 slots are mostly empty, but the products are bound by the experts' weights, which the
    kernel streams through TMA."""
    return (h.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and pairs >= TENSOR_PAIRS
            and up.shape[1] % 8 == 0 and up.shape[2] % 8 == 0
            and (down is None or down.shape[2] % 8 == 0))


TENSOR_PAIRS = 1


def experts_gather(h: torch.Tensor, pair_of: torch.Tensor, top: int, rows: torch.Tensor) -> None:
    """rows[slot] = h[token of the slot's pair], zeros for a slot without a pair."""
    _i32(pair_of, "pair_of")
    _need(h.stride(1) == 1 and rows.is_contiguous() and rows.dtype == h.dtype
          and rows.shape == (pair_of.shape[0], h.shape[1]), "experts_gather: rows [slots, D]")
    lib = library.load("experts")
    _check(lib.de_experts_gather(_tag(h.dtype), h.data_ptr(), h.stride(0), pair_of.data_ptr(),
                                 pair_of.shape[0], top, h.shape[1], rows.data_ptr(), _stream()),
           "experts_gather")


def experts_product(rows: torch.Tensor, w: torch.Tensor, pair_of: torch.Tensor,
                    tile_expert: torch.Tensor, out: torch.Tensor, scatter: bool,
                    act: "str | None", status: torch.Tensor) -> None:
    """The experts' products on the 5th-generation tensor cores (the grouped form of
    ``csrc/gemm_tcgen05.cu``): rows [tiles * 128, k] slots sorted by expert, w [E, n, k];
    out[slot] (``scatter``: out[pair of the slot]) = act(w[expert of the slot's tile] rows[slot])
    for the slots that hold a pair.  bfloat16."""
    experts, n_out, k = w.shape
    tiles = tile_expert.shape[0]
    _need(rows.dtype == w.dtype == out.dtype == torch.bfloat16 and rows.is_contiguous()
          and w.is_contiguous() and out.is_contiguous() and rows.shape == (tiles * 128, k)
          and pair_of.shape == (tiles * 128,) and out.shape[1] == n_out
          and (scatter or out.shape[0] == tiles * 128) and (act is None or act in ACTIVATIONS),
          "experts_product: rows [tiles * 128, k], w [E, n, k], out [.., n], bfloat16")
    lib = library.load("gemm_tcgen05")
    _check(lib.de_gemm_tcgen05_grouped(rows.data_ptr(), rows.stride(0), w.data_ptr(),
                                       out.data_ptr(), out.stride(0), tile_expert.data_ptr(),
                                       pair_of.data_ptr(), tiles, experts, n_out, k,
                                       1 if scatter else 0, -1 if act is None else ACTIVATIONS[act],
                                       status.data_ptr(), _stream()), "experts_product")


def experts_combine(y: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                    hands_on: "tuple | None" = None) -> None:
    """out[n] = sum_k weight[n, k] * y[n * top + k] in float32; out float32 [N, D].
    ``hands_on`` = (chosen [N, top], experts, h [N, D]): a pair whose choice is not below
    ``experts`` has no row in y; it adds weight * h[n]."""
    n, top = weight.shape
    extra = (None, 0, None, 0)
    if hands_on is not None:
        chosen, experts, h = hands_on
        _i32(chosen, "chosen")
        _need(chosen.shape == (n, top) and h.dtype == y.dtype and h.stride(1) == 1
              and h.shape == (n, out.shape[1]), "experts_combine: chosen [N, top], h [N, D]")
        extra = (chosen.data_ptr(), int(experts), h.data_ptr(), h.stride(0))
    _need(y.is_contiguous() and y.shape == (n * top, out.shape[1]) and out.is_contiguous()
          and out.dtype == weight.dtype == torch.float32 and out.shape[0] == n
          and weight.is_contiguous(), "experts_combine: y [N top, D], weight [N, top], out [N, D]")
    lib = library.load("experts")
    _check(lib.de_experts_combine(_tag(y.dtype), y.data_ptr(), weight.data_ptr(), n, top,
                                  out.shape[1], out.data_ptr(), *extra, _stream()),
           "experts_combine")
