"""Routed experts: a feed-forward whose tokens each go through the ``top`` of ``experts`` small
layers down_e(act(up_e x)) (no gate, no biases) that a router picks.

    z = W_router x + b            float32
    the ``top`` largest z are chosen; their weights are the softmax over the chosen z alone
    out = sum over the chosen e of weight_e * W_down_e act(W_up_e x)      summed in float32

Parameters widen this.  ``gated``: an expert is W_down (act(W_gate x) * W_up x); its gate and up
rows are stacked into one product and joined by a kernel after it.  ``scoring``
"corrected_scores": s = softmax(z) over all router outputs (no bias on z), the choice goes by
s + correction (the tensor ``bias_name``), the weights are the chosen s themselves, not
renormalised.  ``identity`` > 0: the router has that many outputs more than there are experts; they
stand for experts that hand their input on, weight * x, and have no tensors.

The experts' matrices are stacked ([E, inner, width] and [E, width, inner]); the (token, choice)
pairs are sorted by expert on the device into tiles of slots of one expert each.  A step of few
pairs, and every float32 step, runs a tile of 64 slots as one block's product on the CUDA cores
(``csrc/experts.cu``); a bfloat16 step of many pairs gathers its rows by slot and runs tiles of
128 slots on the tensor cores (the grouped form of ``csrc/gemm_tcgen05.cu``, the activation in
its epilogue, the down product scattering its rows to their pairs).  The output is float32: it
joins the residual stream unrounded.
"""

from __future__ import annotations

import torch

from ..kernels import latent as lk
from ..kernels import ops
from .base import FeedForward, compute_matrix, register_feed_forward
from .context import StepContext


class RoutedExperts(FeedForward):
    def __init__(self, width: int, inner: int, experts: int, top: int, activation: str,
                 dtype: torch.dtype, device: torch.device, gated: bool = False,
                 scoring: str = "chosen_logits", identity: int = 0,
                 bias_name: str = "router.b") -> None:
        super().__init__(dtype, device)
        if scoring not in ("chosen_logits", "corrected_scores") or identity < 0:
            raise ValueError("routed_experts: scoring is 'chosen_logits' or 'corrected_scores', "
                             "identity >= 0")
        self.gated, self.scoring, self.identity, self.bias_name = gated, scoring, identity, bias_name
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"routed_experts: activation '{activation}' is not implemented; "
                             f"{sorted(ops.ACTIVATIONS)} are")
        if not 0 < top <= experts + identity or top > 32 or experts <= 0:
            raise ValueError(f"routed_experts: top ({top}) must be from 1 to the number of "
                             f"router outputs ({experts + identity}) and at most 32")
        self.width, self.inner, self.experts, self.top = width, inner, experts, top
        self.activation = activation
        self.router = self.bias = self.up = self.down = None

    def tensors(self):
        outputs = self.experts + self.identity
        out = {"router": ((outputs, self.width), "matrix"),
               self.bias_name: ((outputs,), "bias" if self.identity or self.gated else "vector")}
        for e in range(self.experts):
            if self.gated:
                out[f"e{e}.gate"] = ((self.inner, self.width), "matrix")
            out[f"e{e}.up"] = ((self.inner, self.width), "matrix")
            out[f"e{e}.down"] = ((self.width, self.inner), "matrix")
        return out

    def load(self, tensors):
        self.router = tensors["router"].to(device=self.device, dtype=torch.float32).contiguous()
        self.bias = tensors[self.bias_name].to(device=self.device,
                                               dtype=torch.float32).contiguous()
        ups = [tensors[f"e{e}.up"] for e in range(self.experts)]
        if self.gated:          # an expert's rows: [gate; up]
            ups = [torch.cat((tensors[f"e{e}.gate"], up), dim=0) for e, up in enumerate(ups)]
        self.up = compute_matrix(torch.stack(ups), self.dtype, self.device)
        self.down = compute_matrix(
            torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]), self.dtype,
            self.device)

    def kernel_modules(self):
        return ("experts", "gemm_tcgen05") if self.dtype == torch.bfloat16 else ("experts",)

    def forward(self, x: torch.Tensor, ctx: StepContext, ahead=None) -> torch.Tensor:
        n, top = x.shape[0], self.top
        tensor = lk.experts_tensor_ok(x, self.up, n * top, self.down)
        segment = lk.SEGMENT_TENSOR if tensor else lk.SEGMENT
        tiles = lk.experts_tiles(n, top, self.experts, segment)
        chosen = ctx.buffer("experts.chosen", (n, top), torch.int32)
        weight = ctx.buffer("experts.weight", (n, top), torch.float32)
        pair_of = ctx.buffer("experts.pair_of", (tiles * segment,), torch.int32)
        tile_expert = ctx.buffer("experts.tile_expert", (tiles,), torch.int32)
        slot_of = ctx.buffer("experts.slot_of", (n * top,), torch.int32)
        lk.experts_route(x, self.router, self.bias, top, chosen, weight, self.scoring)
        lk.experts_group(chosen, self.experts, pair_of, tile_expert, slot_of, segment)
        inner = ctx.buffer("experts.inner", (tiles * segment, self.inner))
        y = ctx.buffer("experts.y", (n * top, self.width))
        # a gated expert's first product has no activation: [gate | up], joined afterwards
        first = ctx.buffer("experts.gate_up", (tiles * segment, 2 * self.inner)) if self.gated \
            else inner
        first_act = None if self.gated else self.activation
        if tensor:
            rows = ctx.buffer("experts.rows", (tiles * segment, self.width))
            lk.experts_gather(x, pair_of, top, rows)
            lk.experts_product(rows, self.up, pair_of, tile_expert, first, False, first_act,
                               ctx.status)
        else:
            lk.experts_up(x, self.up, pair_of, tile_expert, top, first, first_act)
        if self.gated and self.activation == "silu":
            ops.silu_mul(first, inner)                     # the vectorised form
        elif self.gated:
            ops.act_mul(first, inner, self.activation)
        if tensor:
            lk.experts_product(inner, self.down, pair_of, tile_expert, y, True, None, ctx.status)
        else:
            lk.experts_down(inner, self.down, pair_of, tile_expert, y)
        out = ctx.buffer("experts.out", (n, self.width), torch.float32)
        lk.experts_combine(y, weight, out,
                           (chosen, self.experts, x) if self.identity else None)
        return out


register_feed_forward("routed_experts", RoutedExperts)
