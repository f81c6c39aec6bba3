"""Routed experts: a feed-forward whose tokens each go through the ``top`` of ``experts`` small
layers down_e(act(up_e x)) (no gate, no biases) that a router picks.

    z = W_router x + b            float32
    the ``top`` largest z are chosen; their weights are the softmax over the chosen z alone
    out = sum over the chosen e of weight_e * W_down_e act(W_up_e x)      summed in float32

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
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype, device)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"routed_experts: activation '{activation}' is not implemented; "
                             f"{sorted(ops.ACTIVATIONS)} are")
        if not 0 < top <= experts or top > 32:
            raise ValueError(f"routed_experts: top ({top}) must be from 1 to the number of "
                             f"experts ({experts}) and at most 32")
        self.width, self.inner, self.experts, self.top = width, inner, experts, top
        self.activation = activation
        self.router = self.bias = self.up = self.down = None

    def tensors(self):
        out = {"router": ((self.experts, self.width), "matrix"),
               "router.b": ((self.experts,), "vector")}
        for e in range(self.experts):
            out[f"e{e}.up"] = ((self.inner, self.width), "matrix")
            out[f"e{e}.down"] = ((self.width, self.inner), "matrix")
        return out

    def load(self, tensors):
        self.router = tensors["router"].to(device=self.device, dtype=torch.float32).contiguous()
        self.bias = tensors["router.b"].to(device=self.device, dtype=torch.float32).contiguous()
        self.up = compute_matrix(torch.stack([tensors[f"e{e}.up"] for e in range(self.experts)]),
                                 self.dtype, self.device)
        self.down = compute_matrix(
            torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]), self.dtype,
            self.device)

    def kernel_modules(self):
        return ("experts", "gemm_tcgen05") if self.dtype == torch.bfloat16 else ("experts",)

    def forward(self, x: torch.Tensor, ctx: StepContext, ahead=None) -> torch.Tensor:
        n, top = x.shape[0], self.top
        tensor = lk.experts_tensor_ok(x, self.up, n * top)
        segment = lk.SEGMENT_TENSOR if tensor else lk.SEGMENT
        tiles = lk.experts_tiles(n, top, self.experts, segment)
        chosen = ctx.buffer("experts.chosen", (n, top), torch.int32)
        weight = ctx.buffer("experts.weight", (n, top), torch.float32)
        pair_of = ctx.buffer("experts.pair_of", (tiles * segment,), torch.int32)
        tile_expert = ctx.buffer("experts.tile_expert", (tiles,), torch.int32)
        slot_of = ctx.buffer("experts.slot_of", (n * top,), torch.int32)
        lk.experts_route(x, self.router, self.bias, top, chosen, weight)
        lk.experts_group(chosen, self.experts, pair_of, tile_expert, slot_of, segment)
        inner = ctx.buffer("experts.inner", (tiles * segment, self.inner))
        y = ctx.buffer("experts.y", (n * top, self.width))
        if tensor:
            rows = ctx.buffer("experts.rows", (tiles * segment, self.width))
            lk.experts_gather(x, pair_of, top, rows)
            lk.experts_product(rows, self.up, pair_of, tile_expert, inner, False,
                               self.activation, ctx.status)
            lk.experts_product(inner, self.down, pair_of, tile_expert, y, True, None, ctx.status)
        else:
            lk.experts_up(x, self.up, pair_of, tile_expert, top, inner, self.activation)
            lk.experts_down(inner, self.down, pair_of, tile_expert, y)
        out = ctx.buffer("experts.out", (n, self.width), torch.float32)
        lk.experts_combine(y, weight, out)
        return out


register_feed_forward("routed_experts", RoutedExperts)
