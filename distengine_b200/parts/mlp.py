"""Dense gated feed-forward: down( act(gate(x)) * up(x) ), no biases; act is silu (SwiGLU,
fused into the products) or any other of ``ops.ACTIVATIONS`` (a kernel after the product)
(src/models/llama.py:13-29, src/layers/activation.py:6-9).  gate and up are one product against
the stacked matrix [2 inner, width]; the reference runs two and concatenates (llama.py:23-26).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, compute_matrix, register_feed_forward
from .context import NormAhead, StepContext, UnscaledRows


class GatedMLP(FeedForward):
    def __init__(self, width: int, inner: int, activation: str, dtype: torch.dtype,
                 device: torch.device,
                 names: "tuple[str, str, str]" = ("gate_proj.weight", "up_proj.weight",
                                                  "down_proj.weight")) -> None:
        """``names``: the local names of the gate, up and down matrices."""
        super().__init__(dtype, device)
        self.names = tuple(names)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated_mlp: activation '{activation}' is not implemented; "
                             f"{sorted(ops.ACTIVATIONS)} are")
        self.width, self.inner, self.activation = width, inner, activation
        self.w_gate_up: "torch.Tensor | None" = None
        self.w_down: "torch.Tensor | None" = None

    def tensors(self):
        gate, up, down = self.names
        return {gate: ((self.inner, self.width), "matrix"),
                up: ((self.inner, self.width), "matrix"),
                down: ((self.width, self.inner), "matrix")}

    def load(self, tensors):
        gate, up, down = self.names
        stacked = torch.cat((tensors[gate], tensors[up]), dim=0)
        self.w_gate_up = compute_matrix(stacked, self.dtype, self.device)
        self.w_down = compute_matrix(tensors[down], self.dtype, self.device)

    def takes_unscaled(self, n_rows: int) -> bool:
        # the products' fused gate is the silu one
        return (self.activation == "silu"
                and ops.norm_ride_parts(n_rows, self.w_gate_up, self.dtype) > 0)

    def ahead_parts(self, n_rows: int) -> int:
        return ops.norm_ride_parts(n_rows, self.w_down, self.dtype)

    def forward(self, x: "torch.Tensor | UnscaledRows", ctx: StepContext,
                ahead: "NormAhead | None" = None) -> "torch.Tensor | None":
        before = None
        if isinstance(x, UnscaledRows):
            before, x = x, x.rows
        n = x.shape[0]
        act = ctx.buffer("mlp.act", (n, self.inner))
        scratch = None
        if self.activation != "silu":
            # another gate than the products' own: the product, then the gate as a kernel
            scratch = ctx.buffer("mlp.gate_up", (n, 2 * self.inner))
            ops.linear(x, self.w_gate_up, out=scratch, status=ctx.status)
            ops.act_mul(scratch, act, self.activation)
        else:
            if before is None and ops.gated_needs_scratch(x, self.w_gate_up):
                scratch = ctx.buffer("mlp.gate_up", (n, 2 * self.inner))
            ops.linear_gated(x, self.w_gate_up, act, scratch, status=ctx.status, before=before)
        if ahead is not None:          # the product joins the residual and does the next norm's work
            ops.linear(act, self.w_down, out=ahead.rows, status=ctx.status, after=ahead)
            return None
        out = ctx.buffer("mlp.out", (n, self.width))
        ops.linear(act, self.w_down, out=out, status=ctx.status)
        return out


class DenseMLP(FeedForward):
    """down( act( up(x) ) ) without a gate; ``activation`` is one of ``ops.ACTIVATIONS`` (the
    square of relu, tanh, silu, gelu in its tanh form)."""

    def __init__(self, width: int, inner: int, activation: str, dtype: torch.dtype,
                 device: torch.device, names: "tuple[str, str]" = ("up", "down")) -> None:
        super().__init__(dtype, device)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense_mlp: activation '{activation}' is not implemented; "
                             f"{sorted(ops.ACTIVATIONS)} are")
        self.width, self.inner, self.activation, self.names = width, inner, activation, tuple(names)
        self.w_up: "torch.Tensor | None" = None
        self.w_down: "torch.Tensor | None" = None

    def tensors(self):
        up, down = self.names
        return {up: ((self.inner, self.width), "matrix"), down: ((self.width, self.inner), "matrix")}

    def load(self, tensors):
        up, down = self.names
        self.w_up = compute_matrix(tensors[up], self.dtype, self.device)
        self.w_down = compute_matrix(tensors[down], self.dtype, self.device)

    def forward(self, x: torch.Tensor, ctx: StepContext, ahead=None) -> torch.Tensor:
        n = x.shape[0]
        act = ctx.buffer("mlp.act", (n, self.inner))
        ops.linear(x, self.w_up, out=act, status=ctx.status, act=self.activation)
        out = ctx.buffer("mlp.out", (n, self.width))
        ops.linear(act, self.w_down, out=out, status=ctx.status)
        return out


class PolyNormMLP(FeedForward):
    """down( P( up(x) ) ) whose activation is a learned cubic of normed powers: with N dividing a
    token's vector of inner values by its root mean square (eps inside the root),
    P(z) = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element; (a, b, c, e) are the four
    numbers of the tensor ``coefficients``.  The statistics and the sum are float32."""

    def __init__(self, width: int, inner: int, eps: float, dtype: torch.dtype,
                 device: torch.device, names: "tuple[str, str]" = ("up", "down"),
                 coefficients: str = "act") -> None:
        super().__init__(dtype, device)
        self.width, self.inner, self.eps = width, inner, float(eps)
        self.names, self.coefficients = tuple(names), coefficients
        self.w_up = self.w_down = self.coef = None

    def tensors(self):
        up, down = self.names
        return {up: ((self.inner, self.width), "matrix"), down: ((self.width, self.inner), "matrix"),
                self.coefficients: ((4,), "vector")}

    def load(self, tensors):
        up, down = self.names
        self._host_up = tensors[up]
        self.w_up = None
        self.w_down = compute_matrix(tensors[down], self.dtype, self.device)
        self.coef = tensors[self.coefficients].to(device=self.device,
                                                  dtype=torch.float32).contiguous()

    def kernel_modules(self):
        return ("sublayer",)

    # all this part takes from its input is the up product: whoever owns a wider product stacks
    # ``input_matrix()`` into it and calls ``run`` on that product's rows (row stride free)
    def input_matrix(self) -> torch.Tensor:
        return self._host_up

    def finish_load(self) -> None:
        self._host_up = None

    def forward(self, x: torch.Tensor, ctx: StepContext, ahead=None) -> torch.Tensor:
        if self.w_up is None:
            self.w_up = compute_matrix(self._host_up, self.dtype, self.device)
            self.finish_load()
        z = ctx.buffer("mlp.up", (x.shape[0], self.inner))
        ops.linear(x, self.w_up, out=z, status=ctx.status)
        return self.run(z, ctx)

    def run(self, proj: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n, z = proj.shape[0], proj[:, : self.inner]
        act = ctx.buffer("mlp.act", (n, self.inner))
        ops.poly_norm(z, self.coef, self.eps, act)
        out = ctx.buffer("mlp.out", (n, self.width))
        ops.linear(act, self.w_down, out=out, status=ctx.status)
        return out


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("dense_mlp", DenseMLP)
register_feed_forward("polynorm_mlp", PolyNormMLP)
