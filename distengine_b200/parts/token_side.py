"""A side input from the token itself: after a layer's branches, a row of a table that the token
picks gates a small projection of the stream, and the result joins the stream behind a norm.

    e = table[token][index * dim : (index + 1) * dim]      the table holds every layer's part
    g = gelu_tanh(W_gate x) * e ;  y = W_proj g
    x <- x + y / sqrt(mean(y^2) + eps) * norm              in float32

``table``: the tensor's name ("/..." for a table that all layers share); ``index``: which part of
its rows is this layer's (a layer that runs several times uses the same part every time).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import SideInput, compute_matrix, register_side_input, stored_vector
from .context import ResidualStream, StepContext


class TokenSide(SideInput):
    def __init__(self, width: int, dim: int, index: int, layers: int, vocabulary: int, eps: float,
                 dtype: torch.dtype, device: torch.device, table: str = "/side.embed",
                 activation: str = "gelu_tanh") -> None:
        super().__init__(dtype, device)
        if not 0 <= index < layers:
            raise ValueError(f"token_side: index {index} is not one of the table's {layers} parts")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"token_side: unknown activation '{activation}'")
        self.width, self.dim, self.index, self.layers = width, dim, index, layers
        self.vocabulary, self.eps, self.table_name, self.activation = (vocabulary, eps, table,
                                                                       activation)
        self.table = self.w_gate = self.w_proj = self.norm = None

    def tensors(self):
        return {self.table_name: ((self.vocabulary, self.layers * self.dim), "matrix"),
                "gate": ((self.dim, self.width), "matrix"),
                "proj": ((self.width, self.dim), "matrix"),
                "norm": ((self.width,), "vector")}

    def load(self, tensors):
        part = tensors[self.table_name][:, self.index * self.dim: (self.index + 1) * self.dim]
        self.table = compute_matrix(part, self.dtype, self.device)
        self.w_gate = compute_matrix(tensors["gate"], self.dtype, self.device)
        self.w_proj = compute_matrix(tensors["proj"], self.dtype, self.device)
        self.norm = stored_vector(tensors["norm"], self.dtype, self.device)

    def forward(self, stream: ResidualStream, rows: torch.Tensor, ctx: StepContext) -> None:
        n = rows.shape[0]
        z = ctx.buffer("token_side.z", (n, self.dim))
        ops.linear(rows, self.w_gate, out=z, status=ctx.status)
        ops.act_mul_row(z, ctx.token_ids, self.table, z, self.activation)
        y = ctx.buffer("token_side.y", (n, self.width))
        ops.linear(z, self.w_proj, out=y, status=ctx.status)
        ops.add_normed(stream.resid, y, self.norm, self.eps)


register_side_input("token_side", TokenSide)
