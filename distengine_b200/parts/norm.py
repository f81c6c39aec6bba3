"""RMS norm with the residual sum folded in, optionally in groups; layer norm with weight and bias.

Formula (src/layers/layernorm.py:12-23): float32 mean of squares, x * rsqrt(mean + eps), cast to
the activation dtype, then times the weight.  The block's residual sums
(src/models/llama.py:74-89) happen in the same kernel, in 32-bit.

``groups`` > 1: the row is cut into that many equal consecutive parts and each part is divided by
its own root mean square; the weight still spans the row.  ``tensor``: the local name of the
weight (architectures differ in it).

``layernorm``: (x - mean) / sqrt(mean of squared deviations + eps) * weight + bias, the statistics
in float32 over the whole row; ``tensor`` and ``bias`` are the local names of its two vectors.  The
mean does not commute with a matrix product, so this norm never rides on the products around it.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, register_norm, stored_vector
from .context import NormAhead, ResidualStream, StepContext


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device: torch.device,
                 groups: int = 1, tensor: str = "weight") -> None:
        super().__init__(dtype, device)
        if groups <= 0 or width % groups:
            raise ValueError(f"rmsnorm: groups ({groups}) must divide the width ({width})")
        self.width, self.eps, self.groups, self.tensor = width, eps, groups, tensor
        self.weight: "torch.Tensor | None" = None

    def tensors(self):
        return {self.tensor: ((self.width,), "vector")}

    def load(self, tensors):
        self.weight = stored_vector(tensors[self.tensor], self.dtype, self.device)

    def ahead(self, stream: ResidualStream, ctx: StepContext, count: int):
        if (self.weight.dtype != torch.bfloat16 or stream.pending is not None
                or self.groups != 1):
            return None
        n = stream.resid.shape[0]
        return NormAhead(self, stream.resid, self.weight, self.eps,
                         ctx.buffer("norm.out", (n, self.width)),
                         ctx.buffer("norm.parts", (n, count), torch.float32))

    def forward(self, stream: ResidualStream, ctx: StepContext, rows=None,
                out_name: str = "norm.out") -> torch.Tensor:
        if stream.ahead is not None:
            raise RuntimeError("this norm's work was handed to the product before it: its "
                               "result is stream.ahead.result()")
        n_out = stream.resid.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (n_out, self.width))
        ops.add_rmsnorm(stream.resid, stream.pending, self.weight, self.eps, out, rows,
                        groups=self.groups)
        if rows is None:
            stream.pending = None              # it is part of the residual now
        return out


    def normalize_stream(self, stream: ResidualStream, ctx: StepContext) -> None:
        """The stream itself becomes its norm (float32, in place): the norm of the embedding
        rows.  Its rounding to the activation dtype is left in ``stream.rows``."""
        if self.groups != 1 or stream.pending is not None or stream.ahead is not None:
            raise RuntimeError("rmsnorm: the stream is normed in place over whole rows, with "
                               "nothing pending")
        rows = None
        if self.dtype != torch.float32:
            rows = ctx.buffer("norm.stream_rows", tuple(stream.resid.shape))
        ops.norm_stream(stream.resid, self.weight, self.eps, rows)
        stream.rows = rows


class LayerNorm(Norm):
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device: torch.device,
                 tensor: str = "weight", bias: str = "bias") -> None:
        super().__init__(dtype, device)
        self.width, self.eps, self.tensor, self.bias_name = width, eps, tensor, bias
        self.weight: "torch.Tensor | None" = None
        self.bias: "torch.Tensor | None" = None

    def tensors(self):
        return {self.tensor: ((self.width,), "vector"), self.bias_name: ((self.width,), "bias")}

    def load(self, tensors):
        self.weight = stored_vector(tensors[self.tensor], self.dtype, self.device)
        self.bias = stored_vector(tensors[self.bias_name], self.dtype, self.device)
        if self.bias.dtype != self.weight.dtype:
            self.bias = self.bias.to(self.weight.dtype)

    def forward(self, stream: ResidualStream, ctx: StepContext, rows=None,
                out_name: str = "norm.out") -> torch.Tensor:
        if stream.ahead is not None:
            raise RuntimeError("a layer norm's work cannot be handed to the product before it")
        n_out = stream.resid.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (n_out, self.width))
        ops.add_layernorm(stream.resid, stream.pending, self.weight, self.bias, self.eps, out, rows)
        if rows is None:
            stream.pending = None              # it is part of the residual now
        return out


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
