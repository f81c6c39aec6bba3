"""Pre-norm block: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/llama.py:66-89).  The sums are carried as the stream's pending branch and folded in
by the next norm.  A layer without a feed-forward is the first half only.

``parallel_norms``: both branches read the same x (see ``ParallelNormsBlock``).

``sublayer_norm``: the norm stands on a sublayer's output, the sublayers read x itself, with an
optional gate on every sublayer's result and an optional average over the depth (see
``SublayerNormBlock``)."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, Part, register_block
from .context import CacheBinding, ResidualStream, StepContext


class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following=None) -> None:
        h = _normed(self.mixer_norm, stream, ctx)
        if self.feed_forward is None:
            ahead = None
            if following is not None:
                ahead = _ahead(self.mixer, following[0], following[1], stream, ctx)
        else:
            ahead = _ahead(self.mixer, self.feed_forward_norm, self.feed_forward, stream, ctx)
        if ahead is None:
            stream.pending = self.mixer.forward(h, ctx, cache)
        else:
            self.mixer.forward(h, ctx, cache, ahead=ahead)
            stream.ahead = ahead
        if self.feed_forward is None:
            return
        h = _normed(self.feed_forward_norm, stream, ctx)
        ahead = None
        if following is not None:
            ahead = _ahead(self.feed_forward, following[0], following[1], stream, ctx)
        if ahead is None:
            stream.pending = self.feed_forward.forward(h, ctx)
        else:
            self.feed_forward.forward(h, ctx, ahead=ahead)
            stream.ahead = ahead


def _normed(norm, stream: ResidualStream, ctx: StepContext):
    """The norm's output, from the product before it if that did the work."""
    ahead, stream.ahead = stream.ahead, None
    if ahead is None:
        return norm.forward(stream, ctx)
    if ahead.norm is not norm:
        raise RuntimeError("the stream holds another norm's work than the one that runs next")
    return ahead.result()


def _ahead(producer, norm, consumer, stream: ResidualStream, ctx: StepContext):
    """Buffers for ``producer``'s last product to do ``norm``'s work, if producer, norm and
    ``consumer`` (which must take rows without their factors) all can for this step."""
    n = stream.resid.shape[0]
    abilities = (getattr(producer, "ahead_parts", None), getattr(consumer, "takes_unscaled", None))
    if None in abilities:
        return None
    count = abilities[0](n)
    if not count or not abilities[1](n):
        return None
    return norm.ahead(stream, ctx, count)


register_block("prenorm", PreNormBlock)


class ParallelNormsBlock(Block):
    """Two branches of the same input, each behind a norm of its own:
    x += mixer(norm1(x)) + feed_forward(norm2(x)), the three terms summed in float32; then the
    layer's side input, if it has one, reads the new x and adds to it.  A layer without a
    feed-forward is x += mixer(norm1(x))."""

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following=None) -> None:
        if stream.ahead is not None:
            raise RuntimeError("a block of parallel branches runs its norms itself")
        h = self.mixer_norm.forward(stream, ctx)            # also folds what was pending
        h2 = None
        if self.feed_forward is not None:
            h2 = self.feed_forward_norm.forward(stream, ctx, out_name="norm.out.second")
        a = self.mixer.forward(h, ctx, cache)
        b = self.feed_forward.forward(h2, ctx) if self.feed_forward is not None else None
        if self.side_input is None:
            ops.residual_add(stream.resid, a, b)
            return
        rows = ctx.buffer("block.rows", tuple(stream.resid.shape))
        ops.residual_add(stream.resid, a, b, rows=rows)
        self.side_input.forward(stream, rows, ctx)


register_block("parallel_norms", ParallelNormsBlock)


class ResidualGate(Part):
    """sigmoid(W x + b) on a sublayer's result, W [width, width] and b [width] under the names
    "" and ".b" of the part's prefix.  The block runs the product on the sublayer's input and
    hands the rest to the kernel that also norms and adds."""

    def __init__(self, width: int, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype, device)
        self.width = width
        self._host = self._weight = self.bias = None

    def tensors(self):
        return {"": ((self.width, self.width), "matrix"), ".b": ((self.width,), "bias")}

    def load(self, tensors):
        self._host = tensors[""]                 # until it is known who multiplies with it
        self._weight = None
        self.bias = tensors[".b"].to(device=self.device, dtype=torch.float32).contiguous()

    def host_matrix(self) -> torch.Tensor:
        """The matrix on the host (stored dtype), for a sublayer that stacks it under its own
        input matrix; afterwards call ``stacked()``."""
        return self._host

    def stacked(self) -> None:
        self._host = None

    @property
    def weight(self) -> torch.Tensor:
        if self._weight is None:
            self._weight = self._host.to(device=self.device, dtype=self.dtype).contiguous()
            self._host = None
        return self._weight

    def kernel_modules(self):
        return ("sublayer",)


class DepthMix(Part):
    """The learned weights c [count] with which the stream that leaves a layer is mixed from the
    embedding rows and every layer's result so far, x = sum_j c[j] X_j."""

    def __init__(self, count: int, dtype: torch.dtype, device: torch.device,
                 tensor: str = "dwa") -> None:
        super().__init__(dtype, device)
        self.count, self.tensor = count, tensor
        self.coef = None

    def tensors(self):
        return {self.tensor: ((self.count,), "vector")}

    def load(self, tensors):
        self.coef = tensors[self.tensor].to(device=self.device, dtype=torch.float32).contiguous()

    def kernel_modules(self):
        return ("sublayer",)


class SublayerNormBlock(Block):
    """x <- x + norm1(mixer(x)); x <- x + norm2(feed_forward(x)): the sublayers read the stream
    itself (its rounding to the activation dtype), the RMS norms stand on their results.

    ``gated``: a sublayer's result is first multiplied by sigmoid(W x + b) of the same input x
    (``ResidualGate``; roles "mixer_gate" and "feed_forward_gate").  ``depth``: the layer's result
    X_(i+1) is kept beside the embedding rows X_0 and the earlier layers' results, and what goes on
    to the next layer is sum_j c[j] X_j over all ``depth`` of them (``DepthMix``, role
    "depth_mix"); 0: the layer's result goes on as it is.

    Gate, norm and sum are one kernel a sublayer, float32 throughout; it also leaves the new
    stream's rounding for the next products (``stream.rows``).  A layer without a feed-forward is
    the first half only.

    A sublayer whose only use of its input is one product (it has ``input_matrix()`` and
    ``run(proj, ...)``, as the projected mixers have) shares that product with its gate: the
    gate's matrix is stacked under the sublayer's, so the input is read once and a sublayer
    has one launch less."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, side_input=None,
                 gated: bool = False, depth: int = 0) -> None:
        super().__init__(mixer, feed_forward, mixer_norm, feed_forward_norm, side_input)
        if side_input is not None:
            raise ValueError("sublayer_norm: this arrangement takes no side input")
        for norm in (mixer_norm, feed_forward_norm):
            if norm is not None and (getattr(norm, "groups", 1) != 1
                                     or not hasattr(norm, "eps") or hasattr(norm, "bias")):
                raise ValueError("sublayer_norm: the norms on the sublayers' results are RMS "
                                 "norms over the whole row")
        width, dtype, device = mixer_norm.width, mixer.dtype, mixer.device
        self.mixer_gate = ResidualGate(width, dtype, device) if gated else None
        self.feed_forward_gate = (ResidualGate(width, dtype, device)
                                  if gated and feed_forward is not None else None)
        self.depth_mix = DepthMix(depth, dtype, device) if depth else None
        self._stacks: dict = {}      # role -> (the sublayer's and the gate's matrices, gate column)

    def history_depth(self) -> int:
        return self.depth_mix.count if self.depth_mix is not None else 0

    def parts(self):
        parts = super().parts()
        for role in ("mixer_gate", "feed_forward_gate", "depth_mix"):
            if getattr(self, role) is not None:
                parts[role] = getattr(self, role)
        return parts

    def _sublayer(self, role, part, gate, h, ctx, cache=None):
        """(the sublayer's result, the gate's product on the same input h)."""
        if gate is None:
            raise NotImplementedError("sublayer_norm: only the gated form has a kernel")
        n = h.shape[0]
        if hasattr(part, "input_matrix") and hasattr(part, "run"):
            stack = self._stacks.get(role)
            if stack is None:
                from .base import compute_matrix
                from .recurrent import stack_segments
                both, offsets = stack_segments([part.input_matrix(), gate.host_matrix()])
                stack = self._stacks[role] = (compute_matrix(both, part.dtype, part.device),
                                              offsets[1])
                part.finish_load()
                gate.stacked()
            w_in, col = stack
            proj = ctx.buffer(f"block.{role}.proj", (n, w_in.shape[0]))
            ops.linear(h, w_in, out=proj, status=ctx.status)
            y = part.run(proj, ctx, cache) if role == "mixer" else part.run(proj, ctx)
            return y, proj[:, col: col + gate.width]
        y = part.forward(h, ctx, cache) if role == "mixer" else part.forward(h, ctx)
        z = ctx.buffer("block.gate", (n, gate.width))
        ops.linear(h, gate.weight, out=z, status=ctx.status)
        return y, z

    def _join(self, y, z, gate, norm, stream, ctx, out, rows):
        """out = stream + norm(y * sigmoid(z + b)); ``rows``: where its rounding goes (or
        None)."""
        ops.gated_normed_add(y, z, gate.bias, norm.weight, norm.eps, stream.resid, out, rows)

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following=None) -> None:
        if stream.ahead is not None or stream.pending is not None:
            raise RuntimeError("a block whose sublayers read the stream itself takes a stream "
                               "with nothing pending")
        resid = stream.resid
        wide = ctx.dtype == torch.float32
        shape = tuple(resid.shape)
        rows = None if wide else ctx.buffer("block.rows", shape)
        h = resid if wide else stream.rows
        if h is None:                                  # the stream came without its rounding
            h = rows
            h.copy_(resid)
        result = resid
        if self.depth_mix is not None:
            if stream.history is None or stream.history.shape[0] < self.depth_mix.count:
                raise RuntimeError("the model keeps no history of the stream for this layer "
                                   "(Block.history_depth)")
            if stream.history_count + 1 != self.depth_mix.count:
                raise RuntimeError(f"this layer mixes {self.depth_mix.count} states of the "
                                   f"stream, {stream.history_count + 1} exist")
            result = stream.history[self.depth_mix.count - 1]
        last = self.feed_forward is None
        y, z = self._sublayer("mixer", self.mixer, self.mixer_gate, h, ctx, cache)
        self._join(y, z, self.mixer_gate, self.mixer_norm, stream, ctx,
                   result if last else resid, None if (last and self.depth_mix) else rows)
        if not last:
            h = resid if wide else rows
            y, z = self._sublayer("feed_forward", self.feed_forward, self.feed_forward_gate, h,
                                  ctx)
            self._join(y, z, self.feed_forward_gate, self.feed_forward_norm, stream, ctx, result,
                       None if self.depth_mix else rows)
        if self.depth_mix is not None:
            stream.history_count += 1
            ops.depth_mix(stream.history[: self.depth_mix.count], self.depth_mix.coef, resid, rows)
        stream.rows = rows


register_block("sublayer_norm", SublayerNormBlock)
