"""The generic decoder: embedding, the blocks that the configuration's layer specs describe, run in
the order of its plan, final norm, output matrix.  Nothing in here is specific to one
architecture; an architecture is a configuration class (``config/``) plus one registry entry.

Reference counterpart: ``LlamaModel`` / ``LlamaForCausalLM`` (src/models/llama.py:92-217), whose
forward returns logits at all positions (:217); here only the wanted rows reach the output matrix.
"""

from __future__ import annotations

import torch

from ..config.model import LayerSpec, ModelConfig
from ..kernels import library, ops
from ..parts.base import (Block, PagedKVSpec, StateSpec, build_block, build_feed_forward,
                          build_mixer, build_norm, build_side_input, compute_matrix)
from ..parts.context import CacheBinding, ResidualStream, StepContext, StepPrep


def _layer_parts(spec: LayerSpec, dtype: torch.dtype, device: torch.device) -> Block:
    feed_forward = feed_forward_norm = None
    if spec.feed_forward is not None:
        feed_forward = build_feed_forward(spec.feed_forward, dtype, device)
        feed_forward_norm = build_norm(spec.feed_forward_norm or spec.norm, dtype, device)
    side_input = None
    if spec.side_input is not None:
        side_input = build_side_input(spec.side_input, dtype, device)
    return build_block(spec.block, build_mixer(spec.mixer, dtype, device), feed_forward,
                       build_norm(spec.norm, dtype, device), feed_forward_norm, side_input,
                       dict(spec.block_params))


def _full_name(prefix: str, local: str) -> str:
    """A part's tensor in the weight file: under the part's prefix, or, for a local name that
    starts with "/", the name behind the slash as it is."""
    return local[1:] if local.startswith("/") else prefix + local


class DecoderModel:
    def __init__(self, config: ModelConfig, dtype: torch.dtype,
                 device: "torch.device | str") -> None:
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        self.specs = config.layer_specs()
        self.plan = config.plan()
        for index, entry in enumerate(self.plan):
            if not 0 <= entry.layer < len(self.specs):
                raise ValueError(f"plan entry {index} names layer {entry.layer}, the model has "
                                 f"{len(self.specs)}")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < index:
                raise ValueError(f"plan entry {index} reads the cache of entry "
                                 f"{entry.reads_cache_of}, which does not run before it")
        self.blocks = [_layer_parts(spec, dtype, self.device) for spec in self.specs]
        self.final_norm = build_norm(config.final_norm(), dtype, self.device)
        first = config.embedding_norm()
        self.embedding_norm = None if first is None else build_norm(first, dtype, self.device)
        # the states of the stream that blocks read besides the stream itself
        self.history_depth = max((block.history_depth() for block in self.blocks), default=0)
        self.embedding: "torch.Tensor | None" = None
        self.output: "torch.Tensor | None" = None

    # ------------------------------------------------------------------ weights
    def expected_tensors(self):
        """(name -> shape, names that are vectors, names that may be absent)."""
        names = self.config.tensor_names()
        expected: dict[str, tuple[int, ...]] = {
            names["embedding"]: (self.config.vocabulary, self.config.width)}
        vectors: set[str] = set()
        for spec, block in zip(self.specs, self.blocks):
            for role, part in block.parts().items():
                for local, (shape, kind) in part.tensors().items():
                    full = _full_name(spec.prefix(role), local)
                    if expected.get(full, tuple(shape)) != tuple(shape):
                        raise ValueError(f"tensor '{full}' is expected in two shapes")
                    expected[full] = tuple(shape)
                    if kind == "vector":
                        vectors.add(full)
        outer = [(self.final_norm, names["final_norm"])]
        if self.embedding_norm is not None:
            outer.append((self.embedding_norm, names["embedding_norm"]))
        for norm, prefix in outer:
            for local, (shape, kind) in norm.tensors().items():
                expected[prefix + local] = tuple(shape)
                if kind == "vector":
                    vectors.add(prefix + local)
        expected[names["output"]] = (self.config.vocabulary, self.config.width)
        # a tied output needs no tensor of its own, unless it goes by the embedding's name
        optional = ({names["output"]} - {names["embedding"]}) if self.config.tied_output else set()
        return expected, vectors, optional

    def kernel_modules(self) -> "list[tuple[str, tuple]]":
        """The kernel libraries every step of this model uses: the row-wise kernels, the product
        of its dtype for steps of few tokens, and what its parts name."""
        modules = ["core", "gemm_f32" if self.dtype == torch.float32 else "linear_small"]
        if self.embedding_norm is not None:
            modules.append("sublayer")
        for block in self.blocks:
            for part in block.parts().values():
                for module in part.kernel_modules():
                    if module not in modules:
                        modules.append(module)
        # a part names a library, or (library, the definitions it is built with)
        return [module if isinstance(module, tuple) else (module, ()) for module in modules]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if self.device.type == "cuda":
            library.preload(self.kernel_modules())       # compiled side by side, if not yet
        names = self.config.tensor_names()
        self.embedding = compute_matrix(tensors[names["embedding"]], self.dtype, self.device)
        for spec, block in zip(self.specs, self.blocks):
            for role, part in block.parts().items():
                prefix = spec.prefix(role)
                part.load({local: tensors[_full_name(prefix, local)]
                           for local in part.tensors()})
        self.final_norm.load({local: tensors[names["final_norm"] + local]
                              for local in self.final_norm.tensors()})
        if self.embedding_norm is not None:
            self.embedding_norm.load({local: tensors[names["embedding_norm"] + local]
                                      for local in self.embedding_norm.tensors()})
        if names["output"] in tensors:
            self.output = compute_matrix(tensors[names["output"]], self.dtype, self.device)
        else:
            self.output = self.embedding          # tied: one matrix for both ends

    # ------------------------------------------------------------------ cache needs
    def cache_specs(self) -> "list[PagedKVSpec | StateSpec | None]":
        """For every plan entry what its run must be given: a cache of its own (a spec) or, when
        it reads an earlier entry's cache or its mixer keeps nothing, None."""
        out = []
        for entry in self.plan:
            spec = self.blocks[entry.layer].mixer.cache_spec()
            out.append(None if entry.reads_cache_of is not None else spec)
        for index, entry in enumerate(self.plan):
            if entry.reads_cache_of is not None:
                mine = self.blocks[entry.layer].mixer.cache_spec()
                theirs = self.blocks[self.plan[entry.reads_cache_of].layer].mixer.cache_spec()
                if self.plan[entry.reads_cache_of].reads_cache_of is not None or mine != theirs:
                    raise ValueError(f"plan entry {index} cannot read the cache of entry "
                                     f"{entry.reads_cache_of}: it needs {mine}, that entry "
                                     f"keeps {theirs}")
        return out

    # ------------------------------------------------------------------ step
    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for block in self.blocks for part in block.parts().values())

    def prepare(self, prep: StepPrep) -> None:
        for part in self._preparers():
            part.prepare(prep)

    def _preparers(self):
        """The parts whose ``prepare`` does something, one for each distinct plan key (layers of
        the same shape share their work lists); found once."""
        cached = getattr(self, "_preparer_list", None)
        if cached is None:
            from ..parts.base import Part
            cached, seen = [], set()
            for block in self.blocks:
                for part in block.parts().values():
                    if type(part).prepare is Part.prepare:
                        continue
                    key = getattr(part, "prepare_key", None)
                    if key is not None and key in seen:
                        continue
                    seen.add(key)
                    cached.append(part)
            self._preparer_list = cached
        return cached

    def forward(self, ctx: StepContext,
                caches: "list[CacheBinding | None]") -> torch.Tensor:
        """Run the step's tokens through the plan; logits float32 [R, vocabulary] at
        ``ctx.logit_rows``."""
        resid = ctx.buffer("model.residual", (ctx.n_tokens, self.config.width), torch.float32)
        ops.embed_rows(ctx.token_ids, self.embedding, resid, self.config.embedding_scale)
        stream = ResidualStream(resid)
        if self.embedding_norm is not None:
            self.embedding_norm.normalize_stream(stream, ctx)
        if self.history_depth:
            if len(self.plan) + 1 > self.history_depth:
                raise RuntimeError("the plan runs more layers than its blocks keep states for")
            stream.history = ctx.buffer("model.history", (self.history_depth, ctx.n_tokens,
                                                          self.config.width), torch.float32)
            stream.history[0].copy_(resid)
            stream.history_count = 1
        first = None
        if any(entry.adds_embedding for entry in self.plan):
            first = ctx.buffer("model.embedding", (ctx.n_tokens, self.config.width),
                               torch.float32)
            ops.embed_rows(ctx.token_ids, self.embedding, first, self.config.embedding_scale)
        for index, entry in enumerate(self.plan):
            if entry.adds_embedding:
                if stream.ahead is not None:
                    raise RuntimeError("a pass cannot start while a norm's work is handed ahead")
                ops.residual_add(stream.resid, stream.pending, None, first)
                stream.pending = None
            # the norm and mixer that read the stream next, for blocks that hand a norm's work to
            # the product before it
            following = None
            if index + 1 < len(self.plan) and not self.plan[index + 1].adds_embedding:
                later = self.blocks[self.plan[index + 1].layer]
                following = (later.mixer_norm, later.mixer)
            self.blocks[entry.layer].forward(stream, ctx, caches[index], following=following)
        rows = ctx.logit_rows
        logits = ctx.buffer("model.logits", (rows.shape[0], self.config.vocabulary),
                            torch.float32)
        if rows.shape[0] == 0:
            return logits
        last = self.final_norm.forward(stream, ctx, rows=rows, out_name="model.final_norm")
        ops.linear(last, self.output, out=logits, out_dtype=torch.float32)
        if self.config.logit_softcap is not None:
            ops.softcap_(logits, self.config.logit_softcap)
        return logits


def expected_tensors(config: ModelConfig):
    """Names and shapes without building anything on a device."""
    model = DecoderModel(config, torch.float32, "meta")
    return model.expected_tensors()
