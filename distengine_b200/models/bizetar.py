"""The Bizetar architecture: ``BizetarConfig`` describes it (layers of sink attention in two
forms, each beside a feed-forward with a learned cubic activation or routed gated experts; norms on
the sublayers' gated results; a stream that is mixed over the depth), the generic decoder runs it."""

from __future__ import annotations

from ..config.bizetar import NAME, BizetarConfig
from ..registry import register_architecture
from .decoder import DecoderModel


def build_bizetar(config: BizetarConfig, dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)


register_architecture(NAME, BizetarConfig.from_json, build_bizetar)
