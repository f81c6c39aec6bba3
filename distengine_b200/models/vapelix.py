"""The Vapelix architecture: ``VapelixConfig`` describes it (layers of latent attention beside a
gated dense feed-forward or routed experts, both branches on the same input; a side input from a
table row of the token after every layer; a run of layers that is passed several times with the
embedding rows added again before every further pass), the generic decoder runs it."""

from __future__ import annotations

from ..config.vapelix import NAME, VapelixConfig
from ..registry import register_architecture
from .decoder import DecoderModel


def build_vapelix(config: VapelixConfig, dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)


register_architecture(NAME, VapelixConfig.from_json, build_vapelix)
