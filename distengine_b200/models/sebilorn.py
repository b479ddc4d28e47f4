"""The Sebilorn architecture: ``SebilornConfig`` describes it (layers of three kinds in any order:
windowed attention that may read an earlier layer's keys and values, gated attention beside the
generalized delta rule, lightning attention; layer norms; a feed-forward with a squared relu), the
generic decoder runs it."""

from __future__ import annotations

from ..config.sebilorn import NAME, SebilornConfig
from ..registry import register_architecture
from .decoder import DecoderModel


def build_sebilorn(config: SebilornConfig, dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)


register_architecture(NAME, SebilornConfig.from_json, build_sebilorn)
