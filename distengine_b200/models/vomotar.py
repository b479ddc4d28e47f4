"""The Vomotar architecture: ``VomotarConfig`` describes it (layers of two kinds in any order: the
gated delta rule with a decay per key channel, or chunk-masked attention beside retention), the
generic decoder runs it."""

from __future__ import annotations

from ..config.vomotar import NAME, VomotarConfig
from ..registry import register_architecture
from .decoder import DecoderModel


def build_vomotar(config: VomotarConfig, dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)


register_architecture(NAME, VomotarConfig.from_json, build_vomotar)
