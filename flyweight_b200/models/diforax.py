"""Diforax: registration of the architecture name with its configuration and model.  The model is the
generic ``DecoderModel`` over ``DiforaxConfig.model_spec()``: layers in the sandwich arrangement (a
weighted RMS norm in front of and behind every sublayer), attention inside chunks with a layer-shared
cache or a gated delta rule as mixer, a gated dense feed-forward or routed experts, a final norm and an
untied head."""
from __future__ import annotations

from ..config.diforax import DiforaxConfig
from ..config.registry import register_architecture
from ..parts.base import Precision
from ..parts.model import DecoderModel


class DiforaxForCausalLM(DecoderModel):
    config_class = DiforaxConfig

    def __init__(self, config: DiforaxConfig, precision: Precision, device):
        self.config = config
        super().__init__(config.model_spec(), precision, device)


register_architecture("Diforax", DiforaxConfig, DiforaxForCausalLM)
