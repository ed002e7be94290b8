"""Kemitar: registration of the architecture name with its configuration and model.  The model is
the generic ``DecoderModel`` over ``KemitarConfig.model_spec()``: a hashed-pair embedding, layers in
the output-norm arrangement (token shift, latent attention with a sink, gated feed-forward, gain-only
norms), a gain-only final norm and an untied head."""
from __future__ import annotations

from ..config.kemitar import KemitarConfig
from ..config.registry import register_architecture
from ..parts.base import Precision
from ..parts.model import DecoderModel


class KemitarForCausalLM(DecoderModel):
    config_class = KemitarConfig

    def __init__(self, config: KemitarConfig, precision: Precision, device):
        self.config = config
        super().__init__(config.model_spec(), precision, device)


register_architecture("Kemitar", KemitarConfig, KemitarForCausalLM)
