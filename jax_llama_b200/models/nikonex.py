"""Nikonex causal LM: the model class the registry hands out for ``"architecture": "Nikonex"`` (latent attention and
retention layers with mixture-of-experts feed-forwards in parallel blocks; `config.NikonexConfig`)."""
from __future__ import annotations

from ..config import NikonexConfig
from .hybrid import HybridForCausalLM


class NikonexForCausalLM(HybridForCausalLM):
    config_class = NikonexConfig
