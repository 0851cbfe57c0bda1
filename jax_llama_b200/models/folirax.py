"""Folirax causal LM: the model class the registry hands out for ``"architecture": "Folirax"`` (gated linear attention
and softmax attention layers in sandwich blocks; `config.FoliraxConfig`)."""
from __future__ import annotations

from ..config import FoliraxConfig
from .hybrid import HybridForCausalLM


class FoliraxForCausalLM(HybridForCausalLM):
    config_class = FoliraxConfig
