"""Causal LM of the hybrid decoder family: the model class the registry hands out for its designs.

Same surface as `LLaMAForCausalLM` where it applies (``from_pretrained`` / ``save_pretrained``, ``generate``,
``__call__`` returning logits and a cache, ``_engine_for`` so that the `LLaMA` generation front-end and its
token-at-a-time stream work unchanged).  Parameters are a flat dictionary under the checkpoint's tensor names
(``embed``, ``l<i>.norm1``, ``l<i>.mix.q`` ..., ``final.norm``, ``head``; linear weights ``[out, in]``).  Execution is
the hybrid engine (`models/hybrid_engine.py`) on a CUDA device; this family has no CPU backend.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple

import torch

from ..config import HybridConfig
from .hybrid_engine import HybridEngine, random_tensors
from .llama import WEIGHTS_NAME, GenerateOutput
from .reference import ModelOutput

Params = Dict[str, torch.Tensor]


class HybridForCausalLM:
    """A design of the family subclasses this with its `config_class`."""

    config_class = HybridConfig

    def __init__(self, config: HybridConfig, dtype: torch.dtype = torch.bfloat16, seed: int = 0, _do_init: bool = False,
                 device: Any = "cuda", **runtime_kwargs: Any):
        self.config = config
        self.dtype = dtype
        self.runtime_kwargs = runtime_kwargs          # e.g. use_cuda_graph
        self._params: Optional[Params] = random_tensors(config, device, seed) if _do_init else None
        self._engines: Dict[int, Tuple[Params, HybridEngine]] = {}

    @property
    def params(self) -> Params:
        if self._params is None:
            raise ValueError("model was built without parameters: pass `params=` explicitly")
        return self._params

    @params.setter
    def params(self, value: Params) -> None:
        self._params = value

    # ------------------------------------------------------------------ checkpoint I/O
    @classmethod
    def from_pretrained(cls, path: str, dtype: Optional[torch.dtype] = None, device: Any = "cuda", **kwargs: Any
                        ) -> "HybridForCausalLM":
        """`dtype` is the compute type of the engine (bfloat16 by default; float32 runs every kernel in true fp32).
        Integer tensors of a checkpoint (tables) are kept as they are."""
        from safetensors.torch import load_file

        config = cls.config_class.from_pretrained(path)
        flat = load_file(os.path.join(path, WEIGHTS_NAME), device="cpu")
        model = cls(config, dtype=dtype or torch.bfloat16, **kwargs)
        model.params = {k: v.to(device) for k, v in flat.items()}
        return model

    def save_pretrained(self, save_directory: str, params: Optional[Params] = None) -> None:
        from safetensors.torch import save_file

        os.makedirs(save_directory, exist_ok=True)
        self.config.save_pretrained(save_directory)
        flat = {k: v.detach().cpu().contiguous() for k, v in (params if params is not None else self.params).items()}
        save_file(flat, os.path.join(save_directory, WEIGHTS_NAME), metadata={"format": "pt"})

    # ------------------------------------------------------------------ engine
    def _engine_for(self, params: Optional[Params] = None) -> HybridEngine:
        params = params if params is not None else self.params
        pre = params.get("engine") if isinstance(params, dict) else None
        if pre is not None and not isinstance(pre, torch.Tensor):
            return pre
        hit = self._engines.get(id(params))
        if hit is not None and hit[0] is params:
            return hit[1]
        dev = next(iter(params.values())).device
        if dev.type != "cuda":
            raise NotImplementedError(f"{self.config.architecture} runs on the B200 engine only: move the parameters to a CUDA device")
        eng = HybridEngine(self.config, params, dtype=self.dtype, device=dev, **self.runtime_kwargs)
        self._engines = {id(params): (params, eng)}
        return eng

    # ------------------------------------------------------------------ forward / generate
    @torch.no_grad()
    def __call__(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                 params: Optional[Params] = None, past_key_values: Any = None, last_only: bool = False,
                 **unused: Any) -> ModelOutput:
        eng = self._engine_for(params)
        ids = torch.as_tensor(input_ids).to(eng.device)
        mask = None if attention_mask is None else torch.as_tensor(attention_mask).to(eng.device)
        return eng.forward(ids, attention_mask=mask, cache=past_key_values, last_only=last_only)

    def init_cache(self, batch_size: int, max_length: int, params: Optional[Params] = None) -> Any:
        return self._engine_for(params).new_cache(batch_size, max_length)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                 params: Optional[Params] = None, max_length: Optional[int] = None,
                 max_new_tokens: Optional[int] = None, do_sample: bool = False, temperature: float = 1.0,
                 top_k: Optional[int] = 50, top_p: float = 1.0, pad_token_id: Optional[int] = None,
                 eos_token_id: Optional[int] = None, seed: int = 0) -> GenerateOutput:
        eng = self._engine_for(params)
        ids = torch.as_tensor(input_ids).to(eng.device)
        if max_length is None:
            if max_new_tokens is None:
                raise ValueError("give max_length or max_new_tokens")
            max_length = ids.shape[1] + max_new_tokens
        eos = self.config.eos_token_id if eos_token_id is None else eos_token_id
        pad = self.config.pad_token_id if pad_token_id is None else pad_token_id
        mask = None if attention_mask is None else torch.as_tensor(attention_mask).to(eng.device)
        seqs = eng.generate(ids, mask, max_length=max_length, do_sample=do_sample, temperature=temperature, top_k=top_k,
                            top_p=top_p, pad_token_id=pad, eos_token_id=eos, seed=seed)
        return GenerateOutput(sequences=seqs)
