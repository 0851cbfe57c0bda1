"""CPU-side checks of the Folirax integration: configuration schema, registry, tensor inventory, trace-runner refusals."""
import json

import pytest
import torch

from jax_llama_b200.config import FoliraxConfig, LLaMAConfig
from jax_llama_b200.models import registry
from jax_llama_b200.models.hybrid_engine import tensor_shapes
from tests import folirax_oracle as O

LAYERS = [
    {"type": "gla", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "tau": 4}, "mlp": None},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3,
                                    "rot": {"dims": 4, "base": 1000.0}}, "mlp": {"kind": "dense", "ff": 20}},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "kv_from": 1,
                                    "rot": {"dims": 4, "base": 1000.0}}, "mlp": None},
]


def cfg_dict(**over):
    d = {"architecture": "Folirax", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
         "logit_softcap": 10.0, "layers": json.loads(json.dumps(LAYERS))}
    d.update(over)
    return d


def test_config_round_trip(tmp_path):
    c = FoliraxConfig.from_dict(cfg_dict())
    assert c.vocab_size == 50 and c.hidden_size == 24 and c.num_hidden_layers == 3
    assert c.layers[0].mixer.kind == "gla" and c.layers[0].mixer.tau == 4.0 and c.layers[0].mlp is None
    assert c.layers[2].mixer.kv_from == 1 and c.layers[1].mlp.ff == 20 and c.layers[1].mlp.act == "relu2"
    c.save_pretrained(str(tmp_path))
    again = FoliraxConfig.from_pretrained(str(tmp_path))
    assert again.to_dict() == c.to_dict()
    assert registry.resolve(str(tmp_path))[:2] == ("folirax", FoliraxConfig)
    assert registry.kernel_subset("folirax") == "hybrid" and "float32" in registry.gpu_dtypes("folirax")


def test_config_defaults_and_validation():
    d = cfg_dict()
    del d["logit_softcap"]
    del d["layers"][1]["mixer"]["kv_heads"]
    d["layers"][2]["mixer"]["kv_heads"] = 4
    c = FoliraxConfig.from_dict(d)
    assert c.logit_softcap == 0.0 and c.layers[1].mixer.kv_heads == 4
    for bad in (lambda d: d["layers"][2]["mixer"].update(kv_from=0),          # not an attention layer
                lambda d: d["layers"][2]["mixer"].update(kv_from=2),          # not an earlier layer
                lambda d: d["layers"][1]["mixer"]["rot"].update(dims=3),
                lambda d: d["layers"][1]["mixer"].update(kv_heads=3),
                lambda d: d["layers"][0].update(type="conv"),
                lambda d: d["layers"][0]["mixer"].update(tau=0)):
        d = cfg_dict()
        bad(d)
        with pytest.raises(ValueError):
            FoliraxConfig.from_dict(d)


def test_registry_keeps_llama_as_default(tmp_path):
    LLaMAConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2
                ).save_pretrained(str(tmp_path))
    name, cfg_cls, _ = registry.resolve(str(tmp_path))
    assert name == "llama" and cfg_cls is LLaMAConfig
    assert registry.gpu_dtypes("llama") == ("bfloat16",)
    with pytest.raises(KeyError):
        registry.architecture_of({"architecture": "nonesuch"})


def test_tensor_inventory_matches_the_oracle():
    """Every tensor the engine asks for is one the plain statement of the design reads, with that shape."""
    c = FoliraxConfig.from_dict(cfg_dict())
    shapes = tensor_shapes(c, decay_rank=3)
    assert "l2.mix.k" not in shapes and "l2.mix.v" not in shapes and shapes["l1.mix.g"] == (4, 24)
    assert shapes["l0.mix.a1"] == (3, 24) and shapes["l0.mix.a2"] == (16, 3) and "l0.norm2" not in shapes
    g = torch.Generator().manual_seed(0)
    tensors = {k: (0.3 * torch.randn(s, generator=g)).to(torch.bfloat16) for k, s in shapes.items()}
    logits, streams = O.forward(c.to_dict(), tensors, [3, 1, 4, 1, 5, 9, 2, 6], return_layers=True)
    assert logits.shape == (8, 50) and streams.shape == (3, 8, 24) and torch.isfinite(logits).all()
    assert logits.abs().max() <= 10.0


def test_oracle_recurrence_can_be_cut_anywhere():
    """The plain gated-linear-attention statement carried over a cut with its state equals the uncut run."""
    c = cfg_dict()
    m = c["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(1)
    w = {"q": torch.randn(16, 24, generator=g), "k": torch.randn(16, 24, generator=g), "v": torch.randn(24, 24, generator=g),
         "g": torch.randn(24, 24, generator=g), "o": torch.randn(24, 24, generator=g), "norm": torch.ones(12),
         "a1": torch.randn(3, 24, generator=g), "a2": torch.randn(16, 3, generator=g), "a2.b": torch.randn(16, generator=g)}
    h = torch.randn(11, 24, generator=g, dtype=torch.float64)
    full, s_full = O.gla_mixer(h, w, m, 1e-5)
    a, s_a = O.gla_mixer(h[:4], w, m, 1e-5)
    b, s_b = O.gla_mixer(h[4:], w, m, 1e-5, state=s_a)
    assert torch.allclose(torch.cat([a, b]), full, atol=1e-12) and torch.allclose(s_b, s_full, atol=1e-12)


def test_trace_runner_refuses_what_the_engine_cannot_do(tmp_path, capsys):
    from jax_llama_b200 import trace_run

    LLaMAConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2
                ).save_pretrained(str(tmp_path))
    rc = trace_run.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "o")])
    assert rc == 3                                  # the LLaMA engine is bfloat16 only
