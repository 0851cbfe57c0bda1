"""CPU-side checks of the Nikonex integration: configuration schema, registry, tensor inventory, rotary frequencies, and
the oracle's two forms against each other."""
import json
import math

import pytest
import torch

from jax_llama_b200.config import FoliraxConfig, NikonexConfig
from jax_llama_b200.models import registry
from jax_llama_b200.models.hybrid_engine import tensor_shapes
from jax_llama_b200.models.mixers import rotary_frequencies
from tests import nikonex_oracle as O

MOE = {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}},
       "shared": {"ff": 14}}
LAYERS = [
    {"type": "retention", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.9, 0.99], "rot": {"dims": 4, "base": 100.0}},
     "mlp": None},
    {"type": "latent_attention",
     "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3, "mask": {"size": 7},
               "rot": {"dims": 4, "base": 1000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}},
     "mlp": MOE},
]


def cfg_dict(**over):
    d = {"architecture": "Nikonex", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
         "layers": json.loads(json.dumps(LAYERS))}
    d.update(over)
    return d


def test_config_round_trip(tmp_path):
    c = NikonexConfig.from_dict(cfg_dict())
    assert c.vocab_size == 50 and c.hidden_size == 24 and c.num_hidden_layers == 2 and c.residual_mult == 0.5
    assert c.block == "parallel" and c.norm_offset == 0.0 and FoliraxConfig.block == "sandwich"
    r, a = c.layers[0].mixer, c.layers[1].mixer
    assert r.kind == "retention" and r.decay == [0.9, 0.99] and r.rot.layout == "half" and c.layers[0].mlp is None
    assert a.kind == "latent_attention" and a.window == 7 and a.rot.layout == "interleaved" and a.rot.scaling.factor == 4.0
    f = c.layers[1].mlp
    assert (f.experts, f.top, f.ff, f.groups, f.keep, f.group_top, f.scale, f.shared_ff) == (6, 2, 10, 3, 2, 2, 1.5, 14)
    assert f.score == "sigmoid" and f.act == "relu2" and f.normalise and f.shared_gate
    c.save_pretrained(str(tmp_path))
    again = NikonexConfig.from_pretrained(str(tmp_path))
    assert again.to_dict() == c.to_dict()
    assert registry.resolve(str(tmp_path))[:2] == ("nikonex", NikonexConfig)
    assert registry.kernel_subset("nikonex") == "hybrid" and "float32" in registry.gpu_dtypes("nikonex")


def test_config_defaults_and_validation():
    d = cfg_dict()
    del d["layers"][1]["mixer"]["mask"]
    del d["layers"][1]["mlp"]["router"]["groups"]
    d["layers"][1]["mlp"]["shared"] = None
    c = NikonexConfig.from_dict(d)
    assert c.layers[1].mixer.window == 0 and c.layers[1].mlp.groups == 1 and c.layers[1].mlp.shared_ff == 0
    for bad in (lambda d: d["layers"][0]["mixer"].update(decay=[0.9]),
                lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3),
                lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10),
                lambda d: d["layers"][1]["mixer"]["rot"].update(dims=6),
                lambda d: d["layers"][1]["mlp"]["router"].update(top=7),
                lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6),
                lambda d: d["layers"][1]["mlp"].update(kind="dense"),
                lambda d: d["layers"][0].update(type="conv")):
        d = cfg_dict()
        bad(d)
        with pytest.raises(ValueError):
            NikonexConfig.from_dict(d)


def test_tensor_inventory():
    c = NikonexConfig.from_dict(cfg_dict())
    s = tensor_shapes(c)
    assert s["l0.mix.q"] == (16, 24) and s["l0.mix.v"] == (24, 24) and s["l0.mix.g"] == (24, 24) and s["l0.mix.o"] == (24, 24)
    assert "l0.norm2" not in s and "l0.norm1b" not in s and s["l1.norm2"] == (24,)
    assert s["l1.mix.dq"] == (10, 24) and s["l1.mix.uq"] == (36, 10) and s["l1.mix.dkv"] == (16, 24)
    assert s["l1.mix.dq.norm"] == (10,) and s["l1.mix.dkv.norm"] == (12,)
    assert s["l1.mix.uk"] == (24, 12) and s["l1.mix.uv"] == (18, 12) and s["l1.mix.o"] == (24, 18)
    assert s["l1.mlp.router"] == (6, 24) and s["l1.mlp.e5.up"] == (10, 24) and s["l1.mlp.e0.down"] == (24, 10)
    assert s["l1.mlp.shared.up"] == (14, 24) and s["l1.mlp.shared.down"] == (24, 14) and s["l1.mlp.shared.sg"] == (1, 24)
    assert "l1.mlp.e6.up" not in s and s["final.norm"] == (24,) and s["head"] == (50, 24)


@pytest.mark.parametrize("dims,base,scaling", [(32, 3e5, {"factor": 3.0, "original": 256, "fast": 24.0, "slow": 2.0}),
                                                (8, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}),
                                                (64, 1e4, None)])
def test_rotary_frequencies(dims, base, scaling):
    from jax_llama_b200.config import RotaryScaling
    sc = RotaryScaling(**{k: float(v) for k, v in scaling.items()}) if scaling else None
    f, mult = rotary_frequencies(dims, base, sc)
    want, want_mult = O.rotary_frequencies(dims, base, scaling)
    assert torch.allclose(f, want, rtol=1e-12, atol=0) and mult == want_mult
    if scaling:
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert f[0] == plain[0] and abs(float(f[-1]) - float(plain[-1]) / scaling["factor"]) < 1e-15
        assert abs(mult - (0.1 * math.log(scaling["factor"]) + 1)) < 1e-15


def _random_tensors(c, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        if len(shape) == 1:
            t = 1 + 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16)
    return out


def test_oracle_whole_prompt_equals_its_step_by_step_form():
    """The oracle's two forms (everything at once; a prompt and then token by token, carrying only latents, rotated key
    parts and matrix states) agree, so either can be held against the engine."""
    c = NikonexConfig.from_dict(cfg_dict())
    w = _random_tensors(c)
    toks = torch.randint(0, 50, (21,), generator=torch.Generator().manual_seed(1)).tolist()
    a = O.forward(c.to_dict(), w, toks)
    for cut in (1, 5, 20):
        b = O.forward_stepwise(c.to_dict(), w, toks, cut)
        assert (a - b).abs().max() < 1e-9


def test_oracle_router_respects_groups():
    r = {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([[5.0, -5.0, 4.0, 3.9, 1.0, 0.9]], dtype=torch.float64)      # best single expert sits in the weakest pair
    idx, wt = O.route(z, torch.eye(6, dtype=torch.float64), r)
    assert sorted(idx[0].tolist()) == [2, 3] and abs(float(wt.sum()) - 1.0) < 1e-12
