"""Nikonex on the hybrid engine against the plain float64 statement of the design (`nikonex_oracle.py`).

Small configurations with random weights; every test builds its own.  The float32 engine is held to a tight bound,
the bfloat16 engine to the error that rounding its operands causes.
"""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from jax_llama_b200.config import MoeMlpSpec, NikonexConfig, RotaryScaling       # noqa: E402
from jax_llama_b200.generation import LLaMA                                      # noqa: E402
from jax_llama_b200.models.feedforward import MoeFeedForward                     # noqa: E402
from jax_llama_b200.models.hybrid_engine import HybridEngine, random_tensors     # noqa: E402
from jax_llama_b200.models.mixers import rotary_table                            # noqa: E402
from jax_llama_b200.models.nikonex import NikonexForCausalLM                     # noqa: E402
from jax_llama_b200.ops import seq_kernels as SK                                 # noqa: E402
from jax_llama_b200.tokenizers import IdTokenizer                                # noqa: E402

from tests import nikonex_oracle as O                                            # noqa: E402

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]
YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}


def moe(experts=8, top=2, ff=24, groups=(4, 2), scale=1.5, shared=40):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r, "shared": {"ff": shared} if shared else None}


def ret(heads=2, dim=16, vdim=24, decay=(0.9, 0.995), rot=16, base=10000.0, mlp=None):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                                            "rot": {"dims": rot, "base": base}}, "mlp": mlp}


def lat(heads=3, dim=16, rot_dim=8, vdim=12, q_rank=20, kv_rank=24, window=20, base=10000.0, scale=0.25, scaling=YARN,
        mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling:
        rot["scaling"] = dict(scaling)
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(layers, vocab=96, width=72, eps=1e-5, mult=0.7, dtype=None):
    """With dtype bfloat16 every expert of a layer is chosen (top = experts, no groups): rounding the router's input
    to bfloat16 moves its logits by parts in a thousand, which among random scores flips a close choice every few
    dozen tokens and the oracle would then follow other experts.  The choice itself is checked in float32, and in
    bfloat16 where both sides see the same rounded input (the router and the feed-forward alone)."""
    if dtype == torch.bfloat16:
        layers = json.loads(json.dumps(layers))
        for l in layers:
            if l["mlp"] is not None:
                l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
                l["mlp"]["router"].pop("groups", None)
    return NikonexConfig.from_dict({"architecture": "Nikonex", "vocab": vocab, "width": width, "norm": {"eps": eps},
                                    "residual_mult": mult, "layers": layers})


MIXED = [lat(mlp=moe()), ret(mlp=moe(experts=6, top=3, groups=(3, 2), shared=0)), ret(heads=3, dim=8, vdim=16,
         decay=(0.5, 0.97, 1.0), rot=4), lat(heads=2, dim=8, rot_dim=16, vdim=20, q_rank=12, kv_rank=16, window=0,
                                             scaling=None, mlp=moe(experts=4, top=4, groups=None))]


def build(cfg, dtype, seed=0, graph=True, tweak=None):
    tensors = random_tensors(cfg, "cuda", seed)
    if tweak is not None:
        tweak(tensors)
    eng = HybridEngine(cfg, tensors, dtype=dtype, device="cuda", use_cuda_graph=graph)
    return eng, {k: v.cpu() for k, v in tensors.items()}


def err(got, want):
    """Centred RMS difference over the vocabulary relative to the RMS of the wanted logits, worst row."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def tokens(n, vocab, seed):
    return torch.randint(1, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def oracle_logits(cfg, cpu_tensors, toks):
    return O.forward(cfg.to_dict(), cpu_tensors, toks)


def feed(vals):
    return torch.tensor(vals, dtype=torch.int32).pin_memory()


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("scaling", [None, YARN, {"factor": 3.0, "original": 256, "fast": 24.0, "slow": 2.0}])
@pytest.mark.parametrize("dims", [2, 8, 32, 64])
def test_rotary_tables(dims, scaling):
    sc = RotaryScaling(**{k: float(v) for k, v in scaling.items()}) if scaling else None
    cos, sin = rotary_table(dims, 3e5, 300, torch.device("cuda"), sc)
    f, mult = O.rotary_frequencies(dims, 3e5, scaling)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert (cos.double().cpu() - torch.cos(ang) * mult).abs().max() < 1e-6
    assert (sin.double().cpu() - torch.sin(ang) * mult).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layout", ["interleaved", "half"])
@pytest.mark.parametrize("n,rot", [(8, 8), (12, 6), (16, 2), (5, 0)])
def test_rotation_of_a_head_slice(dtype, layout, n, rot):
    """A slice of every head rotated at the token's position (cache fill level minus left padding) and moved into
    another head layout."""
    B, S, H, pre = 2, 7, 3, 5
    g = torch.Generator(device="cuda").manual_seed(n)
    src = torch.randn(B * S, H * (pre + n), device="cuda", generator=g).to(dtype)
    out = torch.zeros(B * S, H * (n + 3), device="cuda", dtype=dtype)
    cos, sin = rotary_table(max(rot, 2), 100.0, 64, torch.device("cuda"))
    base, pad = torch.tensor([11], dtype=torch.int32, device="cuda"), torch.tensor([0, 4], dtype=torch.int32, device="cuda")
    SK.rotary_slice(src, pre + n, pre, out, n + 3, 3, H, n, rot, SK.ROT_LAYOUTS[layout], cos, sin, base, pad, B, S)
    x = src.double().cpu().view(B, S, H, pre + n)[..., pre:]
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    for b in range(B):
        pos = torch.arange(S) + 11 - int(pad[b])
        want = O.rotate(x[b], pos, rot, 100.0, layout) if rot else x[b]
        got = out.double().cpu().view(B, S, H, n + 3)[b, ..., 3:]
        assert (got - want).abs().max() < tol * 4
    assert out.view(B * S, H, n + 3)[..., :3].abs().max() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 90, 100, 1100])
def test_branch_sum_and_two_norms(dtype, width):
    g = torch.Generator(device="cuda").manual_seed(width)
    x = torch.randn(5, width, device="cuda", generator=g) * 3
    y1 = torch.randn(5, width + 8, device="cuda", generator=g)[:, :width]
    y2 = torch.randn(5, width, device="cuda", generator=g)
    w1 = (1 + 0.2 * torch.randn(width, device="cuda", generator=g)).to(dtype)
    w2 = (1 + 0.2 * torch.randn(width, device="cuda", generator=g)).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for a, b, u, v in [(y1, y2, w1, w2), (y1, None, w1, None), (None, None, w1, w2), (y1, y2, None, None), (None, y2, None, w2)]:
        xx = x.clone()
        h1, h2 = SK.branch_add_norm(xx, a, b, 0.3, u, v, 1e-5)
        want = x.double().cpu() + 0.3 * ((a.double().cpu() if a is not None else 0) + (b.double().cpu() if b is not None else 0))
        assert (xx.double().cpu() - want).abs().max() < 1e-5
        for h, w in ((h1, u), (h2, v)):
            assert (h is None) == (w is None)
            if w is not None:
                assert (h.double().cpu() - O.norm_plain(want, w.cpu(), 1e-5)).abs().max() < tol * 4


@pytest.mark.parametrize("E,top,groups,keep", [(15, 4, 3, 2), (8, 2, 4, 2), (8, 8, 1, 1), (6, 3, 6, 4), (64, 6, 8, 3),
                                               (40, 5, 1, 1), (9, 1, 3, 1), (16, 4, 4, 4)])
def test_router_choices_and_weights(E, top, groups, keep):
    """Sigmoid scores, groups of neighbours scored by their two largest (or the only one), the best groups kept, the
    top of what is left, weights over their sum times a constant: indices as a set and weights per expert."""
    g = torch.Generator(device="cuda").manual_seed(E + top)
    z = torch.randn(37, E + 3, device="cuda", generator=g) * 2
    idx, wt = SK.moe_route(z[:, :E], E, top, groups, keep, 2, SK.SCORE_SIGMOID, True, 1.7)
    r = {"experts": E, "top": top, "scale": 1.7}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    want_idx, want_wt = O.route(z[:, :E].double().cpu(), torch.eye(E, dtype=torch.float64), r)
    for m in range(z.shape[0]):
        got = dict(zip(idx[m].tolist(), wt[m].tolist()))
        want = dict(zip(want_idx[m].tolist(), want_wt[m].tolist()))
        assert set(got) == set(want), m
        assert all(abs(got[e] - want[e]) < 1e-5 for e in got), m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 16, 17, 150])
@pytest.mark.parametrize("spec", [dict(experts=8, top=2, ff=24, groups=4, keep=2, shared_ff=40),
                                  dict(experts=5, top=5, ff=10, groups=1, keep=1, shared_ff=0),
                                  dict(experts=10, top=3, ff=48, groups=5, keep=3, shared_ff=8, scale=2.5)])
def test_mixture_of_experts_alone(dtype, rows, spec):
    """Few rows (every pair streams its expert) and many rows (pairs ordered by expert into row tiles), with and
    without a shared expert."""
    W = 56
    sp = MoeMlpSpec(**spec)
    g = torch.Generator(device="cuda").manual_seed(rows)
    w = {n: (torch.randn(s, device="cuda", generator=g) / math.sqrt(s[1])).to(torch.bfloat16)
         for n, s in MoeFeedForward.shapes(sp, W).items()}
    w["router"] = (w["router"].float() * 6).to(torch.bfloat16)
    h = torch.randn(rows, W, device="cuda", generator=g).to(torch.bfloat16)
    got = MoeFeedForward(sp, {k: v.to(dtype) for k, v in w.items()}).run(h.to(dtype))
    mlp = {"expert": {"ff": sp.ff}, "router": {"experts": sp.experts, "top": sp.top, "scale": sp.scale,
                                               "groups": {"count": sp.groups, "keep": sp.keep} if sp.groups > 1 else None},
           "shared": {"ff": sp.shared_ff} if sp.shared_ff else None}
    want = O.moe(h.double().cpu(), {k: v.cpu() for k, v in w.items()}, mlp)
    assert got.dtype == torch.float32 and got.shape == (rows, W)
    assert (got.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2) * want.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layers", [[ret()], [ret(heads=1, dim=80, vdim=8, decay=(0.99,), rot=80)],
                                    [ret(heads=3, dim=48, vdim=40, decay=(1.0, 0.5, 0.999), rot=10, mlp=moe())],
                                    [lat()], [lat(heads=1, window=0)], [lat(window=1, mlp=moe())],
                                    [lat(heads=5, dim=4, rot_dim=2, vdim=6, q_rank=7, kv_rank=9, window=64, scaling=None)],
                                    [lat(heads=20, dim=8, rot_dim=4, vdim=8, q_rank=16, kv_rank=8, window=33)]],
                         ids=["ret", "ret-wide", "ret-moe", "lat", "lat-full", "lat-self", "lat-odd", "lat-many-heads"])
def test_single_mechanism_models(dtype, layers):
    cfg = config(layers, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=3)
    toks = tokens(75, cfg.vocab_size, 1)
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got, oracle_logits(cfg, cpu, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_stream_after_every_layer(dtype):
    cfg = config(MIXED, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=2)
    toks = tokens(40, cfg.vocab_size, 9)
    eng.capture_streams = []
    eng.forward(torch.tensor([toks], device="cuda"))
    want = []
    O.forward(cfg.to_dict(), cpu, toks, want)
    assert len(eng.capture_streams) == len(want) == len(MIXED)
    for i, (g, w) in enumerate(zip(eng.capture_streams, want)):
        assert g.dtype == torch.float32
        assert (g.double().cpu() - w).abs().max() < (1e-4 if dtype == torch.float32 else 5e-2) * w.abs().max(), i


def test_other_constants():
    """Residual multiplier, eps, weight scale, window and decays far from the usual values."""
    layers = [lat(window=3, scale=1.3, base=50.0, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5},
                  mlp=moe(scale=0.25, groups=(2, 1))), ret(decay=(0.2, 0.9999), base=7.0, mlp=moe(top=1, groups=(8, 1)))]
    cfg = config(layers, eps=0.3, mult=1.75)
    eng, cpu = build(cfg, torch.float32, seed=11)
    toks = tokens(50, cfg.vocab_size, 4)
    assert err(eng.forward(torch.tensor([toks], device="cuda")).logits[0], oracle_logits(cfg, cpu, toks)) < TOL[torch.float32]


# ------------------------------------------------------------------------------------------ prefill vs decoding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("prompt", [1, 2, 31, 33])
def test_decode_matches_prefill_and_oracle(dtype, prompt):
    """The prompt in one step, then 70 tokens one by one through the graph-replayed step: the window passes over
    decoded tokens, the 32-key blocks of the attention kernels and the first tokens of a sequence are all crossed."""
    cfg = config(MIXED, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=4)
    toks = tokens(prompt + 70, cfg.vocab_size, prompt)
    want = oracle_logits(cfg, cpu, toks)
    stream = eng.begin_stream(torch.tensor([toks[:prompt]], device="cuda"), None, max_length=len(toks) + 1, eos_token_id=-1,
                              logit_rows=torch.arange(prompt))
    assert err(stream.prompt_logits(), want[:prompt]) < TOL[dtype]
    rows = []
    for t in toks[prompt:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    assert err(torch.stack(rows), want[prompt:]) < TOL[dtype]
    stream.close()
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole, want) < TOL[dtype]
    if dtype == torch.float32:
        assert err(torch.stack(rows), whole[prompt:]) < 5e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """Three hundred tokens decoded one by one after a two-token prompt, against the oracle's own step-by-step form."""
    cfg = config([ret(mlp=moe()), lat(window=40, mlp=moe(shared=0))], dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=21)
    toks = tokens(302, cfg.vocab_size, 5)
    want = O.forward_stepwise(cfg.to_dict(), cpu, toks, 2)
    stream = eng.begin_stream(torch.tensor([toks[:2]], device="cuda"), None, max_length=310, eos_token_id=-1)
    rows = [stream.logits()[0].clone()]
    for t in toks[2:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[1:]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 30], [33, 2, 9], [5, 64, 3]])
def test_prompt_in_portions(dtype, cuts):
    """The same prompt fed to one cache in portions of several sizes, down to two tokens."""
    cfg = config(MIXED, dtype=dtype)
    eng, cpu = build(cfg, dtype, seed=14)
    toks = tokens(sum(cuts), cfg.vocab_size, 31)
    want = oracle_logits(cfg, cpu, toks)
    cache = eng.new_cache(1, len(toks) + 2)
    cache.set_index(0)
    got, at = [], 0
    for n in cuts:
        got.append(eng.forward(torch.tensor([toks[at:at + n]], device="cuda"), cache=cache).logits[0])
        at += n
    assert err(torch.cat(got), want) < TOL[dtype]


def run_unequal_batch(cfg, dtype, lens, extra, seed):
    """Left-padded batch of prompts of the given lengths, then `extra` tokens decoded together; every row is compared
    with the oracle run of that request alone."""
    eng, cpu = build(cfg, dtype, seed=seed)
    seqs = [tokens(n + extra, cfg.vocab_size, 20 + n + 100 * b) for b, n in enumerate(lens)]
    S, B = max(lens), len(lens)
    ids = torch.zeros((B, S), dtype=torch.long)
    mask = torch.zeros((B, S), dtype=torch.int32)
    rows = []
    for b, (n, s) in enumerate(zip(lens, seqs)):
        ids[b, S - n:] = torch.tensor(s[:n])
        mask[b, S - n:] = 1
        rows += [b * S + S - n + j for j in range(n)]
    stream = eng.begin_stream(ids.cuda(), mask.cuda(), max_length=S + extra + 1, eos_token_id=-1,
                              logit_rows=torch.tensor(rows))
    got_prompt = stream.prompt_logits().clone()
    steps = []
    for j in range(extra):
        stream.step(feed([s[n + j] for n, s in zip(lens, seqs)]))
        steps.append(stream.logits().clone())
    stream.close()
    at = 0
    for b, (n, s) in enumerate(zip(lens, seqs)):
        want = oracle_logits(cfg, cpu, s)
        assert err(got_prompt[at:at + n], want[:n]) < TOL[dtype], b
        assert err(torch.stack([x[b] for x in steps]), want[n:]) < TOL[dtype], b
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_alone(dtype):
    """Prompts of 1, 7 and 40 tokens in one batch: padding must touch neither the recurrent state nor the visible keys,
    the window, the positions or the choice of experts of the real tokens."""
    run_unequal_batch(config(MIXED, dtype=dtype), dtype, [1, 7, 40], 36, seed=6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_odd_sizes_and_a_batch_of_twenty(dtype):
    """Sizes that fit no vector width or tile (width 90, vocab 77, heads of 10 / 6 / 14 channels, ranks 11 and 13) in a
    batch of twenty unequal requests: more rows than the pairwise expert path and the weight-streaming kernel take,
    so decoding runs the sorted experts and the GEMMs."""
    layers = [lat(heads=3, dim=10, rot_dim=6, vdim=14, q_rank=11, kv_rank=13, window=9, mlp=moe(experts=9, top=2, ff=10,
                                                                                                groups=(3, 2), shared=6)),
              ret(heads=3, dim=12, vdim=10, decay=(0.8, 0.9, 0.99), rot=6, mlp=moe(experts=3, top=1, ff=5, groups=None))]
    cfg = config(layers, vocab=77, width=90, dtype=dtype)
    run_unequal_batch(cfg, dtype, [3, 17, 1, 9, 30, 2, 12, 25, 8, 21, 4, 5, 6, 7, 11, 13, 14, 15, 16, 29], 12, seed=17)


def test_realistic_head_sizes():
    """Latent rank 128 with a 32-wide rotated part and 64-wide heads; retention heads of 64 x 128."""
    layers = [lat(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=96, kv_rank=128, window=48, mlp=moe(ff=64)),
              ret(heads=2, dim=64, vdim=128, decay=(0.97, 0.999), rot=64)]
    run_unequal_batch(config(layers, width=256, vocab=128, dtype=torch.bfloat16), torch.bfloat16, [5, 150, 131], 40, seed=13)


def test_state_and_cache_are_clean_when_used_again():
    """The same decode state serves request after request: a second, shorter request must see nothing of the first
    (recurrent state zeroed, old latents invisible, old left-pad counts gone)."""
    cfg = config(MIXED)
    eng, cpu = build(cfg, torch.float32, seed=8)
    a, b = tokens(50, cfg.vocab_size, 1), tokens(9, cfg.vocab_size, 2)
    pad_ids = torch.zeros((2, 50), dtype=torch.long)
    pad_ids[0] = torch.tensor(a)
    pad_ids[1, 41:] = torch.tensor(b)
    mask = (torch.arange(50)[None, :] >= torch.tensor([0, 41])[:, None]).int()
    out1 = eng.generate(pad_ids.cuda(), mask.cuda(), max_length=60, eos_token_id=-1)
    st = eng._decode_state(2, 60)
    ids2 = torch.tensor([b, b[::-1]])
    out2 = eng.generate(ids2.cuda(), None, max_length=60, eos_token_id=-1)          # same (B, max_length): same state, same cache
    assert eng._decode_state(2, 60) is st
    fresh, _ = build(cfg, torch.float32, seed=8)
    out3 = fresh.generate(ids2.cuda(), None, max_length=60, eos_token_id=-1)
    assert torch.equal(out2, out3)
    assert out1.shape == (2, 60)
    eng.release_state(st)
    assert (2, 60) not in eng._decode_states
    out4 = eng.generate(ids2.cuda(), None, max_length=60, eos_token_id=-1)
    assert torch.equal(out4, out3)


# ------------------------------------------------------------------------------------------ made-to-show inputs
def _unit_rows(t, token_channel):
    """Embedding rows that are unit vectors: token -> channel.  With a norm weight of one the mixer then sees exactly
    one (scaled) column of each projection for such a token."""
    for tok, ch in token_channel.items():
        t["embed"][tok] = 0
        t["embed"][tok, ch] = 1.0


def _plant_key(t, m, width, eps, A, B, gain):
    """Rewrite the keys' up-projection of every head so that token A's unrotated key is `gain` times token B's
    unrotated query: U_h := gain · a_h c_Aᵀ / |c_A|², with a_h = B's query and c_A = A's normed latent.  Other tokens'
    keys keep only their latents' component along c_A, so among random tokens A's score stands far out for B."""
    H, D, R, rank = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    root = math.sqrt(width)
    hA = torch.zeros(width, dtype=torch.float64)
    hA[1] = root
    hB = torch.zeros(width, dtype=torch.float64)
    hB[0] = root
    w = {k[len("l0.mix."):]: v.cpu() for k, v in t.items() if k.startswith("l0.mix.")}
    cA = O.norm_plain((w["dkv"].double() @ hA)[:rank], w["dkv.norm"], eps)
    cq = O.norm_plain(w["dq"].double() @ hB, w["dq.norm"], eps)
    q = (w["uq"].double() @ cq).view(H, D + R)[:, :D]
    uk = gain * q[:, :, None] * cA[None, None, :] / (cA @ cA)
    t["l0.mix.uk"].copy_(uk.reshape(H * D, rank).to(t["l0.mix.uk"].dtype))


def _planted_attention(window, dtype, seed=5):
    A, B = 61, 60
    layer = lat(heads=2, dim=16, rot_dim=4, vdim=12, q_rank=12, kv_rank=16, window=window, scale=1.0, base=1e6, scaling=None)
    cfg = config([layer], vocab=64, width=48)

    def tweak(t):
        t["l0.norm1"].fill_(1.0)
        _unit_rows(t, {B: 0, A: 1})
        _plant_key(t, layer["mixer"], 48, 1e-5, A, B, 3.0)
    eng, cpu = build(cfg, dtype, seed=seed, tweak=tweak)
    return cfg, eng, cpu, A, B


def _check_last(cfg, eng, cpu, toks, dtype, at, matters):
    """The last token's logits in a whole prompt and decoded alone, against the oracle; `matters`: whether replacing
    the planted token (at `at`) must move them."""
    want = oracle_logits(cfg, cpu, toks)
    without = list(toks)
    without[at] = 59
    moved = err(oracle_logits(cfg, cpu, without)[-1:], want[-1:])
    assert (moved > 10 * TOL[dtype]) if matters else (moved < 1e-9), moved
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole[-1:], want[-1:]) < TOL[dtype]
    stream = eng.begin_stream(torch.tensor([toks[:-1]], device="cuda"), None, max_length=len(toks) + 3, eos_token_id=-1)
    stream.step(feed([toks[-1]]))
    assert err(stream.logits()[:1], want[-1:]) < TOL[dtype]
    stream.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 63, 64, 290])
def test_one_far_key_decides(dtype, far):
    """Latent attention without a window and with a sharp softmax.  Token A's key is made a multiple of token B's
    query, so when B is the last token and A stands once at position `far`, that single key takes nearly all the
    weight among 300 random ones: a kernel that drops or misplaces it (edges of the 32-key blocks, the first slots,
    hundreds back) moves the logits far beyond the tolerance."""
    cfg, eng, cpu, A, B = _planted_attention(0, dtype)
    toks = [2 + (i % 50) for i in range(300)]
    toks[far] = A
    toks.append(B)
    _check_last(cfg, eng, cpu, toks, dtype, far, True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [2, 24, 32, 33, 70])
@pytest.mark.parametrize("back", ["inside", "outside", "next", "far_outside"])
def test_window_edge_decides(dtype, window, back):
    """The planted key stands on the last position the window still shows, on the first it hides, right before the
    query, or far behind the window: seen where it must be, invisible where it must not."""
    d = {"inside": window - 1, "outside": window, "next": 1, "far_outside": window + 64}[back]
    cfg, eng, cpu, A, B = _planted_attention(window, dtype)
    n = 200
    toks = [2 + (i % 50) for i in range(n)]
    toks[n - d] = A
    toks.append(B)
    _check_last(cfg, eng, cpu, toks, dtype, n - d, d < window)


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_slides_over_decoded_tokens(dtype):
    """The planted key is in the prompt; B is then decoded again and again: A is seen until it leaves the window."""
    window = 12
    cfg, eng, cpu, A, B = _planted_attention(window, dtype)
    toks = [2 + (i % 50) for i in range(40)] + [A] + [B] * 20
    want = oracle_logits(cfg, cpu, toks)
    assert err(want[41 + window - 2:41 + window - 1], want[41 + window - 1:41 + window]) > 10 * TOL[dtype]   # A leaves here
    stream = eng.begin_stream(torch.tensor([toks[:41]], device="cuda"), None, max_length=70, eos_token_id=-1)
    rows = []
    for t in toks[41:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows), want[41:]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gap", [2, 7, 8, 9, 216])
def test_retention_state_keeps_a_far_token(dtype, gap):
    """Retention with slow decays.  The filler token has a zero key (its embedding channel is cut out of W_k), so the
    state holds only what two planted tokens wrote, `gap` steps and one step back.  The read-out is divided by its
    own RMS, so one token alone would hide a wrong decay; the mix of the two shows decay^(gap-1): a state that is lost,
    reset or decayed wrongly at an edge of the scan's token chunks moves the logits.  In a prompt and decoded."""
    filler, first, second = 5, 40, 41
    cfg = config([ret(heads=2, dim=16, vdim=16, decay=(0.999, 0.9995), rot=8, base=1e4)], vocab=64, width=48)

    def tweak(t):
        t["l0.norm1"].fill_(1.0)
        _unit_rows(t, {filler: 3})
        t["l0.mix.k"][:, 3] = 0
    eng, cpu = build(cfg, dtype, seed=7, tweak=tweak)
    n = 230
    toks = [filler] * n
    toks[n - 1 - gap], toks[n - 2] = first, second
    want = oracle_logits(cfg, cpu, toks)
    other = list(toks)
    other[n - 1 - gap] = first + 2
    assert err(oracle_logits(cfg, cpu, other)[-1:], want[-1:]) > 5 * TOL[dtype]
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got[n - 1 - gap:], want[n - 1 - gap:]) < TOL[dtype]
    cut = 10
    stream = eng.begin_stream(torch.tensor([toks[:cut]], device="cuda"), None, max_length=n + 2, eos_token_id=-1)
    rows = []
    for t in toks[cut:]:
        stream.step(feed([t]))
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows)[n - 1 - gap - cut:], want[n - 1 - gap:]) < TOL[dtype]


# ------------------------------------------------------------------------------------------ the framework's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_front_end(dtype, tmp_path):
    """save_pretrained → registry → `LLaMA.generate_from_str` (left-padded batch, scheduler, on-device arg-max): every
    generated token is the oracle's arg-max given its prefix, up to near-ties."""
    from jax_llama_b200.models import registry

    cfg = config(MIXED, vocab=80, dtype=dtype)
    model = NikonexForCausalLM(cfg, dtype=dtype, seed=12, _do_init=True)
    model.save_pretrained(str(tmp_path))
    assert registry.resolve(str(tmp_path))[0] == "nikonex"
    loaded = registry.load_pretrained(str(tmp_path), dtype=dtype, device="cuda")
    assert isinstance(loaded, NikonexForCausalLM) and loaded.config.to_dict() == cfg.to_dict()
    llm = LLaMA(loaded.params, loaded, IdTokenizer(cfg.vocab_size))
    prompts = ["7 8 9 10 11 12", "40", "3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3 3"]
    texts = llm.generate_from_str(prompts, max_gen_len=24, temperature=0.0)
    cpu = {k: v.cpu() for k, v in loaded.params.items()}
    for p, t in zip(prompts, texts):
        ids = [int(x) for x in t.split()]
        n0 = len(p.split()) + 1
        assert ids[:n0] == [1] + [int(x) for x in p.split()]
        assert len(ids) > n0
        want = oracle_logits(cfg, cpu, ids)
        for j in range(n0, len(ids)):
            row = want[j - 1]
            assert row[ids[j]] >= row.max() - (1e-3 if dtype == torch.float32 else 0.15), (p, j)
    sampled = llm.generate_from_str(prompts[:1], max_gen_len=8, temperature=0.9, top_p=0.9)
    assert len(sampled[0].split()) >= 7


def test_command_line_generates_from_a_checkpoint_directory(tmp_path):
    """examples/example.py --model_dir: registry, loader, engine, scheduler and sampler behind the command line."""
    cfg = config(MIXED, vocab=80)
    NikonexForCausalLM(cfg, seed=3, _do_init=True).save_pretrained(str(tmp_path))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "example.py"), "--model_dir", str(tmp_path), "--prompt",
                        "7 8 9", "--prompt", "40", "--max_gen_len", "6", "--temperature", "0"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip() and not l.startswith("=")]
    assert lines[0].split()[:4] == ["1", "7", "8", "9"] and lines[1].split()[:2] == ["1", "40"]
    assert all(0 <= int(t) < 80 for l in lines[:2] for t in l.split())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_batches_that_come_and_go(dtype, tmp_path):
    """bin/trace_run on a saved checkpoint: a request alone, a batch of three unequal requests decoded together while
    its shorter ones end, a second batch that opens while the first is still live and goes on beside it; every wanted
    row against the oracle of that request alone."""
    cfg = config(MIXED, vocab=80, dtype=getattr(torch, dtype))
    model = NikonexForCausalLM(cfg, seed=5, _do_init=True)
    model.save_pretrained(str(tmp_path / "m"))
    cpu = {k: v.cpu() for k, v in model.params.items()}
    seq = {"a": tokens(30, 80, 1), "b": tokens(12, 80, 2), "c": tokens(47, 80, 3), "d": tokens(9, 80, 4), "e": tokens(26, 80, 5)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seq["a"][:25], "want": [0, 24]}], "end": []}]
    for j in range(25, 30):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [seq["a"][j]], "want": [0] if j % 2 else []}],
                      "end": ["a"] if j == 29 else []})
    steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": seq["b"][:9], "want": [8]},
                                                   {"id": "c", "tokens": seq["c"][:41], "want": list(range(0, 41, 5))},
                                                   {"id": "d", "tokens": seq["d"][:6], "want": []}], "end": []})
    for j in range(3):
        live = [("b", 9 + j, 12), ("c", 41 + j, 47), ("d", 6 + j, 9)]
        ent = [{"id": r, "tokens": [seq[r][at]], "want": [0]} for r, at, n in live]
        steps.append({"step": len(steps), "entries": ent, "end": [r for r, at, n in live if at == n - 1]})
    # a second batch opens while the first still has a live request; from then on both go on token by token
    steps.append({"step": len(steps), "entries": [{"id": "e", "tokens": seq["e"][:20], "want": [19]},
                                                   {"id": "a2", "tokens": seq["a"][:3], "want": [2]}], "end": ["a2"]})
    for j in range(6):
        ent = [{"id": "e", "tokens": [seq["e"][20 + j]], "want": [0]}]
        if j < 3:
            ent.insert(0, {"id": "c", "tokens": [seq["c"][44 + j]], "want": [0]})
        steps.append({"step": len(steps), "entries": ent, "end": (["c"] if j == 2 else []) + (["e"] if j == 5 else [])})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out",
                        str(out), "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    seq["a2"] = seq["a"]
    full = {k: oracle_logits(cfg, cpu, v) for k, v in seq.items()}
    at = {k: 0 for k in seq}
    tol = TOL[getattr(torch, dtype)]
    for s in steps:
        want = []
        for e in s["entries"]:
            want += [full[e["id"]][at[e["id"]] + w] for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        path = out / f"{s['step']}.f32"
        if not want:
            assert not path.exists()
            continue
        import numpy as np
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(want), 80).copy())
        assert err(got, torch.stack(want)) < tol, s["step"]
