"""Folirax on the hybrid engine against the plain float64 statement of the design (`folirax_oracle.py`).

Small configurations with random weights; every test builds its own.  The float32 engine is held to a tight bound,
the bfloat16 engine to the error that rounding its operands causes.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from jax_llama_b200.config import FoliraxConfig                              # noqa: E402
from jax_llama_b200.generation import LLaMA                                  # noqa: E402
from jax_llama_b200.models.folirax import FoliraxForCausalLM                 # noqa: E402
from jax_llama_b200.models.hybrid_engine import HybridEngine, random_tensors  # noqa: E402
from jax_llama_b200.ops import seq_kernels as SK                             # noqa: E402
from jax_llama_b200.tokenizers import IdTokenizer                            # noqa: E402

from tests import folirax_oracle as O                                        # noqa: E402

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def gla(heads=2, dim=16, vdim=24, tau=8.0, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def attn(heads=4, kv_heads=2, dim=24, vdim=40, rot=12, base=10000.0, scale=0.2, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"dims": rot, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def ff(n):
    return {"kind": "dense", "ff": n}


def config(layers, vocab=96, width=72, eps=1e-5, scale=0.7, cap=9.0):
    return FoliraxConfig.from_dict({"architecture": "Folirax", "vocab": vocab, "width": width, "norm": {"eps": eps},
                                    "logit_scale": scale, "logit_softcap": cap, "layers": layers})


MIXED = [gla(), attn(mlp=ff(56)), attn(kv_from=1, mlp=ff(56)), gla(heads=3, dim=48, vdim=16, tau=2.0, mlp=ff(40))]


def build(cfg, dtype, seed=0, rank=4, graph=True, tweak=None):
    tensors = random_tensors(cfg, "cuda", seed, decay_rank=rank)
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


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 100, 256])
def test_norms(dtype, width):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(5, width, device="cuda", generator=g) * 3
    y = torch.randn(5, width, device="cuda", generator=g)
    w1 = (0.2 * torch.randn(width, device="cuda", generator=g)).to(dtype)
    w2 = (0.2 * torch.randn(width, device="cuda", generator=g)).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    h = SK.norm_f32(x, w1, 1e-5, 1.0)
    want = O.norm_zero_centred(x.double().cpu(), w1.cpu(), 1e-5)
    assert (h.double().cpu() - want).abs().max() < tol * want.abs().max()
    plain = SK.norm_f32(x, w1, 1e-5, 0.0)
    assert (plain.double().cpu() - O.rms_unit(x.double().cpu(), 1e-5) * w1.double().cpu()).abs().max() < tol * 4
    x2 = x.clone()
    hn = SK.postnorm_add(y, w1, x2, 1e-5, 1.0, w_next=w2)
    want_x = x.double().cpu() + O.norm_zero_centred(y.double().cpu(), w1.cpu(), 1e-5)
    assert (x2.double().cpu() - want_x).abs().max() < 1e-5 * want_x.abs().max()
    want_h = O.norm_zero_centred(want_x, w2.cpu(), 1e-5)
    assert (hn.double().cpu() - want_h).abs().max() < tol * want_h.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 40, 72), (3, 33, 100), (8, 96, 64), (9, 104, 72), (70, 56, 328), (200, 264, 136),
                                   (130, 50, 72)])
def test_linear_paths(dtype, shape):
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(dtype)
    want = x.double().cpu() @ w.double().cpu().T
    tol = 1e-5 if dtype == torch.float32 else 2e-3          # operands are exact in both; the sums are fp32
    for tc in (False, True):
        got = SK.linear(x, w, tensor_cores=tc)
        assert got.dtype == torch.float32
        assert (got.double().cpu() - want).abs().max() < tol * want.abs().max(), (tc, shape)
    r2 = SK.linear(x, w, act=SK.ACT_RELU2, out_f32=False)
    assert r2.dtype == dtype
    assert (r2.double().cpu() - O.relu_squared(want)).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2) * want.abs().max() ** 2
    cap = SK.linear(x, w, act=SK.ACT_SCALE_SOFTCAP, p0=0.5, p1=2.0)
    assert (cap.double().cpu() - 2.0 * torch.tanh(want * 0.5 / 2.0)).abs().max() < tol * 4
    gl = SK.linear(x, w, act=SK.ACT_GELU_TANH)
    assert (gl.double().cpu() - O.gelu_tanh(want)).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layers", [[gla()], [gla(heads=1, dim=80, vdim=8, tau=1.0)], [gla(heads=3, dim=48, vdim=40, tau=64.0, mlp=ff(24))],
                                    [gla(heads=1, dim=272, vdim=6, tau=4.0)],
                                    [attn()], [attn(heads=2, kv_heads=2, dim=16, vdim=16, rot=16, mlp=ff(32))],
                                    [attn(heads=6, kv_heads=1, dim=40, vdim=72, rot=2, scale=1.0)],
                                    [attn(), attn(kv_from=0)]],
                         ids=["gla", "gla-wide-key-tau1", "gla-3h-mlp", "gla-key272", "attn-gqa", "attn-full-rot-mlp", "attn-mqa-rot2", "attn-shared-kv"])
def test_single_mechanism_models(dtype, layers):
    cfg = config(layers)
    eng, cpu = build(cfg, dtype, seed=3)
    toks = tokens(45, cfg.vocab_size, 5)
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got, oracle_logits(cfg, cpu, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_stream_after_every_layer(dtype):
    cfg = config(MIXED)
    eng, cpu = build(cfg, dtype, seed=2)
    toks = tokens(19, cfg.vocab_size, 9)
    eng.capture_streams = []
    eng.forward(torch.tensor([toks], device="cuda"))
    _, want = O.forward(cfg.to_dict(), cpu, toks, return_layers=True)
    tol = 1e-4 if dtype == torch.float32 else 5e-2
    for i, x in enumerate(eng.capture_streams):
        assert (x.double().cpu() - want[i]).abs().max() < tol * want[i].abs().max(), i


def test_other_constants():
    """Values that one model may happen to make equal or one: no soft cap, logit scale 1, tau 1, scale 1, one head,
    kv_heads == heads, rot.dims == dim, eps large, layers in another order (attention first, shared keys far below)."""
    layers = [attn(heads=1, kv_heads=1, dim=32, vdim=32, rot=32, scale=1.0, base=100.0), gla(heads=1, dim=32, vdim=32, tau=1.0),
              gla(mlp=ff(64)), attn(heads=1, kv_heads=1, dim=32, vdim=32, rot=32, scale=1.0, base=100.0, kv_from=0)]
    cfg = config(layers, vocab=130, width=64, eps=1e-2, scale=1.0, cap=0.0)
    eng, cpu = build(cfg, torch.float32, seed=11, rank=2)
    toks = tokens(70, cfg.vocab_size, 2)
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got, oracle_logits(cfg, cpu, toks)) < TOL[torch.float32]


# ------------------------------------------------------------------------------------------ prefill vs decoding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("prompt", [1, 2, 31, 33])
def test_decode_matches_prefill_and_oracle(dtype, prompt):
    """The prompt in one step, then 70 tokens one by one through the graph-replayed step: the 32-key blocks of the
    attention kernels and the first tokens of a sequence are all crossed."""
    cfg = config(MIXED)
    eng, cpu = build(cfg, dtype, seed=4)
    toks = tokens(prompt + 70, cfg.vocab_size, prompt)
    want = oracle_logits(cfg, cpu, toks)
    ids = torch.tensor([toks[:prompt]], device="cuda")
    stream = eng.begin_stream(ids, None, max_length=len(toks) + 1, eos_token_id=-1,
                              logit_rows=torch.arange(prompt))
    assert err(stream.prompt_logits(), want[:prompt]) < TOL[dtype]
    rows = []
    for t in toks[prompt:]:
        stream.step(torch.tensor([t], dtype=torch.int32).pin_memory())
        rows.append(stream.logits()[0].clone())
    assert err(torch.stack(rows), want[prompt:]) < TOL[dtype]
    stream.close()
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole, want) < TOL[dtype]
    if dtype == torch.float32:
        assert err(torch.stack(rows), whole[prompt:]) < 5e-5


def run_unequal_batch(cfg, dtype, lens, extra, seed):
    """Left-padded batch of prompts of the given lengths, then `extra` tokens decoded together; every row is compared
    with the oracle run of that request alone."""
    eng, cpu = build(cfg, dtype, seed=seed)
    seqs = [tokens(n + extra, cfg.vocab_size, 20 + n) for n in lens]
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
        stream.step(torch.tensor([s[n + j] for n, s in zip(lens, seqs)], dtype=torch.int32).pin_memory())
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
    """Prompts of 1, 7 and 40 tokens in one batch: padding must touch neither the recurrent state nor the visible keys
    nor the positions."""
    run_unequal_batch(config(MIXED), dtype, [1, 7, 40], 36, seed=6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_odd_sizes_and_a_batch_of_ten(dtype):
    """Sizes that fit no vector width or tile (width 90, heads of 10 / 14 / 12 channels, 3 query heads on 1 key head, vocab
    77) in a batch of ten unequal requests: more rows than the weight-streaming kernel takes, so decoding runs the GEMMs."""
    layers = [attn(heads=3, kv_heads=1, dim=10, vdim=14, rot=6, scale=0.4, mlp=ff(50)), gla(heads=3, dim=12, vdim=10, tau=3.0),
              attn(heads=3, kv_heads=1, dim=10, vdim=14, rot=6, scale=0.4, kv_from=0)]
    cfg = config(layers, vocab=77, width=90)
    run_unequal_batch(cfg, dtype, [3, 17, 1, 9, 30, 2, 12, 25, 8, 21], 12, seed=17)


@pytest.mark.parametrize("prompt", [2, 9])
def test_wide_heads_short_prompts(prompt):
    a = dict(heads=2, kv_heads=1, dim=128, vdim=128, rot=64, scale=0.09)
    cfg = config([attn(**a), attn(**a, kv_from=0, mlp=ff(64))], width=128)
    run_unequal_batch(cfg, torch.bfloat16, [prompt], 5, seed=19)


@pytest.mark.parametrize("dim", [64, 128])
def test_wide_heads_on_the_shared_attention_kernels(dim):
    """64- and 128-wide heads in bfloat16 run the tcgen05 / split-KV attention kernels the LLaMA models use, with this
    design's score scale, unit-norm q / k, gates and shared keys around them: unequal batch across the 128-query tiles."""
    a = dict(heads=4, kv_heads=2, dim=dim, vdim=dim, rot=dim // 2, scale=0.11)
    cfg = config([attn(**a), gla(), attn(**a, kv_from=0, mlp=ff(64))], width=128)
    run_unequal_batch(cfg, torch.bfloat16, [5, 150, 131], 40, seed=13)


def test_state_and_cache_are_clean_when_used_again():
    """The same decode state serves request after request: a second, shorter request must see nothing of the first
    (recurrent state zeroed, old keys invisible, old left-pad counts gone)."""
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
    """Embedding rows that are unit vectors: token -> channel.  With a zero norm weight the mixer then sees exactly one
    column of each projection for such a token (all values exact in bfloat16)."""
    for tok, ch in token_channel.items():
        t["embed"][tok] = 0
        t["embed"][tok, ch] = 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 63, 64, 290])
def test_one_far_key_decides(dtype, far):
    """An attention-only model with a sharp softmax (large score scale).  Token A's key is made equal to token B's
    query (one column of W_k copied from W_q), so when B is the last token and A stands once at position `far`, that
    single key takes nearly all the weight among 300 random ones: a kernel that drops or misplaces it (edges of the
    32-key blocks, the first slots, hundreds back) moves the logits far beyond the tolerance.  Checked in a prompt and
    with the query decoded alone."""
    A, B = 61, 60
    cfg = config([attn(heads=2, kv_heads=1, dim=32, vdim=24, rot=8, scale=2.0, base=1e6)], vocab=64, width=48)

    def tweak(t):
        t["l0.norm1"].zero_()
        _unit_rows(t, {B: 0, A: 1})
        t["l0.mix.k"][:, 1] = t["l0.mix.q"][:32, 0]
    eng, cpu = build(cfg, dtype, seed=5, tweak=tweak)
    n = 300
    toks = [2 + (i % 50) for i in range(n)]
    toks[far] = A
    toks.append(B)
    want = oracle_logits(cfg, cpu, toks)
    without = list(toks)
    without[far] = 59
    assert err(oracle_logits(cfg, cpu, without)[-1:], want[-1:]) > 10 * TOL[dtype]      # the planted key matters
    whole = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(whole[-1:], want[-1:]) < TOL[dtype]
    stream = eng.begin_stream(torch.tensor([toks[:-1]], device="cuda"), None, max_length=n + 4, eos_token_id=-1)
    stream.step(torch.tensor([toks[-1]], dtype=torch.int32).pin_memory())
    assert err(stream.logits()[:1], want[-1:]) < TOL[dtype]
    stream.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gap", [1, 7, 8, 9, 216])
def test_recurrent_state_keeps_a_far_token(dtype, gap):
    """Gated linear attention with slow decays.  The filler token has a zero key (its embedding channel is cut out of
    W_k), so the state holds only what the one planted token wrote `gap` steps back, and the read-out at the end is that
    token's value: a state that is lost, reset or decayed wrongly at an edge of the scan's token chunks shows at once.
    Checked in a prompt and with the tail decoded token by token."""
    filler, planted = 5, 40
    cfg = config([gla(heads=2, dim=16, vdim=16, tau=16.0)], vocab=64, width=48)

    def tweak(t):
        t["l0.norm1"].zero_()
        _unit_rows(t, {filler: 3})
        t["l0.mix.k"][:, 3] = 0
        t["l0.mix.a2.b"].fill_(6.0)
        t["l0.mix.a2"].mul_(0.05)
    eng, cpu = build(cfg, dtype, seed=7, tweak=tweak)
    n = 230
    toks = [filler] * n
    toks[n - 1 - gap] = planted
    want = oracle_logits(cfg, cpu, toks)
    other = list(toks)
    other[n - 1 - gap] = planted + 1
    assert err(oracle_logits(cfg, cpu, other)[-1:], want[-1:]) > 10 * TOL[dtype]
    got = eng.forward(torch.tensor([toks], device="cuda")).logits[0]
    assert err(got[n - 1 - gap:], want[n - 1 - gap:]) < TOL[dtype]
    cut = 10
    stream = eng.begin_stream(torch.tensor([toks[:cut]], device="cuda"), None, max_length=n + 2, eos_token_id=-1)
    rows = []
    for t in toks[cut:]:
        stream.step(torch.tensor([t], dtype=torch.int32).pin_memory())
        rows.append(stream.logits()[0].clone())
    stream.close()
    assert err(torch.stack(rows)[n - 1 - gap - cut:], want[n - 1 - gap:]) < TOL[dtype]


# ------------------------------------------------------------------------------------------ the framework's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_front_end(dtype, tmp_path):
    """save_pretrained → registry → `LLaMA.generate_from_str` (left-padded batch, scheduler, on-device arg-max): every
    generated token is the oracle's arg-max given its prefix, up to near-ties."""
    from jax_llama_b200.models import registry

    cfg = config(MIXED, vocab=80)
    model = FoliraxForCausalLM(cfg, dtype=dtype, seed=12, _do_init=True)
    model.save_pretrained(str(tmp_path))
    assert registry.resolve(str(tmp_path))[0] == "folirax"
    loaded = registry.load_pretrained(str(tmp_path), dtype=dtype, device="cuda")
    assert isinstance(loaded, FoliraxForCausalLM) and loaded.config.to_dict() == cfg.to_dict()
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
    import os
    import subprocess
    import sys

    cfg = config(MIXED, vocab=80)
    FoliraxForCausalLM(cfg, seed=3, _do_init=True).save_pretrained(str(tmp_path))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "example.py"), "--model_dir", str(tmp_path), "--prompt",
                        "7 8 9", "--prompt", "40", "--max_gen_len", "6", "--temperature", "0"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip() and not l.startswith("=")]
    assert lines[0].split()[:4] == ["1", "7", "8", "9"] and lines[1].split()[:2] == ["1", "40"]
    assert all(0 <= int(t) < 80 for l in lines[:2] for t in l.split())
