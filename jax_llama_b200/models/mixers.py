"""Sequence mixers of the hybrid decoder family, each a small class over the kernels of `ops/seq_kernels.py`.

A mixer owns its projection weights in kernel layout (projections that read the same input are stacked into one
matrix, so a layer issues one GEMM for them), knows what it keeps between tokens (a key / value cache, a recurrent
state, or nothing of its own when it reads another layer's cache) and turns the normalised input ``h [B·S, width]``
into the input of the output projection.  Constants of a mechanism (rotary share and base, score scale, decay
temperature, which norms and gates are on) are parameters of its spec (`config.py`), not of the code.

The output projection, the norms around the sublayer and the residual sum belong to the layer stack
(`models/hybrid_engine.py`), which is the same for every mixer.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from ..config import AttentionMixerSpec, GlaMixerSpec, LatentAttentionMixerSpec, RetentionMixerSpec, RotaryScaling
from ..ops import _lib
from ..ops import kernels as K
from ..ops import seq_kernels as SK


def _stack_rows(parts: List[torch.Tensor], multiple: int = 8) -> Tuple[torch.Tensor, List[int]]:
    """Concatenate weight matrices [n_i, K] on the output axis, zero-padded to a multiple of `multiple` rows (the
    tensor-core GEMM wants N % 8 == 0).  Returns the matrix and the first row of every part."""
    offs, n = [], 0
    for p in parts:
        offs.append(n)
        n += p.shape[0]
    pad = (-n) % multiple
    if pad:
        parts = parts + [torch.zeros((pad, parts[0].shape[1]), dtype=parts[0].dtype, device=parts[0].device)]
    return torch.cat(parts, 0).contiguous(), offs


def rotary_frequencies(dims: int, base: float, scaling: Optional[RotaryScaling] = None) -> Tuple[torch.Tensor, float]:
    """float64 frequencies base^(-2i/dims), i < dims/2, and the factor on cos / sin.  With `scaling`: the channel index
    at which `original` positions make t turns is n(t) = dims · ln(original / (2π t)) / (2 ln base); channels below
    floor(n(fast)) keep their frequency, channels above ceil(n(slow)) are divided by `factor`, linear ramp between."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling is None:
        return freq, 1.0

    def channel_of(turns: float) -> float:
        return dims * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(channel_of(scaling.fast)), 0)
    hi = min(math.ceil(channel_of(scaling.slow)), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / scaling.factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(scaling.factor) + 1.0


def rotary_table(dims: int, base: float, length: int, device: torch.device, scaling: Optional[RotaryScaling] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of position · frequency for the dims/2 channel pairs, as fp32 [length, dims/2] (angles formed in
    float64; the scaling's factor on cos / sin is in the table)."""
    freq, mult = rotary_frequencies(dims, base, scaling)
    ang = torch.arange(length, dtype=torch.float64)[:, None] * freq[None, :]
    return ((torch.cos(ang) * mult).float().to(device).contiguous(),
            (torch.sin(ang) * mult).float().to(device).contiguous())


class AttentionMixer:
    """Softmax attention: grouped key / value heads, query / key size `dim` and value size `vdim` (they may differ),
    rotary embedding on the first `rot.dims` channels, optional unit-RMS q / k, optional sigmoid gate per head,
    optional reuse of another layer's cache (`kv_from`)."""

    kind = "attention"

    def __init__(self, spec: AttentionMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.shares_kv = spec.kv_from is not None
        parts = [w["q"]] + ([] if self.shares_kv else [w["k"], w["v"]]) + ([w["g"]] if spec.head_gate else [])
        self.w_in, offs = _stack_rows(parts)
        self.q_off = offs[0]
        self.k_off, self.v_off = (-1, -1) if self.shares_kv else (offs[1], offs[2])
        self.g_off = offs[-1] if spec.head_gate else -1
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype
        self._decode_plans: Dict[Tuple[int, int], Tuple[int, Optional[torch.Tensor]]] = {}

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        if self.shares_kv:
            return None
        s = self.spec
        return (torch.zeros((batch, s.kv_heads, length, s.dim), dtype=self.dtype, device=device),
                torch.zeros((batch, s.kv_heads, length, s.vdim), dtype=self.dtype, device=device))

    def new_state(self, batch: int, device: torch.device) -> Optional[torch.Tensor]:
        return None

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Tuple[torch.Tensor, torch.Tensor]
            ) -> torch.Tensor:
        s = self.spec
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | gate]
        q = torch.empty((B * S, s.heads * s.dim), dtype=self.dtype, device=h.device)
        src = layer if not self.shares_kv else s.kv_from
        kc, vc = cache.ks[src], cache.vs[src]
        rot = s.rot.dims if s.rot is not None else 0
        SK.attn_prep(y, self.q_off, self.k_off, self.v_off, q, None if self.shares_kv else kc,
                     None if self.shares_kv else vc, rope[0], rope[1], rot, s.qk_unit_norm, self.eps, cache.len_dev,
                     cache.pad_left, B, S, s.heads, s.kv_heads, s.dim, s.vdim)
        gate = y[:, self.g_off:self.g_off + s.heads] if s.head_gate else None
        if self._library_shape():
            # 64- / 128-wide heads in bfloat16 are the shapes the LLaMA kernels are built for: the tcgen05 flash kernel
            # for prompts, the split-KV kernel for one new token; both take the score scale as an argument
            out = self._attend_shared_kernels(q, kc, vc, cache, B, S)
            if gate is not None:
                SK.head_gate(out, gate, s.heads, s.vdim)
            return out
        return SK.attn_generic(q, kc, vc, gate, cache.len_dev, cache.pad_left, B, S, s.heads, s.scale)

    def _library_shape(self) -> bool:
        s = self.spec
        return (SK.tensor_cores_enabled() and self.dtype == torch.bfloat16 and s.dim == s.vdim and s.dim in (64, 128)
                and s.heads // s.kv_heads in (1, 2, 4, 8))

    def _attend_shared_kernels(self, q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, cache: "object", B: int, S: int
                               ) -> torch.Tensor:
        s = self.spec
        L = _lib.lib()
        out = torch.empty((B * S, s.heads * s.vdim), dtype=self.dtype, device=q.device)
        T = kc.shape[2]
        if S > 1:
            _lib.check(L.jl_flash_prefill(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cache.len_dev.data_ptr(),
                                          cache.pad_left.data_ptr(), out.data_ptr(), B, S, s.heads, s.kv_heads, s.dim, T,
                                          int(cache.index), float(s.scale), K._stream()), "jl_flash_prefill")
            return out
        key = (B, T)
        if key not in self._decode_plans:
            self._decode_plans[key] = K.decode_attn_plan(B, s.heads, s.kv_heads, s.dim, T, q.device)
        splits, scratch = self._decode_plans[key]
        _lib.check(L.jl_decode_attn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cache.len_dev.data_ptr(),
                                    cache.pad_left.data_ptr(), K._p(scratch), out.data_ptr(), B, s.heads, s.kv_heads, s.dim,
                                    T, 1, float(s.scale), splits, 0, K._stream()), "jl_decode_attn")
        return out


class GlaMixer:
    """Gated linear attention: S_t = diag(alpha_t) S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t per head, alpha from a low-rank
    projection through sigmoid(·)^(1/tau); read-out normalised per head (plain weight shared by the heads), gated by
    silu of a projection of the input.  The state is fp32 and is what the layer keeps between tokens."""

    kind = "gla"

    def __init__(self, spec: GlaMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.w_in, offs = _stack_rows([w["q"], w["k"], w["v"], w["g"], w["a1"]])
        self.q_off, self.k_off, self.v_off, self.g_off, self.a_off = offs
        self.a2 = w["a2"].contiguous()
        self.a2_bias = w["a2.b"].contiguous()
        self.norm = w["norm"].contiguous()
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.a2, self.a2_bias, self.norm, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> None:
        return None

    def new_state(self, batch: int, device: torch.device) -> torch.Tensor:
        s = self.spec
        return torch.zeros((batch, s.heads, s.dim, s.vdim), dtype=torch.float32, device=device)

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Optional[Tuple] = None
            ) -> torch.Tensor:
        s = self.spec
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | gate | low-rank decay input]
        o = SK.gla_scan(y, self.q_off, self.k_off, self.v_off, self.a_off, self.a2, self.a2_bias, cache.states[layer],
                        cache.len_dev, cache.pad_left, B, S, s.heads, s.dim, s.vdim, s.dim ** -0.5, s.tau)
        gate = y[:, self.g_off:self.g_off + s.heads * s.vdim]
        return SK.headnorm_gate(o, self.norm, gate, s.heads, s.vdim, self.eps, SK.ACT_SILU)


class LatentAttentionMixer:
    """Softmax attention through low-rank latents.  Per token the layer keeps one row [normed key/value latent | rotated
    key part shared by the heads]; nothing per head.

    One token at a time (and prompt portions that continue a cache) the keys' and values' up-projections are applied on
    the query side: with q_h = [r_h | a_h] (rotated | unrotated) the score a_h · (U_h c) + r_h · k_rot equals
    (U_hᵀ a_h) · c + r_h · k_rot, and Σ p_j (V_h c_j) = V_h (Σ p_j c_j) — so the attention runs over the cached rows with
    one shared key/value head of width kv_rank + rot_dim (keys) and kv_rank (values), and two per-head batched products
    map into and out of the latent: every cached row is read once for all heads.

    A prompt that starts a sequence projects its latents up instead (two tensor-core GEMMs for all heads) and attends
    with per-head keys [k_rot | U_h c] and values V_h c in token-major layout, which costs a third of the arithmetic of
    the latent-space form at these head sizes.  Both forms run the windowed generic attention kernel.

    Internally a query head is laid out [rot_dim rotated | dim unrotated] (the rows of the query up-projection are
    permuted once at load), so that the rotation applies to the leading channels of a head as in the other mixers."""

    kind = "latent_attention"

    def __init__(self, spec: LatentAttentionMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        s = spec
        self.w_in, offs = _stack_rows([w["dq"], w["dkv"]])
        self.q_off, self.kv_off = offs
        self.q_norm, self.kv_norm = w["dq.norm"].contiguous(), w["dkv.norm"].contiguous()
        uq = w["uq"].view(s.heads, s.dim + s.rot_dim, s.q_rank)                 # stored [dim unrotated | rot_dim rotated]
        self.uq = torch.cat([uq[:, s.dim:], uq[:, :s.dim]], 1).reshape(s.heads * (s.dim + s.rot_dim), s.q_rank).contiguous()
        self.uk_t = w["uk"].view(s.heads, s.dim, s.kv_rank).transpose(1, 2).contiguous()    # [H, kv_rank, dim]
        self.uv = w["uv"].view(s.heads, s.vdim, s.kv_rank).contiguous()          # [H, vdim, kv_rank]
        self.w_kv, kv_offs = _stack_rows([w["uk"], w["uv"]])                     # [H·dim | H·vdim, kv_rank]: prompts
        self.v_col = kv_offs[1]
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype
        self.row = s.kv_rank + s.rot_dim

    def weights(self) -> List[torch.Tensor]:
        """What a decode step streams (the stacked up-projection of prompts holds the same values once more)."""
        return [self.w_in, self.q_norm, self.kv_norm, self.uq, self.uk_t, self.uv, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> Tuple[torch.Tensor, None]:
        return torch.zeros((batch, length, self.row), dtype=self.dtype, device=device), None

    def new_state(self, batch: int, device: torch.device) -> Optional[torch.Tensor]:
        return None

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Tuple[torch.Tensor, torch.Tensor]
            ) -> torch.Tensor:
        s = self.spec
        M, H, qd = B * S, s.heads, s.dim + s.rot_dim
        rot = s.rot.dims if s.rot is not None else 0
        layout = SK.ROT_LAYOUTS[s.rot.layout] if s.rot is not None else 0
        kc = cache.ks[layer]                                                   # [B, T, kv_rank + rot_dim]
        starts = S > 1 and int(cache.index) == 0                               # a prompt from an empty cache
        y = SK.linear(h, self.w_in)                                            # fp32 [M, query latent | kv latent | key part]
        cq, c_new, kr_new = SK.latent_prep(y, self.q_off, s.q_rank, self.kv_off, s.kv_rank, s.rot_dim, rot, layout,
                                           self.q_norm, self.kv_norm, kc, rope[0], rope[1], self.eps, cache.len_dev,
                                           cache.pad_left, B, S, token_major=starts)
        q = SK.linear(cq, self.uq, out_f32=False)                              # [M, H·(rot_dim + dim)]
        if starts:
            return self._attend_projected(q, c_new, kr_new, cache, B, S, rot, layout, rope)
        qa = torch.empty((M, H * self.row), dtype=self.dtype, device=h.device)
        a = q[:, s.rot_dim:] if s.rot_dim else q                               # head h's unrotated part starts at h·qd
        SK.linear_batched(a, self.uk_t, qa, nbatch=H, rows=M, x_bs=qd, o_bs=self.row)      # U_hᵀ a_h
        if s.rot_dim:
            SK.rotary_slice(q, qd, 0, qa, self.row, s.kv_rank, H, s.rot_dim, rot, layout, rope[0], rope[1],
                            cache.len_dev, cache.pad_left, B, S)
        ctx = SK.attn_windowed(qa, kc, kc, cache.len_dev, cache.pad_left, B, S, H, 1, self.row, s.kv_rank, kc.shape[1],
                               self.row, self.row, s.window, s.scale)         # [M, H·kv_rank]
        out = torch.empty((M, H * s.vdim), dtype=self.dtype, device=h.device)
        SK.linear_batched(ctx, self.uv, out, nbatch=H, rows=M, x_bs=s.kv_rank, o_bs=s.vdim)
        return out

    def _attend_projected(self, q: torch.Tensor, c_new: torch.Tensor, kr_new: torch.Tensor, cache: "object", B: int, S: int,
                          rot: int, layout: int, rope: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
        """Per-head keys and values of the S new tokens of every row, token-major; slot == index within the prompt."""
        s = self.spec
        M, H, qd = B * S, s.heads, s.dim + s.rot_dim
        kv = SK.linear(c_new, self.w_kv, out_f32=False)                        # [M, H·dim | H·vdim (| padding)]
        qf = torch.empty_like(q)
        SK.rotary_slice(q, qd, 0, qf, qd, 0, H, qd, rot, layout, rope[0], rope[1], cache.len_dev, cache.pad_left, B, S)
        kf = torch.empty((M, H * qd), dtype=self.dtype, device=q.device)       # [M, H, rot_dim | dim]
        if s.rot_dim:
            SK.rotary_slice(kr_new, 0, 0, kf, qd, 0, H, s.rot_dim, 0, 0, rope[0], rope[1], cache.len_dev, cache.pad_left, B, S)
        SK.rotary_slice(kv, s.dim, 0, kf, qd, s.rot_dim, H, s.dim, 0, 0, rope[0], rope[1], cache.len_dev, cache.pad_left, B, S)
        v = kv[:, self.v_col:]
        ldv = kv.stride(0)
        return SK.attn_windowed(qf, kf, v, cache.len_dev, cache.pad_left, B, S, H, H, qd, s.vdim, S, H * qd, ldv, s.window,
                                s.scale, strides=(S * H * qd, qd, S * ldv, s.vdim))


class RetentionMixer:
    """Retention: linear attention with one fixed decay per head, S_t = decay_h S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t, rotary
    q / k, k scaled by dim^(-1/2) after the rotation; every head's read-out divided by its RMS (no weight) and gated by
    silu of a projection of the input.  The fp32 state is what the layer keeps between tokens."""

    kind = "retention"

    def __init__(self, spec: RetentionMixerSpec, w: Dict[str, torch.Tensor], eps: float):
        self.spec, self.eps = spec, float(eps)
        self.w_in, offs = _stack_rows([w["q"], w["k"], w["v"], w["g"]])
        self.q_off, self.k_off, self.v_off, self.g_off = offs
        self.wo = w["o"].contiguous()
        self.dtype = self.wo.dtype
        self.decay = torch.tensor([float(a) for a in spec.decay], dtype=torch.float64).to(torch.float32).to(self.wo.device)

    def weights(self) -> List[torch.Tensor]:
        return [self.w_in, self.wo]

    def new_cache(self, batch: int, length: int, device: torch.device) -> None:
        return None

    def new_state(self, batch: int, device: torch.device) -> torch.Tensor:
        s = self.spec
        return torch.zeros((batch, s.heads, s.dim, s.vdim), dtype=torch.float32, device=device)

    def run(self, h: torch.Tensor, B: int, S: int, cache: "object", layer: int, rope: Tuple[torch.Tensor, torch.Tensor]
            ) -> torch.Tensor:
        s = self.spec
        rot = s.rot.dims if s.rot is not None else 0
        layout = SK.ROT_LAYOUTS[s.rot.layout] if s.rot is not None else 0
        y = SK.linear(h, self.w_in)                                   # fp32 [M, q | k | v | gate]
        o = SK.retention_scan(y, self.q_off, self.k_off, self.v_off, self.decay, rope[0], rope[1], rot, layout,
                              s.dim ** -0.5, cache.states[layer], cache.len_dev, cache.pad_left, B, S, s.heads, s.dim,
                              s.vdim)
        gate = y[:, self.g_off:self.g_off + s.heads * s.vdim]
        return SK.headnorm_gate(o, None, gate, s.heads, s.vdim, self.eps, SK.ACT_SILU, dtype=self.dtype)


MIXERS = {"attention": AttentionMixer, "gla": GlaMixer, "latent_attention": LatentAttentionMixer,
          "retention": RetentionMixer}

