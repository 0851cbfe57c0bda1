"""Plain, slow statement of the Nikonex design, one function per mechanism, token by token where the design is recurrent.

Independent of the package: it takes a config dictionary (the keys of a Nikonex ``config.json``) and a dictionary of
tensors under their checkpoint names, and computes everything in float64 (weights keep the values they were stored
with), so that it can judge both the bfloat16 and the float32 kernels.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w.to(F64)


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------ rotary embedding
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    """Frequencies f_i = base^(-2i/dims), i < dims/2, and the factor on cos / sin.  With `scaling` (factor, original,
    fast, slow) slow channels are divided by `factor`, fast ones stay, with a linear ramp between the channel indices
    at which `original` positions make `fast` and `slow` turns; cos and sin grow by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float, layout: str, scaling: Optional[dict] = None
           ) -> torch.Tensor:
    """x [T, heads, n]; the first `dims` channels of every head are turned pairwise by the angle pos * f_i.
    layout "interleaved": channel 2i with 2i+1; "half": channel i with i + dims/2.  The rest pass through."""
    f, mult = rotary_frequencies(dims, base, scaling)
    ang = pos.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        half = dims // 2
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------ mixers
def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int = 0,
                     past: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Softmax attention whose queries and keys / values pass through low-rank latents, with one rotated key part
    shared by the heads and a sliding window.  h [T, width] at positions pos0 .. pos0+T-1; `past` = (latents, rotated
    key parts) of the positions before.  Returns (out [T, width], (latents, rotated key parts) of all positions)."""
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    T = h.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    cq = norm_plain(h @ w["dq"].to(F64).T, w["dq.norm"], eps)
    q = (cq @ w["uq"].to(F64).T).view(T, H, D + R)
    q_plain = q[..., :D]
    q_rot = rotate(q[..., D:], pos, rot["dims"], rot["base"], "interleaved", rot.get("scaling"))
    kv = h @ w["dkv"].to(F64).T
    c = norm_plain(kv[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate(kv[:, None, rank:], pos, rot["dims"], rot["base"], "interleaved", rot.get("scaling"))[:, 0]
    if past is not None:
        c, k_rot = torch.cat([past[0], c]), torch.cat([past[1], k_rot])
    k_plain = (c @ w["uk"].to(F64).T).view(-1, H, D)
    v = (c @ w["uv"].to(F64).T).view(-1, H, V)
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        i = pos0 + t
        j0 = 0 if window is None else max(0, i - int(window) + 1)
        for hh in range(H):
            sc = (k_plain[j0:i + 1, hh] @ q_plain[t, hh] + k_rot[j0:i + 1] @ q_rot[t, hh]) * m["scale"]
            p = torch.softmax(sc, 0)
            out[t, hh] = p @ v[j0:i + 1, hh]
    return out.reshape(T, H * V) @ w["o"].to(F64).T, (c, k_rot)


def retention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int = 0,
              state: Optional[torch.Tensor] = None):
    """Linear attention with one fixed decay per head, token by token: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.
    Returns (out [T, width], final state [heads, dim, vdim])."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    T = h.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    q = rotate((h @ w["q"].to(F64).T).view(T, H, D), pos, rot["dims"], rot["base"], "half", rot.get("scaling"))
    k = rotate((h @ w["k"].to(F64).T).view(T, H, D), pos, rot["dims"], rot["base"], "half", rot.get("scaling"))
    k = k * D ** -0.5
    v = (h @ w["v"].to(F64).T).view(T, H, V)
    decay = torch.tensor([float(d) for d in m["decay"]], dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * V) * silu(h @ w["g"].to(F64).T)
    return o @ w["o"].to(F64).T, S


# ------------------------------------------------------------------------------------------ feed-forward
def route(h: torch.Tensor, w_router: torch.Tensor, r: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    """Experts and weights of every token: sigmoid scores; only experts of the `groups.keep` best groups (a group's
    score is the sum of its two largest scores) can be chosen; the `top` largest of those; weights = their scores
    over their sum, times `scale`.  Returns (indices [T, top], weights [T, top])."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ w_router.to(F64).T)                       # [T, E]
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        sg = s.view(-1, n, per)
        gscore = sg.topk(min(2, per), -1).values.sum(-1)            # [T, n]
        best = gscore.topk(keep, -1).indices
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, best, True)
        allowed = gmask[:, :, None].expand(-1, -1, per).reshape(-1, E)
    idx = s.masked_fill(~allowed, -1.0).topk(top, -1).indices
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))


def expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return relu_squared(h @ up.to(F64).T) @ down.to(F64).T


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    """Weighted sum of each token's chosen experts plus the shared expert times a per-token sigmoid gate."""
    idx, wt = route(h, w["router"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            out[t] += a * expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w["shared.sg"].to(F64).T)          # [T, 1]
        out = out + gate * expert(h, w["shared.up"], w["shared.down"])
    return out


# ------------------------------------------------------------------------------------------ the model
def _sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  `streams` collects the residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    x = tensors["embed"].to(F64)[torch.tensor(tokens)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h1 = norm_plain(x, tensors[p + "norm1"], eps)
        fn = {"latent_attention": latent_attention, "retention": retention}[layer["type"]]
        y, _ = fn(h1, _sub(tensors, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            h2 = norm_plain(x, tensors[p + "norm2"], eps)
            y = y + moe(h2, _sub(tensors, p + "mlp."), layer["mlp"])
        x = x + mult * y
        if streams is not None:
            streams.append(x.clone())
    return norm_plain(x, tensors["final.norm"], eps) @ tensors["head"].to(F64).T


def forward_stepwise(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], cut: int) -> torch.Tensor:
    """The same logits computed as a prompt of `cut` tokens followed by one token at a time, each mixer carrying
    only what the design says it keeps (latents and rotated key parts; the matrix state)."""
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    keep: list = [None] * len(config["layers"])
    rows = []
    bounds = [(0, cut)] + [(t, t + 1) for t in range(cut, len(tokens))]
    for lo, hi in bounds:
        x = tensors["embed"].to(F64)[torch.tensor(tokens[lo:hi])]
        for i, layer in enumerate(config["layers"]):
            p = f"l{i}."
            h1 = norm_plain(x, tensors[p + "norm1"], eps)
            if layer["type"] == "latent_attention":
                y, keep[i] = latent_attention(h1, _sub(tensors, p + "mix."), layer["mixer"], eps, lo, keep[i])
            else:
                y, keep[i] = retention(h1, _sub(tensors, p + "mix."), layer["mixer"], eps, lo, keep[i])
            if layer.get("mlp") is not None:
                y = y + moe(norm_plain(x, tensors[p + "norm2"], eps), _sub(tensors, p + "mlp."), layer["mlp"])
            x = x + mult * y
        rows.append(norm_plain(x, tensors["final.norm"], eps) @ tensors["head"].to(F64).T)
    return torch.cat(rows)
