"""Plain, slow statement of the Folirax design, one function per mechanism, token by token where the design is recurrent.

Independent of the package: it takes a config dictionary (the keys of a Folirax ``config.json``) and a dictionary of
tensors under their checkpoint names, and computes everything in float64 (weights keep the values they were stored
with), so that it can judge both the bfloat16 and the float32 kernels.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_zero_centred(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norm of the design: unit RMS times (1 + w), w stored around zero."""
    return rms_unit(x, eps) * (1.0 + w.to(F64))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def rotate_interleaved(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]; the first `dims` channels of every head are turned pairwise, channel 2i with 2i+1, by the
    angle pos * base^(-2i/dims); the rest pass through."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    ang = pos.to(F64)[:, None] * freq[None, :]                      # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def gla_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
              state: Optional[torch.Tensor] = None):
    """Gated linear attention over h [T, width], token by token.  Returns (out [T, width], final state
    [heads, dim, vdim])."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].to(F64).T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].to(F64).T).view(T, H, D)
    v = (h @ w["v"].to(F64).T).view(T, H, V)
    z = (h @ w["a1"].to(F64).T) @ w["a2"].to(F64).T + w["a2.b"].to(F64)
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * w["norm"].to(F64)
    g = h @ w["g"].to(F64).T
    y = o.reshape(T, H * V) * (g * torch.sigmoid(g))
    return y @ w["o"].to(F64).T, S


def attention_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, pos: torch.Tensor):
    """Keys as a cache holds them (rotated, then unit RMS per head) and values, [T, kv_heads, dim / vdim]."""
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = (h @ w["k"].to(F64).T).view(T, G, D)
    k = rms_unit(rotate_interleaved(k, pos, m["rot"]["dims"], m["rot"]["base"]), eps)
    v = (h @ w["v"].to(F64).T).view(T, G, V)
    return k, v


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, pos: torch.Tensor,
                    k_all: torch.Tensor, v_all: torch.Tensor, key_pos: torch.Tensor) -> torch.Tensor:
    """Softmax attention of the queries of h [T, width] at positions `pos` over keys / values k_all / v_all at
    positions `key_pos` (causal: a query sees keys at positions <= its own), gated per head, projected."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].to(F64).T).view(T, H, D)
    q = rms_unit(rotate_interleaved(q, pos, m["rot"]["dims"], m["rot"]["base"]), eps)
    gate = torch.sigmoid(h @ w["g"].to(F64).T)                      # [T, H]
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k_all[:, g].T) * m["scale"]                 # [T, keys]
        s = s.masked_fill(key_pos[None, :] > pos[:, None], float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v_all[:, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ w["o"].to(F64).T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return relu_squared(h @ w["up"].to(F64).T) @ w["down"].to(F64).T


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] (float64) of one sequence from position 0; optionally the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = torch.arange(T)
    x = tensors["embed"].to(F64)[torch.tensor(tokens)]
    kv: Dict[int, tuple] = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = layer["mixer"]
        h = norm_zero_centred(x, tensors[p + "norm1"], eps)
        w = sub(tensors, p + "mix.")
        if layer["type"] == "gla":
            y, _ = gla_mixer(h, w, m, eps)
        elif layer["type"] == "attention":
            if "kv_from" in m and m["kv_from"] is not None:
                k_all, v_all = kv[m["kv_from"]]
            else:
                k_all, v_all = attention_keys_values(h, w, m, eps, pos)
                kv[i] = (k_all, v_all)
            y = attention_mixer(h, w, m, eps, pos, k_all, v_all, pos)
        else:
            raise ValueError(layer["type"])
        x = x + norm_zero_centred(y, tensors[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm_zero_centred(x, tensors[p + "norm2"], eps)
            x = x + norm_zero_centred(dense_ff(h, sub(tensors, p + "mlp.")), tensors[p + "norm2b"], eps)
        streams.append(x.clone())
    logits = norm_zero_centred(x, tensors["final.norm"], eps) @ tensors["head"].to(F64).T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:                                            # a model without a cap leaves the key out (or null / 0)
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
