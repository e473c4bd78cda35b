"""Plain, slow implementation of the Tovalix decoder: the oracle of its tests.

Whole sequences, no cache, one function per mechanism, float64 on the CPU, recurrences as
loops over the tokens.  It shares no code with the product package: its own reader of the
model folder (through the other oracle's container reader, which is test code too) and its
own arithmetic.

The design in this file's notation (n tokens, width d, x the residual stream):

    x = gnorm(E[token], w_embed)
    for every layer i:   x += mixer_i(gnorm(x, w1));  x += ffn_i(gnorm(x, w2)) if it has one;
                         x += unit(P g) * w_side  with  g = gelu_tanh(G x) * T[token, i*s:(i+1)*s]
    logits = H gnorm(x, w_final)

gnorm(x, w): x is cut into `groups` equal consecutive parts, each part divided by
sqrt(mean(part^2) + eps), the whole times w.  unit(y) = y / sqrt(mean(y^2) + eps).
"""
from __future__ import annotations

import math

import torch

from .qwen3_plain import read_model_folder  # noqa: F401  (re-exported: the folder reader of the oracles)

F64 = torch.float64


# --------------------------------------------------------------------------
# small functions
# --------------------------------------------------------------------------
def unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    """y / sqrt(mean(y^2) + eps) over the last axis."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    n, d = x.shape
    parts = x.reshape(n, groups, d // groups)
    return unit(parts, eps).reshape(n, d) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    ap = softplus(pq[0])
    an = 0.5 + softplus(pq[1])
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


# --------------------------------------------------------------------------
# feed-forward and the per-layer token input
# --------------------------------------------------------------------------
def dense_ffn(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return xielu(h @ w[p + "up"].t(), w[p + "act"]) @ w[p + "down"].t()


def token_side(x: torch.Tensor, tokens, layer: int, side_dim: int, w: dict, p: str, eps: float) -> torch.Tensor:
    """What the layer adds to x from the tokens themselves."""
    e = w["side.embed"][torch.as_tensor(tokens, dtype=torch.long), layer * side_dim:(layer + 1) * side_dim]
    g = gelu_tanh(x @ w[p + "gate"].t()) * e
    return unit(g @ w[p + "proj"].t(), eps) * w[p + "norm"]


# --------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------
def rotate_half(v: torch.Tensor, positions: torch.Tensor, rot_dims: int, base: float) -> torch.Tensor:
    """v: [n, heads, dim]; the first rot_dims of every head are turned, element i with element
    i + rot_dims/2 by the angle p * base^(-2i/rot_dims); the rest is kept."""
    half = rot_dims // 2
    if half == 0:
        return v
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / rot_dims)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:rot_dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., rot_dims:]], dim=-1)


def attention_keys_values(h: torch.Tensor, m: dict, w: dict, p: str, eps: float):
    """What an attention layer keeps per token: keys after rotation and unit norm, and values."""
    n = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    pos = torch.arange(n)
    k = (h @ w[p + "k"].t() + w[p + "k.b"]).reshape(n, G, dk)
    k = unit(rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"]), eps)
    v = (h @ w[p + "v"].t() + w[p + "v.b"]).reshape(n, G, dv)
    return k, v


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap, chunk, first_pos: int = 0,
           window=None) -> torch.Tensor:
    """q: [n, H, dk], the queries of positions first_pos .. first_pos + n - 1; k: [m, G, dk] and v: [m, G, dv],
    the keys and values of positions 0 .. m - 1.  Position p sees the keys j <= p of its own chunk
    (j // chunk == p // chunk), and with a window only those with j > p - window; scores q.k * scale,
    then cap * tanh(score / cap), then a softmax."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        for t in range(n):
            pos = first_pos + t
            lo = (pos // chunk) * chunk if chunk else 0
            if window:
                lo = max(lo, pos - window + 1)
            s = (k[lo:pos + 1, g] @ q[t, head]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            out[t, head] = torch.softmax(s, dim=0) @ v[lo:pos + 1, g]
    return out


def attention_mixer(h: torch.Tensor, m: dict, w: dict, p: str, eps: float, kv) -> torch.Tensor:
    """kv: the (keys, values) this layer looks at (its own, or another layer's)."""
    n = h.shape[0]
    H, dk = m["heads"], m["dim"]
    q = (h @ w[p + "q"].t() + w[p + "q.b"]).reshape(n, H, dk)
    q = unit(rotate_half(q, torch.arange(n), m["rot"]["dims"], m["rot"]["base"]), eps)
    out = attend(q, kv[0], kv[1], m["scale"], m.get("softcap"), (m.get("mask") or {}).get("size"))
    return out.reshape(n, -1) @ w[p + "o"].t() + w[p + "o.b"]


def wkv_mixer(h: torch.Tensor, m: dict, w: dict, p: str, eps: float) -> torch.Tensor:
    """Token-shift mixes, a decay per head and key channel from a two-step projection, the
    matrix-valued state S (key channel x value channel) with a bonus for the current token."""
    n, d = h.shape
    H, D = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, d, dtype=F64), h[:-1]], dim=0)
    mix = {s: h + (before - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].t()).reshape(n, H, D)
    k = (mix["k"] @ w[p + "k"].t()).reshape(n, H, D)
    v = (mix["v"] @ w[p + "v"].t()).reshape(n, H, D)
    gate = silu(mix["g"] @ w[p + "g"].t())
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].t()) @ w[p + "w2"].t() + w[p + "w0"])).reshape(n, H, D)
    u = w[p + "u"]
    out = torch.zeros(n, H, D, dtype=F64)
    S = torch.zeros(H, D, D, dtype=F64)
    for t in range(n):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    o = unit(out, eps).reshape(n, H * D) * w[p + "norm"] * gate
    return o @ w[p + "o"].t()


def hgrn2_mixer(h: torch.Tensor, m: dict, w: dict, p: str, eps: float) -> torch.Tensor:
    """A forget gate f in (lower, 1) per head and channel; 1 - f stands where a key would."""
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].t()).reshape(n, H, D)
    v = (h @ w[p + "v"].t()).reshape(n, H, V)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[p + "f"].t() + w[p + "f.b"])).reshape(n, H, D)
    out = torch.zeros(n, H, V, dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    for t in range(n):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = (unit(out, eps) * w[p + "norm"]).reshape(n, H * V)
    return o @ w[p + "o"].t()


# --------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------
def forward_whole(cfg: dict, w: dict, tokens, layers_out: list | None = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence from its first token; `layers_out` collects the residual
    stream after every layer."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    side = (cfg.get("token_side") or {}).get("dim", 0)
    x = group_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F64), w["embed.norm"], groups, eps)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = group_norm(x, w[p + "norm1"], groups, eps)
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, m, w, p + "mix.", eps)
            x = x + attention_mixer(h, m, w, p + "mix.", eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        elif layer["type"] == "wkv":
            x = x + wkv_mixer(h, m, w, p + "mix.", eps)
        elif layer["type"] == "hgrn2":
            x = x + hgrn2_mixer(h, m, w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_ffn(group_norm(x, w[p + "norm2"], groups, eps), w, p + "mlp.")
        if side:
            x = x + token_side(x, tokens, i, side, w, p + "side.", eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return group_norm(x, w["final.norm"], groups, eps) @ w["head"].t()
