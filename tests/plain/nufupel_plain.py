"""Plain, slow implementation of the Nufupel decoder: the oracle of its tests.

Whole sequences, no cache, one function per mechanism, float64 on the CPU.  It shares no code
with the product package (only the oracles' reader of a model folder, which is test code too).

The design in this file's notation (n tokens, width d, x the residual stream):

    x = E[token] * s_embed
    for every entry of `layers`:   h = onorm(x, w1);  x += mixer(h) + ffn(h)     (one norm, both read h)
    logits = cap * tanh(H onorm(x, w_final) / cap)

onorm(x, w) = x / sqrt(mean(x^2) + eps) * (1 + w).  An entry with `weights_of: j` runs with layer j's tensors.

Mixers: `attention` (no rotation, gate per element) and `attention_2` (q/k RMSNorm with a plain weight shared by the
heads, partial rotation in the rotate-half layout with stretched frequencies, gate per head); both grouped-query,
with a sliding window, a learned sink logit per head in the softmax's denominator and a sigmoid gate computed from h.
Feed-forwards: dense GeGLU (tanh form), or experts with SiLU chosen by a biased linear router (softmax over the chosen
logits) plus a shared expert.
"""
from __future__ import annotations

import math

import torch

from .qwen3_plain import read_model_folder  # noqa: F401  (re-exported: the folder reader of the oracles)

F64 = torch.float64


def one_plus_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (1.0 + w)


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def stretched_frequencies(dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` {factor, low, high, original}: wavelengths shorter than
    original/high keep f, longer than original/low get f/factor, between them a blend linear in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_half(t: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, dims: int) -> torch.Tensor:
    """t: [n, heads, dim]; the first `dims` elements of every head are rotated, element i with i + dims/2."""
    if dims == 0:
        return t
    ang = positions.to(F64)[:, None] * freqs[None, :]           # [n, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v, rest = t[..., : dims // 2], t[..., dims // 2: dims], t[..., dims:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


def window_sink_attention(q, k, v, scale: float, window: int, sink: torch.Tensor) -> torch.Tensor:
    """q: [n, H, dk], k: [n, G, dk], v: [n, G, dv]; query i sees keys j with 0 <= i - j < window; the softmax's
    denominator also holds exp(sink[h]) (no key, no value, not scaled).  Loops, one query at a time."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            lo = max(0, i - window + 1)
            s = (k[lo: i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - m)
            denom = e.sum() + math.exp(float(sink[h]) - m)
            out[i, h] = (e / denom) @ v[lo: i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, w: dict, p: str, mx: dict, eps: float, kind: str) -> torch.Tensor:
    n = h.shape[0]
    H, dk = mx["heads"], mx["dim"]
    G, dv = mx.get("kv_heads", H), mx.get("vdim", dk)       # absent: as many key heads as query heads, values as wide as keys
    window = int(mx["mask"]["size"]) if mx.get("mask") else n   # absent: every earlier key
    scale = float(mx.get("scale", dk ** -0.5))
    q = (h @ w[p + "q"].T).reshape(n, H, dk)
    k = (h @ w[p + "k"].T).reshape(n, G, dk)
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    if kind == "attention_2":
        q = plain_norm(q, w[p + "q.norm"], eps)
        k = plain_norm(k, w[p + "k.norm"], eps)
        rot = mx.get("rot")
        if rot is not None:
            freqs = stretched_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
            pos = torch.arange(n)
            q = rotate_half(q, pos, freqs, rot["dims"])
            k = rotate_half(k, pos, freqs, rot["dims"])
    o = window_sink_attention(q, k, v, scale, window, w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].T)
    if kind == "attention_2":
        o = o * gate[:, :, None]                # one number per head
    else:
        o = o * gate.reshape(n, H, dv)          # one number per element
    return o.reshape(n, H * dv) @ w[p + "o"].T


def gated_mlp(h, w, p: str, act) -> torch.Tensor:
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w_router, bias, top: int):
    """Chosen experts [n, top] and their weights (softmax over the chosen logits only)."""
    z = h @ w_router.T + bias
    vals, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(vals, dim=-1)


def expert_mlp(h, w, p: str, mlp: dict) -> torch.Tensor:
    idx, wt = route(h, w[p + "router"], w[p + "router.b"], int(mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * gated_mlp(h[t: t + 1], w, f"{p}e{e}.", silu)[0]
    if mlp.get("shared") is not None:
        out = out + gated_mlp(h, w, p + "shared.", silu)
    return out


def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [n, vocab] of one whole sequence (float64); with return_layers also the residual stream after
    every entry of `layers`, [entries, n, width]."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    stream = []
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        if src is None:
            src = i
        p = f"l{src}."
        h = one_plus_norm(x, w[p + "norm1"], eps)
        upd = attention_mixer(h, w, p + "mix.", layer["mixer"], eps, layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                upd = upd + gated_mlp(h, w, p + "mlp.", gelu_tanh)
            else:
                upd = upd + expert_mlp(h, w, p + "mlp.", mlp)
        x = x + upd
        stream.append(x.clone())
    logits = one_plus_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = float(config.get("logit_softcap") or 0.0)
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(stream)) if return_layers else logits
