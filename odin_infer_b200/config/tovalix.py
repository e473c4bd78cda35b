"""Configuration of the Tovalix decoder: a stack of layers whose mixers differ from layer to layer
(chunked attention with shared keys and values, a token-shift recurrence, a gated linear recurrence),
each with an optional dense feed-forward and a per-layer input from the tokens.

config.json keys: "architecture" (the name), "vocab", "width", "norm" {"eps", "groups"},
"token_side" {"dim"} (absent or null: none), and "layers": a list of {"type", "mixer": {...}, "mlp":
{"kind": "dense", "ff"} or null}.  Mixer keys by type:

    attention  heads, kv_heads, dim, vdim, scale, softcap (absent: none), rot {dims, base},
               mask {size} (absent: all earlier keys), kv_from (absent: keys and values of its own)
    wkv        heads, dim  [decay_rank: written by random-weights mode; a folder's tensors rule]
    hgrn2      heads, dim, vdim
"""
from __future__ import annotations

import dataclasses

from .base import KeyReader, ModelConfig

LAYER_TYPES = ("attention", "wkv", "hgrn2")


@dataclasses.dataclass(frozen=True)
class TovalixLayer:
    type: str
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    kv_heads: int = 0
    scale: float = 0.0
    softcap: float = 0.0
    rot_dims: int = 0
    rot_base: float = 10000.0
    chunk: int = 0
    kv_from: int | None = None
    decay_rank: int = 0
    ff: int = 0                  # 0: no feed-forward

    def mixer_dict(self) -> dict:
        if self.type == "attention":
            out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                   "rot": {"dims": self.rot_dims, "base": self.rot_base}}
            if self.softcap:
                out["softcap"] = self.softcap
            if self.chunk:
                out["mask"] = {"size": self.chunk}
            if self.kv_from is not None:
                out["kv_from"] = self.kv_from
            return out
        if self.type == "wkv":
            out = {"heads": self.heads, "dim": self.dim}
            if self.decay_rank:
                out["decay_rank"] = self.decay_rank
            return out
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


@dataclasses.dataclass(frozen=True)
class TovalixConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    norm_groups: int = 1
    side_dim: int = 0
    layers: tuple[TovalixLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "TovalixConfig":
        r = KeyReader(raw, where)
        vocab, width = r.get("vocab", int), r.get("width", int)
        norm = KeyReader(r.get("norm", dict) or {}, where + " norm")
        eps, groups = norm.get("eps", float), norm.get("groups", int, 1)
        side = raw.get("token_side")
        side_dim = 0
        if side is not None:
            side_dim = KeyReader(side if isinstance(side, dict) else {}, where + " token_side").get("dim", int, 0)
        r.problems += norm.problems
        r.require(vocab > 0 and width > 0, f"'vocab' and 'width' must be positive, got {vocab} and {width}")
        r.require(eps > 0, f"norm eps must be positive, got {eps}")
        r.require(groups > 0 and (width <= 0 or width % groups == 0), f"norm groups ({groups}) must divide the width ({width})")
        r.require(side_dim >= 0, f"token_side dim must not be negative, got {side_dim}")
        layers = []
        raw_layers = raw.get("layers")
        if not (isinstance(raw_layers, list) and raw_layers):
            r.problems.append("key 'layers' must be a list with a layer in it")
            raw_layers = []
        for i, entry in enumerate(raw_layers):
            layers.append(cls._layer(r, i, entry if isinstance(entry, dict) else {}, layers))
        r.finish()
        return cls(architecture=str(raw.get("architecture", "Tovalix")), vocab=vocab, width=width, norm_eps=eps,
                   norm_groups=groups, side_dim=side_dim, layers=tuple(layers))

    @staticmethod
    def _layer(r: KeyReader, i: int, entry: dict, before: list) -> TovalixLayer:
        kind = entry.get("type")
        if kind not in LAYER_TYPES:
            r.problems.append(f"layer {i}: type must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
            return TovalixLayer(type="attention")
        m = KeyReader(entry.get("mixer") if isinstance(entry.get("mixer"), dict) else {}, f"layer {i} mixer")
        ff = 0
        mlp = entry.get("mlp")
        if mlp is not None:
            k = KeyReader(mlp if isinstance(mlp, dict) else {}, f"layer {i} mlp")
            ff = k.get("ff", int)
            k.require(k.raw.get("kind", "dense") == "dense", f"kind must be 'dense', got {k.raw.get('kind')!r}")
            k.require(ff > 0, f"ff must be positive, got {ff}")
            r.problems += [f"layer {i} mlp: {p}" for p in k.problems]
        heads, dim = m.get("heads", int), m.get("dim", int)
        m.require(heads > 0 and dim > 0, f"heads and dim must be positive, got {heads} and {dim}")
        layer = TovalixLayer(type=kind, heads=heads, dim=dim, ff=ff)
        if kind == "wkv":
            layer = dataclasses.replace(layer, decay_rank=m.get("decay_rank", int, 0))
        elif kind == "hgrn2":
            vdim = m.get("vdim", int)
            m.require(vdim > 0, f"vdim must be positive, got {vdim}")
            layer = dataclasses.replace(layer, vdim=vdim)
        else:
            kv_heads, vdim = m.get("kv_heads", int, heads), m.get("vdim", int, dim)
            scale, cap = m.get("scale", float), m.get("softcap", float, 0.0)
            rot = KeyReader(m.get("rot", dict) or {}, f"layer {i} mixer rot")
            rot_dims, base = rot.get("dims", int), rot.get("base", float)
            mask = m.raw.get("mask")
            chunk = 0
            if mask is not None:
                chunk = KeyReader(mask if isinstance(mask, dict) else {}, f"layer {i} mixer mask").get("size", int, 0)
            kv_from = m.raw.get("kv_from")
            m.problems += rot.problems
            m.require(kv_heads > 0 and heads % max(kv_heads, 1) == 0, f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
            m.require(vdim > 0, f"vdim must be positive, got {vdim}")
            m.require(scale > 0, f"scale must be positive, got {scale}")
            m.require(cap >= 0, f"softcap must not be negative, got {cap}")
            m.require(rot_dims >= 0 and rot_dims % 2 == 0 and rot_dims <= dim, f"rot dims ({rot_dims}) must be even and at most dim ({dim})")
            m.require(base > 0, f"rot base must be positive, got {base}")
            m.require(chunk >= 0, f"mask size must not be negative, got {chunk}")
            if kv_from is not None:
                ok = isinstance(kv_from, int) and not isinstance(kv_from, bool) and 0 <= kv_from < i
                src = before[kv_from] if ok else None
                ok = ok and src.type == "attention" and src.kv_from is None
                m.require(ok, f"kv_from ({kv_from!r}) must name an earlier attention layer with keys and values of its own")
                if ok:
                    m.require((src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base) == (kv_heads, dim, vdim, rot_dims, base),
                              f"kv_from: layer {kv_from} has other key/value heads or another rotation")
            layer = dataclasses.replace(layer, kv_heads=kv_heads, vdim=vdim, scale=scale, softcap=cap, rot_dims=rot_dims,
                                        rot_base=base, chunk=chunk, kv_from=kv_from if isinstance(kv_from, int) else None)
        r.problems += [f"layer {i} mixer: {p}" for p in m.problems]
        return layer

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
               "layers": [{"type": l.type, "mixer": l.mixer_dict(), "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None}
                          for l in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out
