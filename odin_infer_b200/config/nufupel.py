"""Configuration of the Nufupel decoder: blocks whose mixer and feed-forward read one norm's output side by
side; two kinds of windowed grouped-query attention with a sink logit and a sigmoid gate on the heads' outputs;
dense GeGLU feed-forwards or experts chosen per token beside a shared expert; layers that run with another
layer's weights and a cache of their own; scaled embeddings and capped logits.

config.json keys: "architecture", "vocab", "width", "norm" {"eps"}, "embedding" {"scale"} (absent: 1),
"logit_softcap" (absent, null or 0: none), and "layers": a list of

    {"type": "attention" | "attention_2", "mixer": {...}, "mlp": null | {...}, "weights_of": j (optional)}

mixer: heads, kv_heads (absent: heads), dim, vdim (absent: dim), scale (absent: 1 / sqrt(dim)), mask {size}
(absent: every earlier key), and for attention_2 rot {dims, base, scaling {factor, low, high, original} (optional)}.
mlp: {"kind": "dense", "ff"} or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"},
"shared": {"ff"} (optional)}.  A layer with weights_of = j has no tensors; it runs with layer j's.
"""
from __future__ import annotations

import dataclasses

from .base import KeyReader, ModelConfig

LAYER_TYPES = ("attention", "attention_2")


@dataclasses.dataclass(frozen=True)
class NufupelLayer:
    type: str
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 0.0
    window: int = 0                 # 0: every earlier key
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: tuple | None = None   # (factor, low, high, original)
    mlp_kind: str | None = None     # None, "dense", "moe"
    ff: int = 0                     # dense: inner size; moe: an expert's inner size
    experts: int = 0
    top: int = 0
    shared_ff: int = 0
    weights_of: int | None = None

    def mixer_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.type == "attention_2":
            rot = {"dims": self.rot_dims, "base": self.rot_base}
            if self.rot_scaling is not None:
                rot["scaling"] = dict(zip(("factor", "low", "high", "original"), self.rot_scaling))
            out["rot"] = rot
        return out

    def mlp_dict(self):
        if self.mlp_kind is None:
            return None
        if self.mlp_kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclasses.dataclass(frozen=True)
class NufupelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    layers: tuple[NufupelLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "NufupelConfig":
        r = KeyReader(raw, where)
        vocab, width = r.get("vocab", int), r.get("width", int)
        norm = KeyReader(r.get("norm", dict) or {}, where + " norm")
        eps = norm.get("eps", float)
        r.problems += norm.problems
        emb = raw.get("embedding")
        scale = KeyReader(emb if isinstance(emb, dict) else {}, where + " embedding").get("scale", float, 1.0)
        cap = r.get("logit_softcap", float, 0.0)
        r.require(vocab > 0 and width > 0, f"'vocab' and 'width' must be positive, got {vocab} and {width}")
        r.require(eps > 0, f"norm eps must be positive, got {eps}")
        r.require(cap >= 0, f"logit_softcap must not be negative, got {cap}")
        raw_layers = raw.get("layers")
        if not (isinstance(raw_layers, list) and raw_layers):
            r.problems.append("key 'layers' must be a list with a layer in it")
            raw_layers = []
        layers: list[NufupelLayer] = []
        for i, entry in enumerate(raw_layers):
            layers.append(cls._layer(r, i, entry if isinstance(entry, dict) else {}))
        for i, l in enumerate(layers):
            j, hops = l.weights_of, 0
            while j is not None and 0 <= j < len(layers) and layers[j].weights_of is not None and hops < len(layers):
                j, hops = layers[j].weights_of, hops + 1     # a layer that borrows from a borrower uses the lender's
            if l.weights_of is not None:
                ok = j is not None and 0 <= j < len(layers) and j != i and layers[j].weights_of is None
                r.require(ok, f"layer {i}: weights_of ({l.weights_of}) must lead to another layer that has tensors of its own")
                if ok:
                    r.require(dataclasses.replace(l, weights_of=None) == layers[j],
                              f"layer {i}: its entry differs from that of layer {j}, whose weights it uses")
                    layers[i] = dataclasses.replace(l, weights_of=j)
        r.finish()
        return cls(architecture=str(raw.get("architecture", "Nufupel")), vocab=vocab, width=width, norm_eps=eps,
                   embedding_scale=scale, logit_softcap=cap, layers=tuple(layers))

    @staticmethod
    def _layer(r: KeyReader, i: int, entry: dict) -> NufupelLayer:
        kind = entry.get("type")
        if kind not in LAYER_TYPES:
            r.problems.append(f"layer {i}: type must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
            return NufupelLayer(type="attention")
        m = KeyReader(entry.get("mixer") if isinstance(entry.get("mixer"), dict) else {}, f"layer {i} mixer")
        heads, dim = m.get("heads", int), m.get("dim", int)
        kv_heads, vdim = m.get("kv_heads", int, heads), m.get("vdim", int, dim)
        scale = m.get("scale", float, float(dim) ** -0.5 if dim > 0 else 0.0)
        mask = m.raw.get("mask")
        window = 0
        if mask is not None:
            window = KeyReader(mask if isinstance(mask, dict) else {}, f"layer {i} mixer mask").get("size", int, 0)
        m.require(heads > 0 and dim > 0 and vdim > 0, f"heads, dim and vdim must be positive, got {heads}, {dim}, {vdim}")
        m.require(kv_heads > 0 and heads % max(kv_heads, 1) == 0, f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        m.require(scale > 0, f"scale must be positive, got {scale}")
        m.require(window >= 0, f"mask size must not be negative, got {window}")
        layer = NufupelLayer(type=kind, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, window=window)
        if kind == "attention_2":
            rot_raw = m.raw.get("rot")
            if rot_raw is not None:
                rot = KeyReader(rot_raw if isinstance(rot_raw, dict) else {}, f"layer {i} mixer rot")
                rot_dims, base = rot.get("dims", int), rot.get("base", float)
                scaling = None
                if rot.raw.get("scaling") is not None:
                    sc = KeyReader(rot.raw["scaling"] if isinstance(rot.raw["scaling"], dict) else {}, f"layer {i} mixer rot scaling")
                    scaling = tuple(sc.get(k, float) for k in ("factor", "low", "high", "original"))
                    sc.require(scaling[0] > 0 and scaling[2] > scaling[1] and scaling[3] > 0,
                               f"needs factor > 0, high > low and original > 0, got {scaling}")
                    rot.problems += sc.problems
                rot.require(rot_dims >= 0 and rot_dims % 2 == 0 and rot_dims <= dim,
                            f"rot dims ({rot_dims}) must be even and at most dim ({dim})")
                rot.require(base > 0, f"rot base must be positive, got {base}")
                m.problems += rot.problems
                layer = dataclasses.replace(layer, rot_dims=rot_dims, rot_base=base, rot_scaling=scaling)
        r.problems += [f"layer {i} mixer: {p}" for p in m.problems]
        mlp = entry.get("mlp")
        if mlp is not None:
            k = KeyReader(mlp if isinstance(mlp, dict) else {}, f"layer {i} mlp")
            mk = k.raw.get("kind", "dense")
            if mk == "dense":
                ff = k.get("ff", int)
                k.require(ff > 0, f"ff must be positive, got {ff}")
                layer = dataclasses.replace(layer, mlp_kind="dense", ff=ff)
            elif mk == "moe":
                ex = KeyReader(k.get("expert", dict) or {}, "expert")
                ro = KeyReader(k.get("router", dict) or {}, "router")
                ff, n, top = ex.get("ff", int), ro.get("experts", int), ro.get("top", int)
                shared_ff = 0
                if k.raw.get("shared") is not None:
                    sh = KeyReader(k.raw["shared"] if isinstance(k.raw["shared"], dict) else {}, "shared")
                    shared_ff = sh.get("ff", int)
                    sh.require(shared_ff > 0, f"ff must be positive, got {shared_ff}")
                    k.problems += [f"shared: {p}" for p in sh.problems]
                k.problems += [f"expert: {p}" for p in ex.problems] + [f"router: {p}" for p in ro.problems]
                k.require(ff > 0 and n > 0 and 0 < top <= max(n, 1), f"needs ff > 0 and 0 < top <= experts, got ff {ff}, top {top}, experts {n}")
                layer = dataclasses.replace(layer, mlp_kind="moe", ff=ff, experts=n, top=top, shared_ff=shared_ff)
            else:
                k.problems.append(f"kind must be 'dense' or 'moe', got {mk!r}")
            r.problems += [f"layer {i} mlp: {p}" for p in k.problems]
        wo = entry.get("weights_of")
        if wo is not None:
            if isinstance(wo, int) and not isinstance(wo, bool):
                layer = dataclasses.replace(layer, weights_of=wo)
            else:
                r.problems.append(f"layer {i}: weights_of must be a layer's number, got {wo!r}")
        return layer

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            e = {"type": l.type, "mixer": l.mixer_dict(), "mlp": l.mlp_dict()}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out
