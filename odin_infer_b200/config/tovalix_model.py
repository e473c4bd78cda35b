"""The Tovalix decoder written out in parts.

The embedded tokens pass through the model's norm (an RMSNorm in groups) and become the residual stream.
Every layer is a pre-norm block: one of three mixers (grouped-query attention over a chunked mask with
biases, partial rotation, unit-norm q and k and capped scores, possibly on another layer's keys and values;
a token-shift recurrence with a data-dependent decay; a gated linear recurrence), an optional dense
feed-forward with the xIELU activation, and an input from the tokens themselves.  Then the norm and the head.
Tensor names: `embed`, `embed.norm`, `side.embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.up|down|act`,
`l<i>.side.gate|proj|norm`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..parts.base import PartSpec
from ..parts.spec import ModelSpec, ScheduleEntry
from .registry import register_architecture
from .tovalix import TovalixConfig


def _rope_name(dims: int, base: float) -> str:
    return f"rope_{dims}_{base!r}"


def build_tovalix_spec(cfg: TovalixConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight=weight, groups=cfg.norm_groups))

    layers, schedule, encodings = [], [], {}
    table_width = cfg.side_dim * len(cfg.layers)
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        if l.type == "attention":
            pe = None
            if l.rot_dims > 0:
                pe = _rope_name(l.rot_dims, l.rot_base)
                encodings[pe] = PartSpec("rope", dict(rotary_dim=l.rot_dims, theta=l.rot_base))
            mixer = PartSpec("gqa_attention", dict(
                width=cfg.width, n_q_heads=l.heads, n_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim,
                position_encoding=pe, qk_norm="unit_after", eps=cfg.norm_eps, chunk=l.chunk, scale=l.scale,
                softcap=l.softcap, kv_shared=l.kv_from is not None,
                names={"q": m + "q", "k": m + "k", "v": m + "v", "o": m + "o"},
                biases={"q": m + "q.b", "k": m + "k.b", "v": m + "v.b", "o": m + "o.b"}))
        elif l.type == "wkv":
            names = {s: m + s for s in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
            names.update({"mu_" + s: m + "mu." + s for s in ("r", "k", "v", "g", "w")})
            mixer = PartSpec("wkv_token_shift", dict(width=cfg.width, n_heads=l.heads, head_dim=l.dim, eps=cfg.norm_eps,
                                                     decay_rank=l.decay_rank, names=names))
        else:
            mixer = PartSpec("gated_linear_recurrence", dict(
                width=cfg.width, n_heads=l.heads, head_dim=l.dim, v_head_dim=l.vdim, eps=cfg.norm_eps,
                names={"q": m + "q", "f": m + "f", "f_bias": m + "f.b", "lower": m + "lower", "v": m + "v",
                       "norm": m + "norm", "o": m + "o"}))
        ffn = norm2 = None
        if l.ff:
            ffn = PartSpec("activated", dict(width=cfg.width, inner=l.ff, activation="xielu",
                                             names={"up": p + "mlp.up", "down": p + "mlp.down", "act": p + "mlp.act"}))
            norm2 = norm(p + "norm2")
        extras = ()
        if cfg.side_dim:
            extras = (PartSpec("token_side_input", dict(
                width=cfg.width, dim=cfg.side_dim, vocab_size=cfg.vocab, table_width=table_width,
                first_column=i * cfg.side_dim, eps=cfg.norm_eps,
                names={"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj", "norm": p + "side.norm"})),)
        layers.append(PartSpec("prenorm", dict(mixer=mixer, feed_forward=ffn, norm_mixer=norm(p + "norm1"),
                                               norm_feed_forward=norm2, extras=extras)))
        schedule.append(ScheduleEntry(i, reads_cache_of=l.kv_from))
    return ModelSpec(
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=cfg.width, weight="embed", norm=norm("embed.norm"))),
        position_encodings=encodings,
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=cfg.width, weight="head")),
        # a layer without a feed-forward has no use for a second norm; a folder that stores one is still read
        tolerated_tensors=tuple(f"l{i}.norm2" for i, l in enumerate(cfg.layers) if not l.ff),
    )


register_architecture("Tovalix", TovalixConfig, build_tovalix_spec)
