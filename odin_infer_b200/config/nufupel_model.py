"""The Nufupel decoder written out in parts.

x = E[token] * scale.  Every layer is a parallel block: h = norm(x), x += mixer(h) + feed_forward(h), with an
RMSNorm whose stored weight lies around zero (factor 1 + w).  Mixers: grouped-query attention over a sliding
window with a sink logit per head and a sigmoid gate computed from h on the heads' outputs; kind `attention`
has no rotation and gates every element, kind `attention_2` norms q and k per head (plain weight, before the
rotation), rotates the first rot.dims elements of a head with stretched frequencies, and gates per head.
Feed-forwards: a dense GeGLU (tanh form), or SiLU experts chosen by a biased router beside a shared expert.
A layer may run with another layer's tensors (one block, several schedule entries, a cache line each).  Then
the norm, the head, and a cap on the logits.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.q|k|v|o|g|sink|q.norm|k.norm`, `l<i>.mlp.gate|up|down`,
`l<i>.mlp.router|router.b`, `l<i>.mlp.e<n>.gate|up|down`, `l<i>.mlp.shared.gate|up|down`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..parts.base import PartSpec
from ..parts.spec import ModelSpec, ScheduleEntry
from .nufupel import NufupelConfig
from .registry import register_architecture


def build_nufupel_spec(cfg: NufupelConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight=weight, one_plus=True))

    blocks, block_of, schedule, encodings = [], {}, [], {}
    for i, l in enumerate(cfg.layers):
        if l.weights_of is not None:
            continue
        p = f"l{i}."
        m = p + "mix."
        pe, qk_norm = None, False
        names = {"q": m + "q", "k": m + "k", "v": m + "v", "o": m + "o"}
        if l.type == "attention_2":
            qk_norm = True
            names.update({"q_norm": m + "q.norm", "k_norm": m + "k.norm"})
            if l.rot_dims > 0:
                pe = f"rope_{l.rot_dims}_{l.rot_base!r}_{l.rot_scaling!r}"
                stretch = dict(zip(("factor", "low", "high", "original"), l.rot_scaling)) if l.rot_scaling else None
                encodings[pe] = PartSpec("rope", dict(rotary_dim=l.rot_dims, theta=l.rot_base, stretch=stretch, precise=True))
        mixer = PartSpec("gqa_attention", dict(
            width=cfg.width, n_q_heads=l.heads, n_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim,
            position_encoding=pe, qk_norm=qk_norm, eps=cfg.norm_eps, window=l.window, scale=l.scale, names=names,
            sink=m + "sink", gate=m + "g", gate_per_head=l.type == "attention_2"))
        ffn = None
        f = p + "mlp."
        if l.mlp_kind == "dense":
            ffn = PartSpec("swiglu", dict(width=cfg.width, inner=l.ff, activation="gelu_tanh",
                                          names={"gate": f + "gate", "up": f + "up", "down": f + "down"}))
        elif l.mlp_kind == "moe":
            ffn = PartSpec("routed_experts", dict(
                width=cfg.width, inner=l.ff, n_experts=l.experts, top=l.top, activation="silu", shared_inner=l.shared_ff,
                names={"router": f + "router", "router_bias": f + "router.b", "gate": f + "e{e}.gate", "up": f + "e{e}.up",
                       "down": f + "e{e}.down", "shared_gate": f + "shared.gate", "shared_up": f + "shared.up",
                       "shared_down": f + "shared.down"}))
        block_of[i] = len(blocks)
        blocks.append(PartSpec("parallel", dict(mixer=mixer, feed_forward=ffn, norm=norm(p + "norm1"))))
    for i, l in enumerate(cfg.layers):
        schedule.append(ScheduleEntry(block_of[i if l.weights_of is None else l.weights_of]))
    return ModelSpec(
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=cfg.width, weight="embed", scale=cfg.embedding_scale)),
        position_encodings=encodings,
        layers=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=cfg.width, weight="head", softcap=cfg.logit_softcap)),
    )


register_architecture("Nufupel", NufupelConfig, build_nufupel_spec)
