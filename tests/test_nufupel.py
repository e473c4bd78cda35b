"""The Nufupel configuration, its model description, and the plain implementation's own mechanisms (no GPU)."""
import copy
import math

import pytest
import torch

from odin_infer_b200.config import ConfigError, NufupelConfig, config_from_dict, lookup_architecture
from odin_infer_b200.engine.model import DecoderModel
from tests.plain import nufupel_plain as P

F64 = torch.float64
_L1 = {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 40, "scale": 0.2, "mask": {"size": 50}},
       "mlp": {"kind": "moe", "expert": {"ff": 48}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 96}}}
RAW = {"architecture": "Nufupel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
       "logit_softcap": 2.5,
       "layers": [{"type": "attention_2",
                   "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.18, "mask": {"size": 37},
                             "rot": {"dims": 16, "base": 5000.0, "scaling": {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 96}}},
                   "mlp": {"kind": "dense", "ff": 136}},
                  _L1, dict(_L1, weights_of=1),
                  {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 1}},
                   "mlp": None},
                  dict(_L1, weights_of=1)]}


def test_configuration_reads_and_writes_the_same_keys():
    cfg = config_from_dict(RAW)
    assert isinstance(cfg, NufupelConfig) and cfg.to_dict() == RAW
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[0].rot_scaling == (6.0, 1.0, 3.0, 96.0) and cfg.layers[2].weights_of == 1 and cfg.layers[3].mlp_kind is None


def test_absent_keys_mean_absent_mechanisms():
    raw = {"architecture": "Nufupel", "vocab": 50, "width": 40, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention_2", "mixer": {"heads": 2, "dim": 16}, "mlp": None}]}
    cfg = config_from_dict(raw)
    l = cfg.layers[0]
    assert (l.kv_heads, l.vdim, l.window, l.rot_dims, l.rot_scaling) == (2, 16, 0, 0, None)
    assert l.scale == pytest.approx(0.25) and cfg.embedding_scale == 1.0 and cfg.logit_softcap == 0.0
    spec = lookup_architecture("Nufupel").build_spec(cfg)
    assert spec.position_encodings == {} and spec.head.args["softcap"] == 0.0


def test_every_fault_of_a_configuration_in_one_error():
    bad = copy.deepcopy(RAW)
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    bad["layers"][0]["mixer"]["rot"]["dims"] = 33
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    bad["layers"][2]["weights_of"] = 0
    bad["layers"][3]["type"] = "attention_3"
    bad["norm"] = {}
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    for part in ("kv_heads", "rot dims", "top", "whose weights it uses", "attention_3", "eps"):
        assert part in text, part


def test_layers_that_share_weights_are_one_block_with_an_entry_each():
    cfg = config_from_dict(RAW)
    spec = lookup_architecture("Nufupel").build_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 1, 2, 1] and len(spec.layers) == 3
    names = [p.name for p in DecoderModel(spec).params()]
    assert "l1.mlp.e5.down" in names and "l1.mlp.router.b" in names and "l0.mix.q.norm" in names and "l3.mix.sink" in names
    assert not any(n.startswith(("l2.", "l4.")) for n in names)
    assert "l1.mix.q.norm" not in names and "l3.mlp.gate" not in names
    shapes = {p.name: p.shape for p in DecoderModel(spec).params()}
    assert shapes["l0.mix.g"] == (4, 96) and shapes["l1.mix.g"] == (6 * 40, 96) and shapes["l1.mix.o"] == (96, 240)
    assert shapes["l1.mlp.shared.down"] == (96, 96) and shapes["l1.mix.sink"] == (6,)


def test_the_shared_expert_rides_as_experts_when_its_size_allows():
    from odin_infer_b200.parts.base import PartSpec, build_part
    names = {"router": "r", "router_bias": "rb", "gate": "e{e}.g", "up": "e{e}.u", "down": "e{e}.d", "shared_gate": "sg",
             "shared_up": "su", "shared_down": "sd"}
    for shared, as_experts in ((0, 0), (48, 1), (96, 2), (56, 0)):
        part = build_part("feed_forward", PartSpec("routed_experts", dict(width=32, inner=48, n_experts=3, top=2, names=names,
                                                                          shared_inner=shared)))
        assert part.shared_as_experts == as_experts
        tensors = {p.name: torch.randn(p.shape) for p in part.params()}
        part.bind(tensors, None)
        assert tuple(part.w_gate_up.shape) == (3 + as_experts, 96, 32) and tuple(part.w_down.shape) == (3 + as_experts, 32, 48)
        assert (part.ws_gate_up is None) == (shared in (0, 48, 96))
    # cut into experts, the shared expert is the same sum over its inner columns
    torch.manual_seed(0)
    h = torch.randn(4, 32, dtype=F64)
    w = {"gate": torch.randn(96, 32, dtype=F64), "up": torch.randn(96, 32, dtype=F64), "down": torch.randn(32, 96, dtype=F64)}
    whole = P.gated_mlp(h, w, "", P.silu)
    halves = sum(P.gated_mlp(h, {"gate": w["gate"][a:a + 48], "up": w["up"][a:a + 48], "down": w["down"][:, a:a + 48]}, "", P.silu)
                 for a in (0, 48))
    assert torch.allclose(whole, halves, atol=1e-12)


# ---- the plain implementation's own mechanisms ----------------------------------------------------
def test_plain_window_by_perturbation_and_sink_by_its_limits():
    torch.manual_seed(0)
    n, H, G, d = 12, 4, 2, 8
    q, k, v = (torch.randn(n, h, d, dtype=F64) for h in (H, G, G))
    sink = torch.randn(H, dtype=F64)
    base = P.window_sink_attention(q, k, v, 0.3, 5, sink)
    for j in range(n):
        k2, v2 = k.clone(), v.clone()
        k2[j] += 1.0
        v2[j] -= 2.0
        moved = (P.window_sink_attention(q, k2, v2, 0.3, 5, sink) - base).abs().amax(dim=(1, 2)) > 1e-9
        assert moved.tolist() == [0 <= i - j < 5 for i in range(n)], j
    # a sink far below every score changes nothing; a sink far above takes the whole denominator
    gone = P.window_sink_attention(q, k, v, 0.3, 5, torch.full((H,), -1e4, dtype=F64))
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(H // G, dim=1)) * 0.3
    mask = torch.tensor([[0 <= i - j < 5 for j in range(n)] for i in range(n)])
    ref = torch.einsum("hij,jhd->ihd", torch.softmax(s.masked_fill(~mask, -math.inf), dim=-1), v.repeat_interleave(H // G, dim=1))
    assert torch.allclose(gone, ref, atol=1e-12)
    assert P.window_sink_attention(q, k, v, 0.3, 5, torch.full((H,), 1e3, dtype=F64)).abs().max() < 1e-100
    # one key and a sink of the same logit: half of the value
    one = P.window_sink_attention(q[:1], k[:1], v[:1], 0.3, 5, (q[0] * k[0].repeat_interleave(H // G, dim=0)).sum(-1) * 0.3)
    assert torch.allclose(one[0], 0.5 * v[0].repeat_interleave(H // G, dim=0), atol=1e-12)


def test_plain_rotation_and_stretched_frequencies():
    f = P.stretched_frequencies(40, 70000.0, {"factor": 5.0, "low": 2.0, "high": 6.0, "original": 3000})
    plain = P.stretched_frequencies(40, 70000.0, None)
    assert torch.allclose(plain, torch.tensor([70000.0 ** (-2 * i / 40) for i in range(20)], dtype=F64))
    wavelength = 2 * math.pi / plain
    assert torch.equal(f[wavelength < 500], plain[wavelength < 500]) and torch.allclose(f[wavelength > 1500], plain[wavelength > 1500] / 5)
    assert (wavelength < 500).any() and (wavelength > 1500).any()
    mid = (wavelength >= 500) & (wavelength <= 1500)
    assert mid.any() and ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 5)).all()
    # a rotation keeps lengths, leaves the tail alone, and scores depend on the distance of the positions only
    torch.manual_seed(1)
    t = torch.randn(6, 2, 12, dtype=F64)
    fr = P.stretched_frequencies(8, 100.0, None)
    r = P.rotate_half(t, torch.arange(6), fr, 8)
    assert torch.allclose(r[..., 8:], t[..., 8:]) and torch.allclose(r[..., :8].norm(dim=-1), t[..., :8].norm(dim=-1))
    a, b = torch.randn(1, 1, 8, dtype=F64), torch.randn(1, 1, 8, dtype=F64)
    dots = [float((P.rotate_half(a, torch.tensor([p]), fr, 8) * P.rotate_half(b, torch.tensor([p + 3]), fr, 8)).sum()) for p in (0, 5, 40)]
    assert max(dots) - min(dots) < 1e-12
    assert torch.allclose(r[0], t[0])    # position 0 is not rotated


def test_plain_router_norm_and_cap():
    torch.manual_seed(2)
    h, wr, b = torch.randn(7, 10, dtype=F64), torch.randn(5, 10, dtype=F64), torch.randn(5, dtype=F64)
    idx, wt = P.route(h, wr, b, 3)
    z = h @ wr.T + b
    assert torch.allclose(wt.sum(-1), torch.ones(7, dtype=F64))
    for t in range(7):
        order = sorted(range(5), key=lambda e: -float(z[t, e]))[:3]
        assert idx[t].tolist() == order
        assert torch.allclose(wt[t], torch.softmax(z[t, order], dim=0))
    x = torch.randn(3, 16, dtype=F64) * 4
    assert torch.allclose(P.one_plus_norm(x, torch.zeros(16, dtype=F64), 0.0).pow(2).mean(-1), torch.ones(3, dtype=F64))
    assert torch.allclose(P.one_plus_norm(x, torch.full((16,), 0.5, dtype=F64), 1e-6), 1.5 * P.one_plus_norm(x, torch.zeros(16, dtype=F64), 1e-6))
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=F64))) - 0.8411919906082768) < 1e-12
