"""Tovalix without a GPU: its configuration, the parts and tensors its builder names, the cache's chunk groups,
and the plain implementation's recurrences against a second way of writing them."""
import dataclasses

import numpy as np
import pytest
import torch

from tests.plain import tovalix_plain as P

F64 = torch.float64


def raw_config():
    att = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.3, "softcap": 9.0, "rot": {"dims": 8, "base": 1e3},
           "mask": {"size": 21}}
    return {"architecture": "Tovalix", "vocab": 50, "width": 48, "norm": {"eps": 1e-5, "groups": 2}, "token_side": {"dim": 6},
            "layers": [{"type": "attention", "mixer": att, "mlp": {"kind": "dense", "ff": 40}},
                       {"type": "wkv", "mixer": {"heads": 2, "dim": 8}, "mlp": None},
                       {"type": "hgrn2", "mixer": {"heads": 3, "dim": 8, "vdim": 4}, "mlp": {"kind": "dense", "ff": 24}},
                       {"type": "attention", "mixer": dict(att, kv_from=0, mask={"size": 33}), "mlp": {"kind": "dense", "ff": 16}}]}


def test_config_reads_and_writes_back():
    from odin_infer_b200.config import TovalixConfig, config_from_dict
    cfg = config_from_dict(raw_config())
    assert isinstance(cfg, TovalixConfig) and cfg.layers[3].kv_from == 0 and cfg.layers[1].ff == 0
    assert cfg.layers[0].chunk == 21 and cfg.layers[0].rot_dims == 8 and cfg.norm_groups == 2 and cfg.side_dim == 6
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"][1]["mlp"] is None


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_heads=4), "other key/value heads"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot dims"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda r: r["norm"].update(groups=5), "groups"),
    (lambda r: r["layers"][2].update(type="mamba"), "type must be"),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), "kind must be"),
    (lambda r: r.pop("vocab"), "vocab"),
])
def test_config_faults_are_named(change, word):
    from odin_infer_b200.config import ConfigError, config_from_dict
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_builder_names_the_tensors():
    from odin_infer_b200.config import config_from_dict, lookup_architecture
    from odin_infer_b200.engine.model import DecoderModel
    cfg = config_from_dict(raw_config())
    model = DecoderModel(lookup_architecture("Tovalix").build_spec(cfg))
    params = {p.name: p for p in model.params()}
    assert params["side.embed"].shape == (50, 24) and params["l0.mix.v"].shape == (16, 48) and params["l0.mix.o"].shape == (48, 32)
    assert "l3.mix.k" not in params and "l3.mix.q.b" in params and "l1.norm2" in params and params["l1.norm2"].optional
    assert "l1.mlp.up" not in params and params["l1.mix.w1"].shape == (-1, 48) and params["l1.mix.w1"].matches((7, 48))
    assert params["l2.mix.norm"].shape == (4,) and params["l1.mix.norm"].shape == (16,) and params["l1.mix.u"].shape == (2, 8)
    assert [e.reads_cache_of for e in model.spec.schedule] == [None, None, None, 0]
    assert model.graph_safe


def test_cache_keeps_what_every_reader_of_a_line_sees():
    from odin_infer_b200.cache import CacheManager, KVRequest
    from odin_infer_b200.config import config_from_dict, lookup_architecture
    from odin_infer_b200.engine.model import DecoderModel
    raw = raw_config()
    model = DecoderModel(lookup_architecture("Tovalix").build_spec(config_from_dict(raw)))
    cache = CacheManager(64 * 20, 64 * 10)
    model.register_cache(cache)
    (group,) = cache.groups.values()
    assert group.request.chunk == 0 and group.request.value_dim == 8      # chunks 21 and 33 on one line: all is kept
    raw["layers"][3]["mixer"]["mask"] = {"size": 21}
    model = DecoderModel(lookup_architecture("Tovalix").build_spec(config_from_dict(raw)))
    cache = CacheManager(64 * 20, 64 * 10)
    model.register_cache(cache)
    (group,) = cache.groups.values()
    assert group.request.chunk == 21
    # pages wholly before the next query's chunk go back, one by one as the sequence grows
    req = KVRequest(2, 16, chunk=100)
    assert [req.first_visible(p) for p in (0, 99, 100, 199, 200)] == [0, 0, 100, 100, 200]
    big = CacheManager(64 * 20, 64 * 10)
    big.add_entry(req, 0)
    slot = big.take_slot()
    held = []
    for _ in range(260):
        big.extend(slot, 1)
        big.after_step(slot)
        held.append(big.groups[req.key].pool.n_held)
        big.check()
    assert held[63] == 1 and held[64] == 2 and held[98] == 2      # 64 tokens: one page; 65 and 99 tokens: pages 0 and 1
    assert held[99] == 1                                          # the next query is 100: page 0 is gone
    assert held[199] == 1 and held[255] == 1 and held[256] == 2   # 200 -> page 3 alone; position 256 opens page 4
    big.give_back_slot(slot)
    assert big.groups[req.key].pool.n_held == 0


def test_plain_recurrences_against_their_sums():
    """The two recurrences of the plain implementation, unrolled: an output is a sum over the earlier tokens of
    products of decays (no state at all)."""
    torch.manual_seed(0)
    n, d, H, D, V = 7, 12, 2, 3, 4
    h = torch.randn(n, d, dtype=F64)
    w = {"m.q": torch.randn(H * D, d, dtype=F64), "m.v": torch.randn(H * V, d, dtype=F64), "m.f": torch.randn(H * D, d, dtype=F64),
         "m.f.b": torch.randn(H * D, dtype=F64), "m.lower": torch.rand(H * D, dtype=F64), "m.norm": torch.ones(V, dtype=F64),
         "m.o": torch.eye(H * V, dtype=F64)}
    got = P.hgrn2_mixer(h, {"heads": H, "dim": D, "vdim": V}, w, "m.", 1e-6).reshape(n, H, V)
    q = P.silu(h @ w["m.q"].t()).reshape(n, H, D)
    v = (h @ w["m.v"].t()).reshape(n, H, V)
    f = (w["m.lower"] + (1 - w["m.lower"]) * torch.sigmoid(h @ w["m.f"].t() + w["m.f.b"])).reshape(n, H, D)
    for t in range(n):
        o = torch.zeros(H, V, dtype=F64)
        for j in range(t + 1):
            keep = torch.ones(H, D, dtype=F64)
            for s in range(j + 1, t + 1):
                keep = keep * f[s]
            o += torch.einsum("hk,hv->hv", q[t] * keep * (1 - f[j]), v[j])
        assert torch.allclose(P.unit(o, 1e-6), got[t], atol=1e-12)
    ww = {"m.mu." + s: torch.rand(d, dtype=F64) for s in "rkvgw"}
    ww.update({"m." + s: torch.randn(H * D, d, dtype=F64) for s in "rkvg"})
    ww.update({"m.w1": torch.randn(5, d, dtype=F64), "m.w2": torch.randn(H * D, 5, dtype=F64), "m.w0": torch.randn(H * D, dtype=F64) - 1,
               "m.u": torch.randn(H, D, dtype=F64), "m.norm": torch.ones(H * D, dtype=F64), "m.o": torch.eye(H * D, dtype=F64)})
    got = P.wkv_mixer(h, {"heads": H, "dim": D}, ww, "m.", 1e-6).reshape(n, H, D)
    before = torch.cat([torch.zeros(1, d, dtype=F64), h[:-1]])
    mix = {s: h + (before - h) * ww["m.mu." + s] for s in "rkvgw"}
    r, k, v = ((mix[s] @ ww["m." + s].t()).reshape(n, H, D) for s in "rkv")
    gate = P.silu(mix["g"] @ ww["m.g"].t()).reshape(n, H, D)
    dec = torch.exp(-torch.exp(torch.tanh(mix["w"] @ ww["m.w1"].t()) @ ww["m.w2"].t() + ww["m.w0"])).reshape(n, H, D)
    for t in range(n):
        o = torch.einsum("hk,hv->hv", r[t] * ww["m.u"] * k[t], v[t])
        for j in range(t):
            keep = torch.ones(H, D, dtype=F64)
            for s in range(j + 1, t):
                keep = keep * dec[s]
            o += torch.einsum("hk,hv->hv", r[t] * keep * k[j], v[j])
        assert torch.allclose(P.unit(o, 1e-6) * gate[t], got[t], atol=1e-12)


def test_plain_attention_sees_its_chunk_only():
    torch.manual_seed(1)
    n = 23
    q, k, v = torch.randn(n, 2, 4, dtype=F64), torch.randn(n, 1, 4, dtype=F64), torch.randn(n, 1, 3, dtype=F64)
    out = P.attend(q, k, v, 0.5, 4.0, 5)
    k2, v2 = k.clone(), v.clone()
    k2[:20] += 100.0      # whatever lies before position 22's chunk [20, 22] changes nothing for it
    v2[:20] -= 50.0
    out2 = P.attend(q, k2, v2, 0.5, 4.0, 5)
    assert torch.equal(out[20:], out2[20:]) and not torch.allclose(out[:20], out2[:20])
    assert torch.allclose(out[20], v[20, 0].expand(2, 3))      # the first position of a chunk sees itself alone
    s = torch.tensor([3.0, -2.0])
    assert torch.allclose(P.attend(q[:2], k[:2], v[:2], 1.0, None, None)[1, 0],
                          torch.softmax(k[:2, 0] @ q[1, 0], 0) @ v[:2, 0])
