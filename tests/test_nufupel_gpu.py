"""The Nufupel decoder through the engine against its plain implementation (tests/plain/nufupel_plain.py):
every mechanism alone, whole prompts against token-by-token decoding, prompts in portions, unequal batches,
slots and pages that are used again, keys at the edges of windows and pages, the first tokens of a sequence,
long decoding, sizes that the fast kernels take and sizes that they do not, and greedy generation through the
engine's own entry point.  The tests write their own weights (matrices of unit gain, loud sinks, a router whose
logits spread) so that every mechanism leaves a mark on the logits."""
import json
import math
import os

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import nufupel_plain as P
from tests.tiny import TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def mixer(heads, kv_heads, dim, vdim, window, scale, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=0):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mx, mlp, weights_of=None):
    out = {"type": kind, "mixer": mx, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


STRETCH = {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 96}
_M1 = layer("attention", mixer(6, 3, 24, 40, 50, 0.21), moe(6, 2, 48, 96))
# MIXED: value heads larger than keys, a shared expert of twice the experts' size (rides as two experts), a shared
# expert of another size (runs beside them), one expert per token, a layer run three times, a layer without a
# feed-forward whose window is a single key, a partial and a whole rotation with and without stretched frequencies
MIXED = {"architecture": "Nufupel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
         "logit_softcap": 2.5,
         "layers": [layer("attention_2", mixer(4, 2, 32, 32, 37, 0.18, {"dims": 16, "base": 5000.0, "scaling": STRETCH}), dense(136)),
                    _M1, dict(_M1, weights_of=1),
                    layer("attention_2", mixer(2, 2, 48, 16, 64, 0.15, {"dims": 48, "base": 1e4}), moe(5, 1, 40, 56)),
                    dict(_M1, weights_of=1),
                    layer("attention", mixer(3, 1, 16, 16, 1, 0.25), None)]}
# ODD: a width that is no multiple of 8 (products on CUDA cores), one head, every expert chosen, no shared expert,
# no cap, no window, no scale given, attention_2 without rotation
ODD = {"architecture": "Nufupel", "vocab": 97, "width": 100, "norm": {"eps": 1e-6},
       "layers": [layer("attention", {"heads": 1, "dim": 20}, moe(3, 3, 28)),
                  layer("attention_2", {"heads": 5, "kv_heads": 1, "dim": 8, "vdim": 12, "scale": 0.4, "mask": {"size": 9}}, dense(60)),
                  layer("attention", {"heads": 1, "dim": 20}, moe(3, 3, 28), weights_of=0)]}
# FAST: the head sizes of the tensor-core attention kernels, windows across several pages, widths the tensor-core
# products take
_F1 = layer("attention", mixer(4, 2, 64, 64, 100, 0.11), moe(8, 3, 80, 160))
FAST = {"architecture": "Nufupel", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3},
        "logit_softcap": 8.0,
        "layers": [layer("attention_2", mixer(4, 1, 128, 128, 300, 0.088, {"dims": 64, "base": 25000.0, "scaling": STRETCH}), dense(384)),
                   _F1, dict(_F1, weights_of=1),
                   layer("attention_2", mixer(8, 2, 64, 64, 70, 0.125, {"dims": 32, "base": 1e4}), moe(4, 2, 128)),
                   dict(_F1, weights_of=1)]}
CONFIGS = {"mixed": (MIXED, 3), "odd": (ODD, 5), "fast": (FAST, 7)}


def write_model(folder: str, raw: dict, seed: int) -> str:
    """A model folder with weights of the test's own making: matrices N(0, 1/in) so that activations keep their
    size from layer to layer, norm weights around zero, sinks around +1 (a fifth of the denominator at least),
    a router of gain 3 with a bias of its own."""
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import model_param_specs
    from odin_infer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    gen = torch.Generator().manual_seed(seed)
    specs = model_param_specs(cfg)

    def make(name):
        shape = next(s.concrete_shape for s in specs if s.name == name)
        r = torch.randn(shape, generator=gen)
        if name.endswith("sink"):
            t = 1.0 + r
        elif name.endswith("router.b"):
            t = 0.5 * r
        elif name.endswith(("norm1", "final.norm")):
            t = 0.3 * r
        elif name.endswith((".q.norm", ".k.norm")):
            t = 1.0 + 0.2 * r
        elif name == "embed":
            t = r / float(raw.get("embedding", {}).get("scale", 1.0))
        elif name.endswith("router"):
            t = 3.0 * r / math.sqrt(shape[1])
        elif name.endswith((".o", "down")):
            t = 0.5 * r / math.sqrt(shape[1])
        else:
            t = r / math.sqrt(shape[1])
        return t.to(torch.bfloat16)
    write_safetensors(os.path.join(folder, "model.safetensors"), [(s.name, torch.bfloat16, s.concrete_shape) for s in specs], make)
    return folder


_folders = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    if not _folders:
        base = tmp_path_factory.mktemp("nufupel")
        for name, (raw, seed) in CONFIGS.items():
            _folders[name] = write_model(os.path.join(str(base), name), raw, seed)
    return _folders


_plain = {}


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain:
        cfg, w = P.read_model_folder(folder, F64)
        _plain[key] = P.forward(cfg, w, tokens).numpy()
    return _plain[key]


def engine_for(folder, dtype, max_tokens=4096, max_ctx=1024, graphs=True):
    from odin_infer_b200 import Engine, Engine_Opts
    return Engine.load(folder, Engine_Opts(max_ctx=max_ctx, max_tokens=max_tokens, dtype=dtype, verbose=False,
                                           cuda_graphs=graphs))


def replay(engine, recs):
    from odin_infer_b200.engine.trace import replay as run
    return run(engine, recs)


def requests_for(raw, lengths, seed=0):
    return {f"r{i}": random_tokens(n, raw["vocab"], seed + i) for i, n in enumerate(lengths)}


# In bfloat16 a router's close call may fall the other way than in the plain implementation (the two differ by
# rounding in what the router reads); the token's update then differs by one expert's share (all of the experts'
# update where a token uses one expert), and later tokens see it through attention.  The serving engine is therefore
# assessed position by position: the median far inside the tolerance, one position in ten outside it at most, none
# wild (a token's logits after another expert are a different but ordinary row).  Every kernel alone is held to its
# tolerance in bfloat16 further down, with choices that are no close calls.  The 32-bit
# engine, whose router reads what the plain one reads to six digits, is held to the tolerance at every position.
def check_rows(got: dict, folder, requests, dtype):
    for rid, rows in got.items():
        ref = plain_logits(folder, requests[rid])[:rows.shape[0]]
        top = max(np.abs(ref).max(), 1e-30)
        err = np.abs(rows.astype(np.float64) - ref).max(axis=1) / top
        if dtype == "float32":
            assert err.max() <= TOL[dtype], f"{rid}: relative error {err.max():.3e} > {TOL[dtype]:.1e} at {int(err.argmax())}"
        else:
            over = int((err > TOL[dtype]).sum())
            assert over <= max(2, len(err) // 10) and err.max() <= 2.0 and np.median(err) <= TOL[dtype] / 4, \
                f"{rid}: {over} of {len(err)} positions over {TOL[dtype]:.1e}, median {np.median(err):.3e}, worst {err.max():.3e} at {int(err.argmax())}"


# --------------------------------------------------------------------------------------
# the whole model in every cut
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_one_by_one(folders, name, dtype):
    """Whole prompts (across several windows and pages), then the same with the last tokens one by one, so that
    decoding walks over window and page borders; the first tokens of a sequence alone (prompts of 1 and 2)."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [1, 2, 131, 330])
    engine = engine_for(folders[name], dtype)
    check_rows(traces.collect(traces.whole(reqs), replay(engine, traces.whole(reqs))), folders[name], reqs, dtype)
    recs = traces.tail_one_by_one(reqs, tail=70)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.cache.check()
    assert all(g.pool.n_held == 0 for g in engine.cache.groups.values())
    engine.destroy()


def portions(requests, sizes):
    """Each request alone, fed in portions of the given sizes in turn (the last one takes what is left)."""
    recs, n = [], 0
    for rid, toks in requests.items():
        at, i = 0, 0
        while at < len(toks):
            k = min(sizes[i % len(sizes)], len(toks) - at)
            recs.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + k], "want": list(range(k))}],
                         "end": [rid] if at + k == len(toks) else []})
            at, i, n = at + k, i + 1, n + 1
    return recs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,sizes", [("mixed", (2, 35, 3, 64)), ("odd", (17, 2, 2, 90)), ("fast", (130, 2, 70, 1, 129)),
                                        ("mixed", (2,))])
def test_prompts_in_portions(folders, name, sizes, dtype):
    """Portions of several sizes, down to two tokens: a portion's first tokens see the window's keys of the portions
    before it, from pages that a longer history has already given back in part."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [150, 41] if sizes == (2,) else [333, 77], seed=10)
    engine = engine_for(folders[name], dtype)
    recs = portions(reqs, sizes)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.destroy()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_and_reuse(folders, name, dtype, graphs):
    """Batches of unequal requests, batch after batch in a cache that holds one batch only, so that every slot and
    every page is used again; shorter requests end earlier."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [5, 180, 66, 1, 129, 40, 97, 260, 3], seed=20)
    recs = traces.batches(reqs, 3, first_part=lambda n: max(1, n - 9))
    engine = engine_for(folders[name], dtype, max_tokens=traces.max_live_tokens(recs) + 64, graphs=graphs)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.cache.check()
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_join_a_running_batch(folders, dtype):
    raw = CONFIGS["mixed"][0]
    reqs = requests_for(raw, [60, 45, 90, 30, 75], seed=30)
    recs = traces.joining(reqs)
    engine = engine_for(folders["mixed"], dtype)
    check_rows(traces.collect(recs, replay(engine, recs)), folders["mixed"], reqs, dtype)
    engine.destroy()


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_cuts_agree_bit_for_bit_in_32_bit(folders, name):
    """In 32-bit a position's logits are the same bits whole, in portions, one by one and in a batch."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [140, 59], seed=40)
    engine = engine_for(folders[name], "float32")
    ref = traces.collect(traces.whole(reqs), replay(engine, traces.whole(reqs)))
    for recs in (portions(reqs, (3, 50, 2)), traces.tail_one_by_one(reqs, tail=25), traces.batches(reqs, 2)):
        got = traces.collect(recs, replay(engine, recs))
        for rid in reqs:
            assert np.array_equal(got[rid], ref[rid]), rid
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "fast"])
def test_long_decoding(folders, name, dtype):
    """Three hundred tokens decoded one by one after a short prompt: every window passes over decoded tokens many
    times, and the pages that fall out of a window go back to the pool."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [330, 318], seed=50)
    recs = traces.batches(reqs, 2, first_part=lambda n: 12)
    engine = engine_for(folders[name], dtype)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    assert all(g.request.window > 0 for g in engine.cache.groups.values())
    assert all(g.pool.n_held == 0 for g in engine.cache.groups.values())
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt(folders, dtype):
    """A prompt of 1,100 tokens whole, and with its last 40 tokens one by one: windows many pages back from the start, block
    tables of 18 pages of which a window keeps two to six, experts with several tiles of rows each."""
    raw = CONFIGS["fast"][0]
    reqs = requests_for(raw, [1100], seed=70)
    engine = engine_for(folders["fast"], dtype, max_tokens=2048, max_ctx=1280)
    for recs in (traces.whole(reqs), traces.tail_one_by_one(reqs, tail=40)):
        check_rows(traces.collect(recs, replay(engine, recs)), folders["fast"], reqs, dtype)
    engine.cache.check()
    engine.destroy()


def test_window_groups_keep_a_cache_line_per_run_and_give_pages_back(folders):
    """A layer that runs several times keeps a line per run in one group; a windowed group holds only the pages
    that its window still reaches."""
    from odin_infer_b200 import StepEntry
    engine = engine_for(folders["mixed"], "float32")
    lines = {g.request.window: g.n_lines for g in engine.cache.groups.values()}
    assert lines == {37: 1, 50: 3, 64: 1, 1: 1}
    slot = engine.take_slot()
    engine.step([StepEntry(slot, random_tokens(200, 211, 1), [199])])
    held = {g.request.window: g.pool.n_held for g in engine.cache.groups.values()}
    # the next query sits at position 200: it sees from 200 - window + 1 on; pages are 64 tokens
    assert held == {37: 2, 50: 2, 64: 2, 1: 1}, held   # pages 2..3 (from 164, 151, 137), page 3 (from 200)
    engine.give_back_slot(slot)
    engine.destroy()


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-5), ("bfloat16", 6e-2)])
@pytest.mark.parametrize("name", ["mixed", "fast"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype, margin):
    """`Engine.generate` (the scheduler's batches, sampling on the device, one step ahead of the host): every token
    it chose is the plain logits' maximum, or within rounding of it."""
    raw = CONFIGS[name][0]
    prompts = [random_tokens(n, raw["vocab"], 60 + i) for i, n in enumerate((4, 150, 33, 71, 9))]
    engine = engine_for(folders[name], dtype, max_tokens=0, max_ctx=256)
    outs = engine.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain_logits(folders[name], p + o.tokens)
        for i, tok in enumerate(o.tokens):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= margin * float(np.abs(row).max()), (i, tok, int(row.argmax()))
    engine.destroy()


def test_the_command_line_generates(folders, capsys):
    from odin_infer_b200 import cli
    assert cli.main([folders["odd"], "--prompt-ids", "1,2,3,4", "-n", "5", "-t", "0", "-c", "128", "--json"]) == 0
    out = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert out and len(out[0]["tokens"]) == 5


def random_config(seed: int) -> dict:
    """A configuration drawn at random: order and number of layers, every size, every constant."""
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]   # noqa: E731
    width = pick([40, 64, 72, 96, 100, 128])
    layers, own = [], []
    for i in range(int(rng.integers(2, 7))):
        if own and rng.random() < 0.35:
            src = pick(own)
            layers.append(dict(layers[src], weights_of=src))
            continue
        kind = pick(["attention", "attention_2"])
        dim = pick([8, 16, 24, 40, 64, 64, 96, 128])
        kv = pick([1, 2, 3])
        mx = mixer(kv * pick([1, 2, 4]), kv, dim, pick([dim, dim, 8, 48]), pick([0, 1, 2, 17, 63, 64, 65, 130, 259]),
                   float(rng.uniform(0.08, 0.3)))
        if kind == "attention_2" and rng.random() < 0.85:
            mx["rot"] = {"dims": pick([dim, dim // 2, 2 * (dim // 8)]), "base": float(pick([1e3, 1e4, 25e4]))}
            if rng.random() < 0.6:
                mx["rot"]["scaling"] = {"factor": float(pick([2, 8, 32])), "low": 1.0, "high": float(pick([2, 4])),
                                        "original": int(pick([32, 128, 2048]))}
        kind_ff = pick(["none", "dense", "moe", "moe"])
        if kind_ff == "none":
            mlp = None
        elif kind_ff == "dense":
            mlp = dense(pick([40, 72, 128]))
        else:
            n = pick([2, 4, 7, 12])
            ff = pick([16, 40, 64])
            mlp = moe(n, int(rng.integers(1, n + 1)), ff, pick([0, ff, 2 * ff, ff + 8]))
        own.append(len(layers))
        layers.append(layer(kind, mx, mlp))
    cfg = {"architecture": "Nufupel", "vocab": int(rng.integers(40, 400)), "width": width,
           "norm": {"eps": float(pick([1e-5, 1e-6]))}, "embedding": {"scale": float(rng.uniform(0.5, 20))}, "layers": layers}
    if rng.random() < 0.7:
        cfg["logit_softcap"] = float(rng.uniform(1, 30))
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106, 107, 108])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Whole prompts, the last tokens one by one, and an unequal batch, for configurations that nobody chose."""
    raw = random_config(seed)
    folder = write_model(os.path.join(str(tmp_path), "m"), raw, seed)
    reqs = requests_for(raw, [1, 47, 290], seed=seed)
    engine = engine_for(folder, dtype)
    for recs in (traces.whole(reqs), traces.tail_one_by_one(reqs, tail=33), traces.batches(reqs, 3, first_part=lambda n: max(1, n - 20))):
        check_rows(traces.collect(recs, replay(engine, recs)), folder, reqs, dtype)
    engine.destroy()


# --------------------------------------------------------------------------------------
# every mechanism alone, with inputs that show a fault
# --------------------------------------------------------------------------------------
def close(got, ref, tol):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err <= tol, f"relative error {err:.3e} > {tol:.1e}"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 6e-3)])
@pytest.mark.parametrize("d", [96, 100, 7])
def test_one_plus_norm_adds_several_updates(dtype, tol, d):
    """x += a (two parts) + b + c (three parts), then x / rms * (1 + w): the sum goes back to x, the norm comes out;
    with a row gather x stays as it is."""
    from odin_infer_b200.parts.base import PartSpec, build_part
    from odin_infer_b200.engine.runtime import Runtime
    torch.manual_seed(d)
    rt = Runtime(DEV, dtype)
    norm = build_part("norm", PartSpec("rmsnorm", dict(width=d, eps=1e-5, weight="w", one_plus=True)))
    w = (0.3 * torch.randn(d, device=DEV)).to(dtype)
    norm.bind({"w": w}, rt)
    x = torch.randn(6, d, device=DEV) * 3
    a, b, c = torch.randn(2, 6, d, device=DEV), torch.randn(6, d, device=DEV), torch.randn(3, 6, d, device=DEV)
    want_x = x.double() + a.double().sum(0) + b.double() + c.double().sum(0)
    want_h = P.one_plus_norm(want_x.cpu(), w.double().cpu(), 1e-5)
    x1 = x.clone()
    close(norm.forward(rt, x1, [a, b, c]), want_h, tol)
    close(x1, want_x, 1e-6)
    x2 = x.clone()
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    close(norm.forward(rt, x2, [a, b, c], rows=rows), want_h[[4, 0, 4]], tol)
    assert torch.equal(x2, x)
    x3 = x.clone()
    close(norm.forward(rt, x3, b), P.one_plus_norm((x.double() + b.double()).cpu(), w.double().cpu(), 1e-5), tol)


def test_stretched_frequencies_have_all_three_branches():
    """Frequencies kept, divided and blended: against the plain formula, with constants under which each branch holds
    some of the pairs; the tables' angles are 32-bit products of position and frequency."""
    from odin_infer_b200.parts.position import RotaryEncoding
    for dims, base, sc in ((40, 70000.0, {"factor": 5.0, "low": 2.0, "high": 6.0, "original": 3000}),
                           (16, 5000.0, STRETCH), (48, 1e4, None), (2, 10.0, {"factor": 2.0, "low": 0.5, "high": 8.0, "original": 7})):
        pe = RotaryEncoding(dims, base, sc, precise=True)
        ref = P.stretched_frequencies(dims, base, sc)
        got = torch.from_numpy(pe.frequencies()).double()
        assert ((got - ref).abs() <= 1e-7 * ref.abs()).all()
        if sc is not None and dims >= 16:
            plain = P.stretched_frequencies(dims, base, None)
            ratio = (ref / plain).numpy()
            assert (ratio == 1.0).any() and np.isclose(ratio, 1.0 / sc["factor"]).any()
            assert ((ratio < 0.999) & (ratio > 1.001 / sc["factor"])).any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates_activations_and_the_cap(dtype):
    from odin_infer_b200.csrc import ops
    torch.manual_seed(1)
    T, H, vd = 5, 3, 12
    o = torch.randn(T, H * vd, device=DEV).to(dtype)
    # the gate as columns of a wider product that came back in two parts
    wide = torch.randn(2, T, 7 + H * vd, device=DEV)
    for per_head, n in ((False, H * vd), (True, H)):
        got = o.clone()
        ops.sigmoid_gate(got, wide[..., 7:7 + n], H, vd, per_head)
        g = torch.sigmoid(wide[..., 7:7 + n].double().sum(0))
        want = o.double().reshape(T, H, vd) * (g[:, :, None] if per_head else g.reshape(T, H, vd))
        close(got, want.reshape(T, H * vd), 1e-6 if dtype == torch.float32 else 8e-3)
    gu = torch.randn(3, T, 2 * 20, device=DEV) * 2
    for kind, act in (("silu", P.silu), ("gelu_tanh", P.gelu_tanh)):
        out = torch.empty(T, 20, dtype=dtype, device=DEV)
        ops.gated_activation(gu, kind, out)
        s = gu.double().sum(0)
        close(out, act(s[:, :20]) * s[:, 20:], 2e-6 if dtype == torch.float32 else 8e-3)
    z = torch.cat([torch.randn(4, 33, device=DEV) * 20, torch.tensor([[0.0, 1e-4, -1e-4, 300.0, -300.0] + [1.0] * 28], device=DEV)])
    want = 7.5 * torch.tanh(z.double() / 7.5)
    ops.softcap(z, 7.5)
    close(z, want, 1e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("E,top,always,d,ff", [(6, 2, 2, 96, 48), (3, 3, 0, 100, 28), (10, 3, 1, 64, 16), (40, 1, 0, 72, 8)])
def test_router_and_experts(dtype, tol, E, top, always, d, ff):
    """The router's choices and weights against a sort of the plain logits (logits made distinct by construction),
    padding rows, and the experts' update against a loop over tokens and choices."""
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine.runtime import Runtime
    torch.manual_seed(E * 7 + top)
    T = 9
    h = torch.randn(T, d, device=DEV).to(dtype)
    wr = (torch.randn(E, d, device=DEV) * 3 / math.sqrt(d)).to(dtype)
    bias = torch.randn(E, device=DEV)
    tok_seq = torch.tensor([0, 0, 1, -1, 2, 2, 2, -1, 3], dtype=torch.int32, device=DEV)
    ids = torch.empty(T, top + always, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top + always, dtype=torch.float32, device=DEV)
    ops.moe_router(h, wr, bias, top, always, tok_seq, ids, wts)
    ref_ids, ref_w = P.route(h.double().cpu(), wr.double().cpu(), bias.double().cpu(), top)
    real = (tok_seq >= 0).cpu()
    assert torch.equal(ids[:, :top].cpu()[real].long(), ref_ids[real])
    close(wts[:, :top].cpu()[real], ref_w[real], 1e-5)
    assert (ids.cpu()[~real] == -1).all() and (wts.cpu()[~real] == 0).all()
    if always:
        assert torch.equal(ids[:, top:].cpu()[real], torch.arange(E, E + always, dtype=torch.int32).expand(int(real.sum()), always))
        assert (wts[:, top:].cpu()[real] == 1).all()
    n_e = E + always
    wgu = (torch.randn(n_e, 2 * ff, d, device=DEV) / math.sqrt(d)).to(dtype)
    wd = (torch.randn(n_e, d, ff, device=DEV) / math.sqrt(ff)).to(dtype)
    from odin_infer_b200.engine import runtime as R
    old = R.MOE_GROUPED_FROM_ROWS
    try:
        R.MOE_GROUPED_FROM_ROWS = 1 << 30     # the row-by-row kernels (the grouped products have a test of their own)
        y = Runtime(DEV, dtype).experts(h, wgu, wd, ids, wts, "silu")
    finally:
        R.MOE_GROUPED_FROM_ROWS = old
    assert tuple(y.shape) == (top + always, T, d)
    want = torch.zeros(T, d, dtype=F64)
    hd_, g_, d_ = h.double().cpu(), wgu.double().cpu(), wd.double().cpu()
    for t in range(T):
        for k in range(top + always):
            e = int(ids[t, k])
            if e >= 0:
                a = P.silu(g_[e, :ff] @ hd_[t]) * (g_[e, ff:] @ hd_[t])
                want[t] += float(wts[t, k]) * (d_[e] @ a)
    close(y.sum(0), want, tol)
    assert (y[:, ~real.to(DEV)] == 0).all()


def test_ties_in_the_router_go_to_the_lower_index():
    from odin_infer_b200.csrc import ops
    h = torch.ones(2, 8, device=DEV)
    wr = torch.zeros(5, 8, device=DEV)
    bias = torch.tensor([1.0, 3.0, 3.0, 0.0, 3.0], device=DEV)
    ids = torch.empty(2, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(2, 2, dtype=torch.float32, device=DEV)
    ops.moe_router(h, wr, bias, 2, 0, None, ids, wts)
    assert ids.cpu().tolist() == [[1, 2], [1, 2]] and torch.allclose(wts.cpu(), torch.full((2, 2), 0.5))


def _paged(k, v, n_pages_extra=3, seed=0):
    """Keys and values [n, G, d] of one sequence scattered over scrambled pages; unwritten slots hold NaN."""
    from odin_infer_b200.cache import PAGE
    n, G, dk = k.shape
    dv = v.shape[2]
    n_pages = (n + PAGE - 1) // PAGE
    perm = np.random.default_rng(seed).permutation(n_pages + n_pages_extra)[:n_pages]
    kc = torch.full((n_pages + n_pages_extra, G, PAGE, dk), float("nan"), dtype=k.dtype, device=DEV)
    vc = torch.full((n_pages + n_pages_extra, G, PAGE, dv), float("nan"), dtype=v.dtype, device=DEV)
    for p in range(n_pages):
        rows = slice(p * PAGE, min(n, (p + 1) * PAGE))
        kc[perm[p], :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
        vc[perm[p], :, : rows.stop - rows.start] = v[rows].transpose(0, 1)
    bt = torch.full((1, n_pages + 2), -1, dtype=torch.int32, device=DEV)
    bt[0, :n_pages] = torch.from_numpy(perm.astype(np.int32))
    return kc, vc, bt


@pytest.mark.parametrize("kernel", ["plain32", "plain16", "decode", "prefill"])
@pytest.mark.parametrize("H,G,hd,window,n", [(4, 2, 64, 100, 333), (2, 1, 128, 70, 200), (4, 4, 64, 64, 130), (8, 2, 64, 300, 140),
                                            (6, 2, 80, 44, 150), (3, 1, 32, 1, 70), (4, 2, 64, 3, 200), (4, 2, 64, 65, 200), (2, 2, 128, 128, 300),
                                            (4, 1, 128, 1, 140), (4, 2, 64, 129, 450)])
def test_attention_kernels_with_a_sink_and_keys_at_the_windows_edge(kernel, H, G, hd, window, n):
    """One loud key is planted just inside the last query's window and one just outside it (and at a page's border);
    the sinks are loud enough to take a fifth to a half of the denominator.  Every kernel that serves the mixers
    against the plain loop: a kernel that is one token off, or leaves the sink out, is off by a large factor."""
    from odin_infer_b200.csrc import ops
    if kernel in ("decode", "prefill") and hd not in (64, 128) and not (kernel == "decode" and hd == 32):
        pytest.skip("the fast kernels take other head sizes")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    torch.manual_seed(H * 100 + window)
    q = torch.randn(n, H, hd, device=DEV) * 0.5
    k = torch.randn(n, G, hd, device=DEV) * 0.5
    v = torch.randn(n, G, hd, device=DEV)
    last = n - 1
    inside, outside = last - window + 1, last - window
    for g in range(G):
        if inside >= 0:
            k[inside, g] = q[last, g * (H // G)] * 3.0      # loud for the last query, and seen
            v[inside, g] += 5.0
        if outside >= 0:
            k[outside, g] = q[last, g * (H // G)] * 6.0     # louder still, and hidden from it
            v[outside, g] -= 9.0
    sink = (torch.randn(H, device=DEV) + 2.0).float()
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 0.11
    want = P.window_sink_attention(q.double().cpu(), k.double().cpu(), v.double().cpu(), scale, window, sink.double().cpu())
    kc, vc, bt = _paged(k, v, seed=n)
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    q2 = q.reshape(n, H * hd).contiguous()
    if kernel in ("plain32", "plain16", "prefill"):
        out = torch.zeros(n, H * hd, dtype=dtype, device=DEV)
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        seq = torch.zeros(n, dtype=torch.int32, device=DEV)
        if kernel == "prefill":
            ops.attention_prefill(q2, out, 1, n, H, G, hd, kc, vc, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                                  torch.tensor([n], dtype=torch.int32, device=DEV), bt, window, 0, scale, 0.0, sink)
            torch.cuda.synchronize()
            ops.attention_prefill_check()
        else:
            ops.attention_plain(q2, out, H, G, hd, kc, vc, pos, seq, bt, window, 0, scale, 0.0, None, sink)
        close(out.reshape(n, H, hd), want, tol)
        # without the sink the same kernel is far off: the sink is not a rounding matter
        bare = torch.zeros_like(out)
        if kernel != "prefill":
            ops.attention_plain(q2, bare, H, G, hd, kc, vc, pos, seq, bt, window, 0, scale, 0.0, None, None)
            assert (bare.double().cpu().reshape(n, H, hd) - want).abs().max() > 0.05 * want.abs().max()
        return
    # decoding: the last few tokens, each as a step of its own row, in every number of key splits
    rows = [last, last - 1, max(0, last - 70)]
    pos = torch.tensor(rows, dtype=torch.int32, device=DEV)
    bt3 = bt.expand(3, -1).contiguous()
    seq = torch.arange(3, dtype=torch.int32, device=DEV)
    for n_split in (1, 2, 5):
        out = torch.zeros(3, H * hd, dtype=dtype, device=DEV)
        scratch = torch.empty(ops.attention_decode_scratch(3, H, hd, n_split), dtype=torch.float32, device=DEV)
        ops.attention_decode(q2[rows].contiguous(), out, H, G, hd, kc, vc, pos, seq, bt3, window, scratch, n_split, 0, scale, 0.0, sink)
        torch.cuda.synchronize()
        ops.attention_decode_check()
        close(out.reshape(3, H, hd), want[rows], tol)


@pytest.mark.parametrize("T,E,top,always,d,ff", [(300, 6, 2, 2, 128, 96), (700, 10, 3, 1, 64, 64), (257, 3, 1, 0, 256, 136),
                                                 (90, 40, 3, 0, 72, 8)])
def test_experts_as_grouped_tensor_core_products(T, E, top, always, d, ff):
    """Many rows: sorted by expert, padded to tiles, multiplied by the tile's own expert on the tensor cores.  Against
    a loop over tokens and choices; experts without a row, experts with more than a tile of rows, an inner size that
    is no multiple of the tile; twice with equal bits (the places differ from run to run, the values do not); padding
    rows; and against the row-by-row kernels."""
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine import runtime as R
    torch.manual_seed(T + E)
    dtype = torch.bfloat16
    h = torch.randn(T, d, device=DEV).to(dtype)
    wr = (torch.randn(E, d, device=DEV) * 3 / math.sqrt(d)).to(dtype)
    wr[E // 2] = 0          # an expert that is chosen by its bias alone ...
    bias = torch.randn(E, device=DEV)
    bias[E // 2] = -50.0    # ... never
    bias[0] = 2.5           # and one that most tokens choose: more than a tile of rows
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    tok_seq[5] = tok_seq[T - 1] = -1
    ids = torch.empty(T, top + always, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top + always, dtype=torch.float32, device=DEV)
    ops.moe_router(h, wr, bias, top, always, tok_seq, ids, wts)
    n_e = E + always
    wgu = (torch.randn(n_e, 2 * ff, d, device=DEV) / math.sqrt(d)).to(dtype)
    wd = (torch.randn(n_e, d, ff, device=DEV) / math.sqrt(ff)).to(dtype)
    rt = R.Runtime(DEV, dtype)
    old = R.MOE_GROUPED_FROM_ROWS
    try:
        R.MOE_GROUPED_FROM_ROWS = 1
        y1 = rt.experts(h, wgu, wd, ids, wts, "silu")
        y2 = rt.experts(h, wgu, wd, ids, wts, "silu")
        g1 = rt.experts(h, wgu, wd, ids, wts, "gelu_tanh")
        R.MOE_GROUPED_FROM_ROWS = 1 << 30
        rows = rt.experts(h, wgu, wd, ids, wts, "silu")
    finally:
        R.MOE_GROUPED_FROM_ROWS = old
    torch.cuda.synchronize()
    ops.moe_tc_check()
    assert tuple(y1.shape) == (T, d) and tuple(rows.shape) == (top + always, T, d)
    assert torch.equal(y1, y2)
    assert (y1[5] == 0).all() and (y1[T - 1] == 0).all()
    hd_, g_, d_ = h.double().cpu(), wgu.double().cpu(), wd.double().cpu()
    idc, wtc = ids.cpu(), wts.double().cpu()
    for act, got in ((P.silu, y1), (P.gelu_tanh, g1)):
        want = torch.zeros(T, d, dtype=F64)
        for k in range(top + always):
            e = idc[:, k].long()
            ok = e >= 0
            ee = e.clamp(min=0)
            a = act(torch.einsum("tfd,td->tf", g_[ee, :ff], hd_)) * torch.einsum("tfd,td->tf", g_[ee, ff:], hd_)
            a = a.to(torch.bfloat16).double()    # the activations between the two products are bfloat16
            want += torch.where(ok[:, None], wtc[:, k, None] * torch.einsum("tdf,tf->td", d_[ee], a), torch.zeros(1, dtype=F64))
        close(got, want, 4e-3)
    close(rows.sum(0), y1, 4e-3)
