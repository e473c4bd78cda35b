"""The Tovalix decoder through the engine against its plain implementation (tests/plain/tovalix_plain.py):
every mechanism alone, whole prompts against token-by-token decoding, prompts in portions, unequal batches,
slots and pages that are used again, keys at the edges of chunks and pages, long decoding, sizes that the
fast kernels take and sizes that they do not, and greedy generation through the engine's own entry point."""
import json
import os

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import tovalix_plain as P
from tests.tiny import TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def att(heads, kv_heads, dim, vdim, rot, base, chunk, scale, cap=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot, "base": base},
         "mask": {"size": chunk}}
    if cap:
        m["softcap"] = cap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# every size differs between the configurations; ODD has a width that is no multiple of 8 (products on CUDA
# cores), head sizes that the recurrence keeps outside its register kernels, one group, one kv head per query
# head, a layer without a feed-forward and a reader whose chunk differs from its writer's; FAST has the head
# sizes of the tensor-core attention kernels and no token input.
MIXED = {"architecture": "Tovalix", "vocab": 211, "width": 96, "norm": {"eps": 1e-5, "groups": 3}, "token_side": {"dim": 8},
         "layers": [layer("wkv", {"heads": 3, "dim": 16, "decay_rank": 8}, 136),
                    layer("attention", att(6, 2, 32, 16, 16, 1e4, 37, 0.2, 8.0), 0),
                    layer("hgrn2", {"heads": 2, "dim": 24, "vdim": 40}, 200),
                    layer("attention", att(6, 2, 32, 16, 16, 1e4, 50, 0.15, 12.0, kv_from=1), 64),
                    layer("attention", att(2, 2, 48, 48, 48, 3e5, 64, 0.3), 128)]}
ODD = {"architecture": "Tovalix", "vocab": 97, "width": 100, "norm": {"eps": 1e-6, "groups": 1}, "token_side": {"dim": 5},
       "layers": [layer("hgrn2", {"heads": 1, "dim": 20, "vdim": 12}, 60),
                  layer("attention", att(3, 3, 24, 8, 8, 777.0, 16, 0.25, 5.0), 44),
                  layer("wkv", {"heads": 2, "dim": 40, "decay_rank": 12}, 0),
                  layer("attention", att(3, 3, 24, 8, 8, 777.0, 16, 0.25, 5.0, kv_from=1), 36)]}
FAST = {"architecture": "Tovalix", "vocab": 512, "width": 128, "norm": {"eps": 1e-5, "groups": 4},
        "layers": [layer("attention", att(4, 2, 64, 64, 64, 5e4, 100, 0.125, 15.0), 256),
                   layer("attention", att(4, 2, 64, 64, 64, 5e4, 100, 0.125, 15.0, kv_from=0), 192),
                   layer("wkv", {"heads": 2, "dim": 64, "decay_rank": 16}, 256),
                   layer("hgrn2", {"heads": 2, "dim": 64, "vdim": 64}, 0),
                   layer("attention", att(2, 1, 128, 128, 64, 1e4, 300, 0.09, 30.0), 128)]}
CONFIGS = {"mixed": (MIXED, 3), "odd": (ODD, 5), "fast": (FAST, 7)}


_folders = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import write_random_model
    if not _folders:
        base = tmp_path_factory.mktemp("tovalix")
        for name, (raw, seed) in CONFIGS.items():
            _folders[name] = write_random_model(os.path.join(str(base), name), config_from_dict(raw), seed)
    return _folders


_plain = {}


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain:
        cfg, w = P.read_model_folder(folder, F64)
        _plain[key] = P.forward_whole(cfg, w, tokens).numpy()
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


def check_rows(got: dict, folder, requests, dtype):
    for rid, rows in got.items():
        ref = plain_logits(folder, requests[rid])
        err = rel_err(rows, ref[:rows.shape[0]])
        assert err <= TOL[dtype], f"{rid}: relative error {err:.3e} > {TOL[dtype]:.1e}"


# --------------------------------------------------------------------------------------
# the whole model in every cut
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_one_by_one(folders, name, dtype):
    """Whole prompts (across several chunks and pages), then the same with the last tokens one by one, so that
    decoding walks over chunk and page borders; the first tokens of a sequence alone (prompts of 1 and 2)."""
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
    """Portions of several sizes, down to two tokens: the state, the token shift and the chunk's first key go
    from portion to portion."""
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
    """Batches of unequal requests, batch after batch in a cache that holds one batch only, so that every slot
    (with its recurrent state) and every page is used again; shorter requests end earlier."""
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


def test_cuts_agree_bit_for_bit_in_32_bit(folders):
    """In 32-bit a position's logits are the same bits whole, in portions, one by one and in a batch."""
    raw = CONFIGS["mixed"][0]
    reqs = requests_for(raw, [140, 59], seed=40)
    engine = engine_for(folders["mixed"], "float32")
    ref = traces.collect(traces.whole(reqs), replay(engine, traces.whole(reqs)))
    for recs in (portions(reqs, (3, 50, 2)), traces.tail_one_by_one(reqs, tail=25), traces.batches(reqs, 2)):
        got = traces.collect(recs, replay(engine, recs))
        for rid in reqs:
            assert np.array_equal(got[rid], ref[rid]), rid
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """Three hundred tokens decoded one by one after a short prompt: the state is carried three hundred times,
    the chunks turn over several times, pages of past chunks go back to the pool."""
    raw = CONFIGS["mixed"][0]
    reqs = requests_for(raw, [330, 318], seed=50)
    recs = traces.batches(reqs, 2, first_part=lambda n: 12)
    engine = engine_for(folders["mixed"], dtype)
    check_rows(traces.collect(recs, replay(engine, recs)), folders["mixed"], reqs, dtype)
    chunked = [g for g in engine.cache.groups.values() if g.request.chunk > 0]
    assert chunked and all(g.pool.n_held == 0 for g in engine.cache.groups.values())
    engine.destroy()


def test_chunk_groups_give_pages_back(folders):
    """A layer that sees only its chunk keeps only the chunk's pages; a line whose reader has another chunk keeps all."""
    from odin_infer_b200 import StepEntry
    engine = engine_for(folders["mixed"], "float32")
    slot = engine.take_slot()
    engine.step([StepEntry(slot, random_tokens(200, 211, 1), [199])])
    held = {key: g.pool.n_held for key, g in engine.cache.groups.items()}
    by_chunk = {g.request.chunk: g.pool.n_held for g in engine.cache.groups.values()}
    assert by_chunk[64] == 1          # positions 192.. of the chunk [192, 256)
    assert by_chunk[0] == 4, held     # chunks 37 and 50 share a line: everything is kept
    engine.give_back_slot(slot)
    engine.destroy()


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-5), ("bfloat16", 3e-2)])
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
    groups = pick([1, 2, 3, 4])
    width = groups * pick([8, 12, 20, 24, 32]) * pick([1, 2])
    layers, writers = [], []
    for i in range(int(rng.integers(3, 7))):
        kind = pick(["attention", "attention", "wkv", "hgrn2"])
        ff = pick([0, 40, 72, 128])
        if kind == "attention":
            if writers and rng.random() < 0.5:
                src = pick(writers)
                m = json.loads(json.dumps(layers[src]["mixer"]))
                m.update(kv_from=src, scale=float(rng.uniform(0.05, 0.4)), mask={"size": int(rng.integers(3, 260))})
                m["heads"] = m["kv_heads"] * pick([1, 2, 3])
                if rng.random() < 0.5:
                    m["softcap"] = float(rng.uniform(3, 40))
            else:
                dim = pick([16, 24, 40, 64, 64, 96, 128])
                kv = pick([1, 2, 3])
                m = att(kv * pick([1, 2, 4]), kv, dim, pick([dim, dim, 8, 48]), pick([dim, dim, dim // 2, 2 * (dim // 8)]),
                        float(pick([1e3, 1e4, 5e5])), int(rng.integers(3, 260)), float(rng.uniform(0.05, 0.4)),
                        float(rng.uniform(3, 40)) if rng.random() < 0.8 else None)
                writers.append(i)
        elif kind == "wkv":
            m = {"heads": pick([1, 2, 5]), "dim": pick([8, 16, 24, 64]), "decay_rank": pick([4, 8, 24])}
        else:
            m = {"heads": pick([1, 3, 4]), "dim": pick([8, 20, 32, 64]), "vdim": pick([8, 12, 32, 64])}
        layers.append(layer(kind, m, ff))
    cfg = {"architecture": "Tovalix", "vocab": int(rng.integers(40, 400)), "width": width,
           "norm": {"eps": float(pick([1e-5, 1e-6])), "groups": groups}, "layers": layers}
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": pick([3, 8, 16])}
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106, 107, 108])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Whole prompts, the last tokens one by one, and an unequal batch, for configurations that nobody chose."""
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import write_random_model
    raw = random_config(seed)
    folder = write_random_model(os.path.join(str(tmp_path), "m"), config_from_dict(raw), seed)
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
@pytest.mark.parametrize("d,groups", [(96, 3), (100, 1), (64, 64), (20, 4)])
def test_group_norm_with_update_and_bias(dtype, tol, d, groups):
    from odin_infer_b200.csrc import ops
    torch.manual_seed(d)
    x, delta = torch.randn(7, d, device=DEV) * 3, torch.randn(2, 7, d, device=DEV)
    x[:, : d // groups] *= 50    # one loud group must not quieten the others
    bias, w = torch.randn(d, device=DEV).to(dtype), (1 + 0.2 * torch.randn(d, device=DEV)).to(dtype)
    x0 = x.clone()
    out = torch.empty(7, d, dtype=dtype, device=DEV)
    ops.row_update(x, delta, bias, w, 1e-5, groups, out)
    new = x0.double() + delta.double().sum(0) + bias.double()
    close(x, new, 1e-6)
    close(out, P.group_norm(new.cpu(), w.double().cpu(), groups, 1e-5), tol)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, d, dtype=dtype, device=DEV)
    ops.row_update(x, None, None, w, 1e-5, groups, picked, rows)
    close(picked, P.group_norm(new.cpu(), w.double().cpu(), groups, 1e-5)[[5, 0, 5]], tol)
    inplace = x.clone()
    ops.row_update(inplace, None, None, w, 1e-5, groups, inplace)
    close(inplace, P.group_norm(new.cpu(), w.double().cpu(), groups, 1e-5), 3e-6)


def test_activations_and_the_normed_add():
    from odin_infer_b200.csrc import ops
    torch.manual_seed(0)
    z = torch.cat([torch.randn(5, 33, device=DEV) * 4, torch.tensor([[0.0, -0.0, 1e-4, -1e-4, 30.0, -30.0] + [0.5] * 27], device=DEV)])
    pq = torch.tensor([0.3, -0.7], device=DEV)
    for kind, ref in (("tanh", torch.tanh), ("silu", P.silu), ("gelu_tanh", P.gelu_tanh), ("xielu", lambda t: P.xielu(t, pq.double().cpu()))):
        out = torch.empty_like(z)
        ops.activation(z, kind, out, pq if kind == "xielu" else None)
        close(out, ref(z.double().cpu()), 2e-6)
    parts = torch.randn(3, 6, 33, device=DEV)
    out = torch.empty(6, 33, dtype=torch.bfloat16, device=DEV)
    ops.activation(parts, "xielu", out, pq)
    close(out, P.xielu(parts.double().cpu().sum(0), pq.double().cpu()), 6e-3)
    x, y, w = torch.randn(6, 33, device=DEV), torch.randn(2, 6, 33, device=DEV) * 7, torch.randn(33, device=DEV)
    x0 = x.clone()
    seq = torch.tensor([0, 0, -1, 1, 1, 1], dtype=torch.int32, device=DEV)
    ops.normed_add(x, y, w, 1e-5, seq)
    ref = x0.double().cpu() + P.unit(y.double().cpu().sum(0), 1e-5) * w.double().cpu()
    ref[2] = x0[2].double().cpu()     # a padding row stays as it was
    close(x, ref, 2e-6)


def _recurrence_inputs(T, H, dk, dv, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(T, H * dk, generator=g), torch.randn(T, H * dk, generator=g), torch.randn(T, H * dk, generator=g) * 2,
            torch.randn(T, H * dv, generator=g), torch.randn(H * dk, generator=g), torch.rand(H * dk, generator=g))


def plain_recurrence(mode, q, k, g, v, c0, c1, H, dk, dv, S):
    """The recurrence token by token in float64; returns the outputs, updates S in place."""
    T = q.shape[0]
    q, k, g, v = (t.double().reshape(T, H, -1) for t in (q, k, g, v))
    c0, c1 = c0.double().reshape(H, dk), c1.double().reshape(H, dk)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        if mode == "bonus":
            w = torch.exp(-torch.exp(g[t] + c0))
            kv = k[t][:, :, None] * v[t][:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S + c1[:, :, None] * kv, q[t])
            S.copy_(w[:, :, None] * S + kv)
        else:
            f = c1 + (1 - c1) * torch.sigmoid(g[t] + c0)
            S.copy_(f[:, :, None] * S + (1 - f)[:, :, None] * v[t][:, None, :])
            out[t] = torch.einsum("hkv,hk->hv", S, P.silu(q[t]))
    return out.reshape(T, H * dv)


@pytest.mark.parametrize("mode", ["bonus", "gated"])
@pytest.mark.parametrize("H,dk,dv", [(3, 16, 16), (2, 64, 64), (1, 20, 12), (2, 40, 72), (2, 128, 32), (1, 160, 136), (1, 256, 8)])
def test_linear_recurrence_alone(mode, H, dk, dv):
    """Two sequences of unequal length and an empty one in one launch, then a second launch that goes on from the
    state; state rows far apart (another mixer's bytes between them); register kernels and the general one."""
    from odin_infer_b200.csrc import ops
    lens = [37, 0, 9]
    T = sum(lens)
    q, k, g, v, c0, c1 = _recurrence_inputs(2 * T, H, dk, dv, seed=dk + dv)
    n_state = H * dk * dv
    state = torch.zeros(5, n_state + 24, device=DEV)
    slots = torch.tensor([3, 0, 1], dtype=torch.int32, device=DEV)
    starts = torch.tensor([0, 37, 37, 46], dtype=torch.int32, device=DEV)
    S_ref = {3: torch.zeros(H, dk, dv, dtype=F64), 1: torch.zeros(H, dk, dv, dtype=F64)}
    dev = [t.to(DEV) for t in (q, k, g, v, c0, c1)]
    for call in range(2):
        rows = slice(call * T, (call + 1) * T)
        out = torch.empty(T, H * dv, device=DEV)
        ops.linear_recurrence(mode, dev[0][rows], dev[1][rows] if mode == "bonus" else None, dev[2][rows], dev[3][rows], dev[4],
                              dev[5], out, state[:, :n_state], starts, slots, 3, H, dk, dv)
        at = call * T
        for slot, n in ((3, 37), (1, 9)):
            ref = plain_recurrence(mode, q[at:at + n], k[at:at + n], g[at:at + n], v[at:at + n], c0, c1, H, dk, dv, S_ref[slot])
            close(out[at - call * T:at - call * T + n], ref, 5e-6)
            at += n
    close(state[3, :n_state], S_ref[3].reshape(-1), 5e-6)
    assert float(state[0].abs().max()) == 0 and float(state[:, n_state:].abs().max()) == 0   # the empty sequence's slot, the neighbours' bytes


@pytest.mark.parametrize("mode", ["bonus", "gated"])
@pytest.mark.parametrize("H,dk,dv,block", [(2, 64, 64, 32), (3, 16, 24, 7), (1, 128, 40, 64), (2, 40, 72, 16), (1, 200, 256, 50)])
def test_linear_recurrence_in_blocks_of_tokens(mode, H, dk, dv, block):
    """The same recurrence with every sequence cut into blocks that are walked side by side: sequences of 150, 0, 1 and
    block + 1 tokens that go on from a state which is not zero, against the walk token by token in float64."""
    from odin_infer_b200.csrc import ops
    lens = [150, 0, 1, block + 1]
    T = sum(lens)
    q, k, g, v, c0, c1 = _recurrence_inputs(T, H, dk, dv, seed=3 * dk + dv)
    n_state = H * dk * dv
    state = torch.randn(6, n_state + 8, device=DEV)
    slots = torch.tensor([4, 0, 2, 5], dtype=torch.int32, device=DEV)
    starts = torch.tensor([0, 150, 150, 151, T], dtype=torch.int32, device=DEV)
    before = state.clone()
    dev = [t.to(DEV) for t in (q, k, g, v, c0, c1)]
    out = torch.empty(T, H * dv, device=DEV)
    ops.linear_recurrence(mode, dev[0], dev[1] if mode == "bonus" else None, dev[2], dev[3], dev[4], dev[5], out,
                          state[:, :n_state], starts, slots, 4, H, dk, dv, block_len=block, max_new=150)
    at = 0
    for slot, n in zip(slots.tolist(), lens):
        if n == 0:
            continue
        S = before[slot, :n_state].double().cpu().reshape(H, dk, dv).clone()
        ref = plain_recurrence(mode, q[at:at + n], k[at:at + n], g[at:at + n], v[at:at + n], c0, c1, H, dk, dv, S)
        close(out[at:at + n], ref, 2e-5)
        close(state[slot, :n_state], S.reshape(-1), 2e-5)
        at += n
    assert torch.equal(state[0], before[0]) and torch.equal(state[:, n_state:], before[:, n_state:])


def test_token_shift_alone():
    from odin_infer_b200.csrc import ops
    torch.manual_seed(3)
    d, T = 40, 9
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 5e-3)):
        h = torch.randn(T, d, device=DEV).to(dtype)
        mu = torch.rand(3, d, device=DEV).to(dtype)
        state = torch.randn(4, d + 8, device=DEV)
        seq = torch.tensor([0, 0, 0, 0, -1, 1, 1, 2, -1], dtype=torch.int32, device=DEV)
        starts = torch.tensor([0, 5, 7, 8], dtype=torch.int32, device=DEV)
        slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
        out = torch.zeros(3, T, d, dtype=dtype, device=DEV)
        ops.token_shift(h, state[:, :d], mu, out, seq, starts, slots)
        hd, md = h.double().cpu(), mu.double().cpu()
        for t in range(T):
            if seq[t] < 0:
                assert float(out[:, t].abs().max()) == 0
                continue
            first = int(starts[int(seq[t])])
            before = state[int(slots[int(seq[t])]), :d].double().cpu() if t == first else hd[t - 1]
            close(out[:, t], hd[t] + (before - hd[t]) * md, tol)


def _paged(k, v, n_pages_extra=3, dtype=torch.float32, seed=0):
    """Keys [n, G, dk] and values [n, G, dv] scattered over scrambled pages; unwritten slots hold NaN."""
    n, G, dk = k.shape
    dv = v.shape[2]
    pages = (n + 63) // 64
    perm = torch.randperm(pages + n_pages_extra, generator=torch.Generator().manual_seed(seed))[:pages]
    kc = torch.full((pages + n_pages_extra, G, 64, dk), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((pages + n_pages_extra, G, 64, dv), float("nan"), dtype=dtype, device=DEV)
    for p in range(pages):
        rows = slice(p * 64, min(n, (p + 1) * 64))
        kc[perm[p], :, : rows.stop - rows.start] = k[rows].transpose(0, 1).to(dtype).to(DEV)
        vc[perm[p], :, : rows.stop - rows.start] = v[rows].transpose(0, 1).to(dtype).to(DEV)
    return kc, vc, perm.to(torch.int32).to(DEV).reshape(1, -1)


def planted(n, H, G, dk, dv, places, strength, seed):
    """Random unit queries and keys; for every (query position, key position) pair of `places` the key is made
    the query's own direction, so that its score stands out (if it is visible) or must not (if it is not)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(n, H, dk, generator=g, dtype=F64), dim=-1) * dk ** 0.5
    k = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g, dtype=F64), dim=-1) * dk ** 0.5
    v = torch.randn(n, G, dv, generator=g, dtype=F64)
    for qp, kp in places:
        k[kp] = q[qp, :: H // G] * strength
        v[kp] += 3.0
    return q, k, v


@pytest.mark.parametrize("hd,vd,H,G,chunk,cap", [(24, 8, 3, 3, 16, 5.0), (32, 16, 6, 2, 37, 8.0), (64, 64, 4, 2, 100, 15.0),
                                                   (128, 128, 2, 1, 300, 0.0), (64, 64, 4, 4, 64, 20.0), (32, 32, 4, 1, 50, 6.0)])
def test_attention_kernels_at_the_edges(hd, vd, H, G, chunk, cap):
    """Every attention kernel against the plain function: a key that stands out far back in the chunk, just inside
    the chunk (its first position), just outside (the position before), at a page's last and first slot, for queries
    in a prompt's portion and for queries decoded alone; pages scrambled, unwritten slots NaN."""
    from odin_infer_b200.csrc import ops
    n = 700
    scale = 1.0 / hd ** 0.5
    last = n - 1
    c0 = (last // chunk) * chunk
    mid = n - 200
    m0 = (mid // chunk) * chunk
    places = [(last, c0), (last - 1, max(c0 - 1, 0)), (mid, m0), (mid + 1, max(m0 - 1, 0)), (last - 2, (last // 64) * 64 - 1),
              (last - 3, (last // 64) * 64), (mid + 2, mid + 2)]
    q, k, v = planted(n, H, G, hd, vd, places, 2.0, seed=hd + chunk)
    ref = P.attend(q, k, v, scale, cap or None, chunk)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    seq = torch.zeros(n, dtype=torch.int32, device=DEV)
    for dtype, tol in ((torch.float32, 5e-6), (torch.bfloat16, 2e-2)):
        kc, vc, bt = _paged(k, v, dtype=dtype, seed=hd)
        qd = q.reshape(n, H * hd).to(dtype).to(DEV)
        out = torch.empty(n, H * vd, dtype=dtype, device=DEV)
        ops.attention_plain(qd, out, H, G, hd, kc, vc, pos, seq, bt, 0, chunk, scale, cap, vd)
        close(out, ref.reshape(n, -1), tol)
    if vd != hd:
        return
    # a prompt's second portion on the tensor cores (the first 300 positions are in the cache already) ...
    if ops.attention_prefill_supported(hd):
        first = 300
        out = torch.zeros(n - first, H * vd, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill(qd[first:], out, 1, n - first, H, G, hd, kc, vc,
                              torch.tensor([0, n - first], dtype=torch.int32, device=DEV),
                              torch.tensor([n], dtype=torch.int32, device=DEV), bt, 0, chunk, scale, cap)
        ops.attention_prefill_check()
        close(out, ref.reshape(n, -1)[first:], 2e-2)
    # ... and single queries on the split-key kernel, alone and in a batch, with one to five splits
    if ops.attention_decode_supported(hd):
        for rows in ([last], [mid, last - 1, mid + 1, last - 2, last - 3, mid + 2, last]):
            for n_split in (1, 2, 5):
                B = len(rows)
                # every row is a sequence of its own over the same pages, at its own position
                tp = torch.tensor(rows, dtype=torch.int32, device=DEV)
                ts = torch.arange(B, dtype=torch.int32, device=DEV)
                out = torch.zeros(B, H * vd, dtype=torch.bfloat16, device=DEV)
                scratch = torch.empty(ops.attention_decode_scratch(B, H, hd, n_split), device=DEV)
                ops.attention_decode(qd[rows].contiguous(), out, H, G, hd, kc, vc, tp, ts, bt.expand(B, -1).contiguous(), 0,
                                     scratch, n_split, chunk, scale, cap)
                ops.attention_decode_check()
                close(out, ref.reshape(n, -1)[rows], 2e-2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 4e-6), (torch.bfloat16, 8e-3)])
def test_head_preparation_with_bias_partial_rotation_and_unit_norm(dtype, tol):
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.parts import PartSpec, build_part
    from odin_infer_b200.engine.runtime import Runtime
    H, G, hd, vd, rot, base, T = 3, 1, 40, 24, 16, 2e4, 70
    torch.manual_seed(4)
    width = (H + G) * hd + G * vd
    qkv = torch.randn(2, T, width, device=DEV)
    bias = torch.randn(width, device=DEV).to(dtype)
    pe = build_part("position_encoding", PartSpec("rope", dict(rotary_dim=rot, theta=base)))
    pe.prepare(Runtime(DEV, dtype), 128)
    kc = torch.zeros(3, G, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros(3, G, 64, vd, dtype=dtype, device=DEV)
    bt = torch.tensor([[2, 0, -1]], dtype=torch.int32, device=DEV)
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device=DEV)
    q_out = torch.empty(T, H * hd, dtype=dtype, device=DEV)
    ops.head_prep(qkv, H, G, hd, None, None, 1e-5, pe.cos, pe.sin, rot, pos, torch.zeros(T, dtype=torch.int32, device=DEV), bt,
                  kc, vc, q_out=q_out, bias=bias, unit_norm_after=True, v_head_dim=vd)
    full = qkv.double().cpu().sum(0) + bias.double().cpu()
    qr = P.unit(P.rotate_half(full[:, : H * hd].reshape(T, H, hd), pos.cpu(), rot, base), 1e-5)
    kr = P.unit(P.rotate_half(full[:, H * hd:(H + G) * hd].reshape(T, G, hd), pos.cpu(), rot, base), 1e-5)
    close(q_out, qr.reshape(T, -1), tol)
    for t in (0, 58, 59, 69):      # positions 5, 63 | 64, 74: both sides of the page border
        p = 5 + t
        page = [2, 0][p // 64]
        close(kc[page, :, p % 64], kr[t], tol)
        close(vc[page, :, p % 64], full[t, (H + G) * hd:].reshape(G, vd), tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_token_input_and_feed_forward_parts(dtype, tol):
    from tests.test_parts_gpu import make_step, runtime
    from odin_infer_b200.parts import PartSpec, build_part
    rt = runtime(dtype)
    torch.manual_seed(5)
    width, dim, vocab, tw = 72, 10, 50, 30
    names = {"table": "t", "gate": "g", "proj": "p", "norm": "n"}
    side = build_part("block_extra", PartSpec("token_side_input", dict(width=width, dim=dim, vocab_size=vocab, table_width=tw,
                                                                       first_column=20, names=names, eps=1e-5)))
    t = {"t": torch.randn(vocab, tw, device=DEV), "g": torch.randn(dim, width, device=DEV) * 0.3,
         "p": torch.randn(width, dim, device=DEV), "n": 1 + 0.1 * torch.randn(width, device=DEV)}
    t = {k: v.to(dtype) for k, v in t.items()}
    side.bind(dict(t), rt)
    toks = [3, 49, 0, 17, 3]
    _, step = make_step([], [toks], dtype)
    x = torch.randn(5, width, device=DEV)
    pending = torch.randn(2, 5, width, device=DEV)
    x0 = x.double().cpu() + pending.double().cpu().sum(0)
    x_new, left = side.forward(rt, step, x, pending)
    assert left is None
    w = {"side.embed": t["t"].double().cpu(), "s.gate": t["g"].double().cpu(), "s.proj": t["p"].double().cpu(),
         "s.norm": t["n"].double().cpu()}
    close(x_new, x0 + P.token_side(x0, toks, 2, dim, w, "s.", 1e-5), tol)
    ffn = build_part("feed_forward", PartSpec("activated", dict(width=width, inner=88, names={"up": "u", "down": "d", "act": "a"})))
    f = {"u": (torch.randn(88, width, device=DEV) * 0.4).to(dtype), "d": (torch.randn(width, 88, device=DEV) * 0.2).to(dtype),
         "a": torch.tensor([0.4, -0.2], device=DEV).to(dtype)}
    ffn.bind(dict(f), rt)
    h = torch.randn(9, width, device=DEV).to(dtype)
    out = ffn.forward(rt, None, h)
    out = out.sum(0) if out.dim() == 3 else out
    close(out, P.dense_ffn(h.double().cpu(), {"m.up": f["u"].double().cpu(), "m.down": f["d"].double().cpu(),
                                              "m.act": f["a"].double().cpu()}, "m."), tol)
