"""Tonanex in the engine against the plain implementation (tests/plain_tonanex.py): every mechanism alone and
the layers stacked, under every way of cutting the work, with pages and slots used again, and through the
generation loop.  The configurations are made here; weights are random, then sharpened so that a key at a
window's edge, a distance penalty, an expert's clamp or the logits' cap shows in the result."""
import json
import os

import numpy as np
import pytest
import torch
from helpers import TOL, cut_bulk_tail, cut_portions, cut_whole, note_error, random_tokens, replay

import plain_tonanex as P

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def attn(heads=4, kv_heads=2, dim=16, vdim=24, window=24, mlp="dense", **more):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if mlp == "dense":
        mlp = {"kind": "dense", "ff": 96}
    return dict({"type": "attention", "mixer": m, "mlp": mlp}, **more)


def moe(experts=6, top=2, ff=24, limit=2.0, shared=40, shared_limit=1.5):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit}
    return m


def config(layers, width=64, vocab=200, eps=1e-6, softcap=6.0):
    cfg = {"architecture": "Tonanex", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


CONFIGS = {
    # the mixer alone (with a dense feed-forward), and the routed feed-forward behind an attention without a window
    "attention": config([attn()]),
    "experts": config([attn(window=None, mlp=moe())]),
    # stacked: borrowed weights (also of the first layer, and a borrower of a borrower), a layer without a
    # feed-forward, windows of several lengths and none, one expert of three, no shared expert
    "stack": config([attn(), attn(window=None, mlp=moe()), attn(window=None, mlp=moe(), weights_of=1),
                     attn(heads=2, kv_heads=2, dim=8, vdim=8, window=7, mlp=None),
                     attn(heads=6, kv_heads=1, dim=16, vdim=16, window=33, mlp=moe(experts=3, top=1, ff=40, shared=0)),
                     attn(window=None, mlp=moe(), weights_of=2), attn(weights_of=0)]),
    # sizes that the tensor-core forms of the attention take (keys a multiple of 16, values of 64 or 128), windows
    # that end inside and outside a tile of keys
    "wide": config([attn(heads=4, kv_heads=2, dim=32, vdim=64, window=40, mlp=moe(experts=8, top=2, ff=32, shared=64)),
                    attn(heads=4, kv_heads=1, dim=64, vdim=128, window=150),
                    attn(heads=8, kv_heads=8, dim=16, vdim=64, window=None, mlp=moe(experts=4, top=4, ff=16, shared=16))],
                   width=128, vocab=260, softcap=9.0),
    # heads of 128 for keys and values: prompts and portions run the tensor-memory kernel, which changes a row of
    # scores in registers; decode steps the mma.sync form
    "heads128": config([attn(heads=4, kv_heads=2, dim=128, vdim=128, window=100),
                        attn(heads=2, kv_heads=2, dim=128, vdim=128, window=None, mlp=moe(experts=4, top=2, ff=32, shared=32))],
                       width=128, vocab=210, softcap=8.0),
    # sizes that are 1, odd or no multiple of 8; a window of one token, a window longer than any request;
    # all experts chosen, one expert of two; no cap on the logits
    "odd": config([attn(heads=3, kv_heads=1, dim=24, vdim=8, window=1, mlp=moe(experts=3, top=3, ff=20, shared=12, limit=1.0)),
                   attn(heads=2, kv_heads=2, dim=8, vdim=8, window=5000, mlp=moe(experts=2, top=1, ff=9, shared=0)),
                   attn(heads=1, kv_heads=1, dim=40, vdim=33, window=2, mlp={"kind": "dense", "ff": 52})],
                  width=36, vocab=131, eps=1e-5, softcap=None),
}


def sharpen(tensors, cfg, seed):
    """Random N(0, 0.02) matrices hide faults: a router whose logits all lie within 0.2 of its bias always takes
    the same experts, gates of 0.1 never reach an expert's limit, logits of 0.2 never feel the cap, a mixer whose
    values and output weights are small adds next to nothing to the stream, and norm-like numbers near 1 make every
    head's temperature and penalty alike.  The router, the values, the output and feed-forward weights and the
    embedding are scaled up; temperatures, penalties and the router's bias are spread out."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    uni = lambda n, lo, hi: lo + (hi - lo) * torch.rand(n, generator=g)
    scaled = lambda t, f: (t.float() * f).to(torch.bfloat16)
    tensors["embed"] = scaled(tensors["embed"], 25.0)
    for name in list(tensors):
        if name.endswith((".mix.temp",)):
            tensors[name] = uni(tensors[name].shape[0], 0.7, 2.5)
        elif name.endswith(".mix.r1"):
            tensors[name] = uni(tensors[name].shape[0], 0.5, 2.5)
        elif name.endswith(".mix.r2"):
            tensors[name] = uni(tensors[name].shape[0], 0.05, 2.0)
        elif name.endswith(".mix.g"):
            tensors[name] = scaled(tensors[name], 20.0)
        elif name.endswith((".mix.v", ".mix.o")):           # so that what the mixer adds to the stream is as large as the stream
            tensors[name] = scaled(tensors[name], 4.0)
        elif name.endswith((".mlp.gate", ".mlp.up")):
            tensors[name] = scaled(tensors[name], 6.0)
        elif name.endswith(".mlp.down"):
            tensors[name] = scaled(tensors[name], 3.0)
        elif name.endswith(".mlp.router"):
            tensors[name] = scaled(tensors[name], 10.0)
        elif name.endswith(".mlp.router.b"):
            tensors[name] = 0.5 * rnd(tensors[name].shape[0])
        elif ".mlp.e" in name or ".mlp.shared." in name:
            tensors[name] = scaled(tensors[name], 8.0 if name.endswith((".gate", ".up")) else 3.0)
    return tensors


_folders = {}


def folder_of(name, tmp_path_factory):
    """(folder, config, weights) of a configuration, written once per session."""
    if name not in _folders:
        from safetyraise_lmengine_b200.weights.random_init import write_model_folder
        from safetyraise_lmengine_b200.weights.safetensors_io import WeightFolder, write_safetensors
        cfg = CONFIGS[name]
        out = write_model_folder(cfg, 70 + len(_folders), str(tmp_path_factory.mktemp("tonanex_" + name)))
        src = WeightFolder(out)
        tensors = sharpen({n: src.get(n).clone() for n in src.names()}, cfg, 11 + len(_folders))
        del src
        write_safetensors(os.path.join(out, "model.safetensors"), tensors)
        _folders[name] = (out, cfg, tensors)
    return _folders[name]


@pytest.fixture(scope="session", params=list(CONFIGS))
def model(request, tmp_path_factory):
    return (request.param,) + folder_of(request.param, tmp_path_factory)


_plain = {}


def plain(name, cfg, W, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = P.forward(cfg, W, tokens).numpy()
    return _plain[key]


def build(folder, dtype, num_pages=64, page_size=16, **kw):
    from safetyraise_lmengine_b200 import Engine
    kw.setdefault("max_context", 1024)
    kw.setdefault("max_batch_tokens", 512)
    return Engine.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages, max_requests=4, **kw)


def check(got, model, requests, dtype):
    name, _, cfg, W = model
    for rid, tokens in requests.items():
        ref = plain(name, cfg, W, tokens)
        rows = np.stack([got[(rid, p)] for p in range(len(tokens))])
        err = np.abs(rows.astype(np.float64) - ref).max(axis=1) / np.abs(ref).max()
        # float32: every position within the tolerance.  bfloat16: a router is a discrete choice, and rounding tips it
        # between two experts at a few positions in a hundred (measured against the float32 engine, layer by layer:
        # the stream is off by a third at such a position, right behind the routed layer, and back within half a
        # percent at the next one); the tipped position's keys and values then colour the positions that see it.
        # So one position in six may be off, the median must lie within half the tolerance, and a fault of the
        # cache, which is wrong everywhere after it, still shows.  The tolerance, set for models of two layers,
        # grows with the root of the depth.
        tol = TOL[dtype] * (max(1.0, (len(cfg["layers"]) / 2) ** 0.5) if dtype == "bfloat16" else 1.0)
        bad = np.nonzero(err > tol)[0]
        allowed = len(tokens) // 6 + 2 if dtype == "bfloat16" else 0
        assert dtype == "float32" or np.median(err) <= tol / 2, (name, rid, float(np.median(err)))
        assert bad.size <= allowed, (
            f"{name} request {rid}: first wrong position {bad[0]} of {len(tokens)} "
            f"(rel err {err[bad[0]]:.3e} > {tol:.1e}); wrong positions {bad[:20]}")
        label = dtype if dtype == "float32" else ("bfloat16, Tonanex: median over positions; the tolerance grows with the root "
                                                  "of the depth, one position in six may exceed it")
        note_error(label, float(err.max() if dtype == "float32" else np.median(err)), "tonanex " + name)


def all_pages_free(eng, n):
    return eng.cache.audit() == 0 and all(eng.cache.free_pages(g.name) == n for g in eng.cache.paged_groups)


def requests_for(cfg, lens=(1, 7, 33, 64, 100), seed=0):
    rng = np.random.default_rng(500 + seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lens)}


def test_the_sharpened_models_use_what_they_have(model):
    """The tests below mean something only if a window's edge, a choice of experts, a clamp and the cap change
    the logits by far more than the tolerances: the plain implementation with each of them taken away differs."""
    import copy
    name, _, cfg, W = model
    toks = requests_for(cfg, lens=(60,), seed=1)["r0"]
    ref = plain(name, cfg, W, toks)
    big = np.abs(ref).max()
    for i, layer in enumerate(cfg["layers"]):
        other = copy.deepcopy(cfg)
        size = (layer["mixer"].get("mask") or {}).get("size")
        if size and size < 60:
            for l in other["layers"]:
                if l["mixer"] == layer["mixer"]:
                    l["mixer"]["mask"]["size"] = size + 1
            assert np.abs(P.forward(other, W, toks).numpy() - ref).max() > 50 * TOL["float32"] * big, (i, "window")
    W2 = dict(W)
    for n in W:
        if n.endswith(".mix.r1"):
            W2[n] = W[n] * 0
    assert np.abs(P.forward(cfg, W2, toks).numpy() - ref).max() > 0.01 * big
    if cfg.get("logit_softcap"):
        assert np.abs(P.forward(dict(cfg, logit_softcap=None), W, toks).numpy() - ref).max() > 0.01 * big


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_requests_alone(model, dtype):
    eng = build(model[1], dtype)
    reqs = requests_for(model[2])
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_whole(rid, toks)))
    check(got, model, reqs, dtype)
    assert all_pages_free(eng, 64)


def test_the_stream_after_every_layer(model):
    """float32, layer by layer: the engine's model is cut off behind its first k run steps and its stream
    compared with the plain one's (a looped layer counts each time it runs)."""
    import copy
    name, folder, cfg, W = model
    toks = requests_for(cfg, lens=(40,), seed=7)["r0"]
    streams = []
    P.forward(cfg, W, toks, streams)
    from safetyraise_lmengine_b200 import StepEntry
    eng = build(folder, "float32")
    order = eng.model.spec.run_order
    for k in range(1, len(order) + 1):
        object.__setattr__(eng.model.spec, "run_order", order[:k])
        slot = eng.open_request()
        eng.step([StepEntry(slot, toks, [])])
        x = eng.workspace.get("residual", len(toks), cfg["width"], torch.float32).cpu().double()
        pend_name = "moe.out" if cfg["layers"][k - 1].get("mlp", None) and cfg["layers"][k - 1]["mlp"]["kind"] == "moe" else \
            ("ffn.down" if cfg["layers"][k - 1].get("mlp") else "dist_attn.o")
        x = x + eng.workspace.get(pend_name, len(toks), cfg["width"], torch.float32).cpu().double()   # the last sublayer's result is still pending
        eng.close_request(slot)
        want = streams[k - 1]
        assert (x - want).abs().max() <= 2e-5 * want.abs().max(), (name, k, float((x - want).abs().max()))
    object.__setattr__(eng.model.spec, "run_order", order)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token(model, dtype):
    """Most of a prompt in one step, the rest decoded one by one (replayed from CUDA graphs): the window passes
    over decoded tokens, pages behind it are given back."""
    eng = build(model[1], dtype)
    reqs = {k: v for k, v in requests_for(model[2]).items() if len(v) >= 33}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_bulk_tail(rid, toks, 32)))
    check(got, model, reqs, dtype)
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_token_at_a_time_from_the_start(model, dtype):
    eng = build(model[1], dtype)
    reqs = requests_for(model[2], lens=(45,), seed=2)
    got = replay(eng, cut_bulk_tail("r0", reqs["r0"], 44))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [4, 16])
def test_portions_of_changing_size(model, dtype, page_size):
    """Portions down to two tokens, cut in the middle of pages, of key blocks and of windows."""
    eng = build(model[1], dtype, num_pages=40, page_size=page_size)
    reqs = {k: v for k, v in requests_for(model[2]).items() if len(v) >= 2}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_portions(rid, toks)))
        got.update({(rid + "b", p): row for (_, p), row in
                    replay(eng, cut_portions(rid, toks, sizes=(2, 2, 3, 2, 29, 2, 2, 35, 2))).items()})
    check(got, model, reqs, dtype)
    check(got, model, {rid + "b": toks for rid, toks in reqs.items()}, dtype)
    assert eng.cache.audit() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_and_reuse_of_pages_and_slots(model, dtype):
    """Up to four live requests: portions of some beside single tokens of others; requests end and new
    ones take their slots and pages (few pages, so the page freed last is used next)."""
    cfg = model[2]
    rng = np.random.default_rng(9)
    lens = {"a": 70, "b": 23, "c": 41, "d": 9, "e": 55, "f": 30, "g": 12}
    reqs = {k: random_tokens(rng, n, cfg["vocab"]) for k, n in lens.items()}
    fed = {k: 0 for k in reqs}

    def take(rid, n):
        lo = fed[rid]
        hi = min(len(reqs[rid]), lo + n)
        fed[rid] = hi
        return (rid, reqs[rid][lo:hi], list(range(hi - lo)))

    steps = [
        {"entries": [take("a", 20), take("b", 5)]},
        {"entries": [take("a", 1), take("b", 18), take("c", 2), take("d", 8)], "end": ["b"]},
        {"entries": [take("a", 1), take("c", 30), take("d", 1), take("e", 7)], "end": ["d"]},
        {"entries": [take("f", 30), take("a", 48), take("c", 1), take("e", 2)], "end": ["a", "f"]},
        {"entries": [take("g", 3), take("c", 8), take("e", 1)], "end": ["c"]},
        {"entries": [take("e", 45), take("g", 1)]},
        {"entries": [take("g", 8)], "end": ["e", "g"]},
    ]
    assert all(fed[k] == len(reqs[k]) for k in reqs)
    eng = build(model[1], dtype, num_pages=24, page_size=8)
    got = replay(eng, steps)
    check(got, model, reqs, dtype)
    opened, reused = eng.cache.reuse_counts()
    assert reused > 0 and all_pages_free(eng, 24)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """300 tokens, the last 260 one by one: pages fill, windows move on and their pages turn over."""
    reqs = requests_for(model[2], lens=(300,), seed=3)
    eng = build(model[1], dtype, num_pages=24, page_size=16)
    got = replay(eng, cut_bulk_tail("r0", reqs["r0"], 260))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions(model, dtype):
    """700 tokens in portions of 48: the later portions stand behind hundreds of cached keys, most of them
    behind the window and their pages gone."""
    if model[0] not in ("wide", "attention", "stack", "heads128"):
        pytest.skip("one configuration of each attention kernel is enough")
    reqs = requests_for(model[2], lens=(700,), seed=6)
    eng = build(model[1], dtype, num_pages=48, page_size=16)
    got = replay(eng, cut_portions("r0", reqs["r0"], sizes=(48,)))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_one_step(model, dtype):
    """900 tokens at once, beside a short request: steps of many tokens run the experts' products in whole tiles on
    the tensor-memory kernel (bfloat16), and the attention's row tiles stand behind hundreds of keys of their own step."""
    reqs = requests_for(model[2], lens=(900, 40), seed=8)
    eng = build(model[1], dtype, num_pages=72, page_size=16, max_batch_tokens=1024)
    got = replay(eng, [{"entries": [("r1", reqs["r1"], list(range(40))), ("r0", reqs["r0"], list(range(900)))],
                        "end": ["r0", "r1"]}])
    check(got, model, reqs, dtype)
    assert all_pages_free(eng, 72)


def test_cuttings_agree_bit_for_bit_in_float32(model):
    """In float32 no sum depends on the cutting or on the batch: the logits of a position are the same bits."""
    reqs = requests_for(model[2], lens=(90, 37), seed=4)
    toks, other = reqs["r0"], reqs["r1"]
    eng = build(model[1], "float32")
    whole = replay(eng, cut_whole("r0", toks))
    tail = replay(eng, cut_bulk_tail("r0", toks, 40))
    parts = replay(eng, cut_portions("r0", toks))
    beside = replay(eng, [{"entries": [("x", other[:30], []), ("r0", toks[:50], list(range(50)))]},
                          {"entries": [("r0", toks[50:], list(range(40))), ("x", other[30:31], [])]}])
    for p in range(len(toks)):
        assert np.array_equal(whole[("r0", p)], tail[("r0", p)]), p
        assert np.array_equal(whole[("r0", p)], parts[("r0", p)]), p
        assert np.array_equal(whole[("r0", p)], beside[("r0", p)]), p


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_refused_step_leaves_nothing_behind(model, dtype):
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import ShapeError
    reqs = requests_for(model[2], lens=(30,), seed=5)
    toks = reqs["r0"]
    eng = build(model[1], dtype)
    slot = eng.open_request()
    rows = [eng.step([StepEntry(slot, toks[:11], list(range(11)))]).cpu().numpy().copy()]
    with pytest.raises(ShapeError):
        eng.step([StepEntry(slot, [model[2]["vocab"] + 5, 1], [0])])
    rows.append(eng.step([StepEntry(slot, toks[11:], list(range(19)))]).cpu().numpy().copy())
    check({("r0", p): r for p, r in enumerate(np.concatenate(rows))}, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(model, dtype):
    from safetyraise_lmengine_b200 import LLM, SamplingParams
    name, folder, cfg, W = model
    rng = np.random.default_rng(21)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 19, 11, 3, 26)]        # more requests than slots
    llm = LLM.from_folder(folder, dtype=dtype, page_size=4, num_pages=64, max_active=3, max_batch_tokens=48,
                          prefill_chunk=8, max_context=128, queue_capacity=8)
    llm.eos = set()
    res = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10))
    for prompt, r in zip(prompts, res):
        assert r.finish_reason == "length" and len(r.tokens) == 10
        toks = list(prompt) + list(r.tokens)
        ref = P.forward(cfg, W, toks[:-1]).numpy()
        for i, tok in enumerate(r.tokens):
            row = ref[len(prompt) - 1 + i]
            if dtype == "float32":
                assert tok == int(np.argmax(row)) or row[tok] >= row.max() - 1e-5 * np.abs(row).max(), (i, tok)
            else:
                assert row[tok] >= row.max() - 3 * TOL[dtype] * np.abs(row).max(), (i, tok)
    assert all_pages_free(llm.engine, 64)


# ---- mechanisms alone, with inputs made so that a fault shows --------------------------------------------------

class _Ctx:
    """The fields of a step's context that the attention kernels' wrappers read."""
    def __init__(self, q_lens, kv_lens, dev):
        self.n_entries, self.max_q_len = len(q_lens), max(q_lens)
        self.cu_q = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=dev)
        self.kv_lens = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
        from safetyraise_lmengine_b200.parts import Workspace
        self.kv_bound, self.workspace = max(kv_lens), Workspace(torch.device(dev), 64)
        self.host = {"q_lens": list(q_lens), "kv_lens": list(kv_lens), "starts": [k - q for q, k in zip(q_lens, kv_lens)]}
        self.tables = {}


def _paged(keys, page_size, order, dtype, dev, first_kept=0):
    """keys [L, heads, d] -> (pool [pages, heads, page_size, d], table); pages wholly before ``first_kept``
    are not stored and their table entries are -1, as a window group leaves them."""
    L, H, d = keys.shape
    n = (L + page_size - 1) // page_size
    pool = torch.zeros(len(order), H, page_size, d, dtype=dtype, device=dev)
    table = []
    for i in range(n):
        if (i + 1) * page_size <= first_kept:
            table.append(-1)
            continue
        chunk = keys[i * page_size:(i + 1) * page_size]
        pool[order[i], :, :chunk.shape[0]] = chunk.transpose(0, 1).to(dtype)
        table.append(order[i])
    return pool, torch.tensor([table], dtype=torch.int32, device=dev)


@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv,heads,kv_heads,window", [(24, 40, 4, 2, 100), (48, 16, 3, 3, 37), (16, 16, 2, 1, 0),
                                                         (32, 64, 4, 2, 64), (64, 128, 8, 2, 129), (48, 64, 6, 1, 33),
                                                         (88, 72, 4, 4, 300), (32, 256, 2, 2, 65), (128, 128, 4, 2, 129),
                                                         (128, 128, 2, 2, 0)])
def test_attention_kernel_window_edges_penalty_and_temperature(cache_dtype, dk, dv, heads, kv_heads, window):
    """Queries aimed at one key each: just inside the window, just outside it (where a still heavier key waits),
    far back, at page borders and at position 0.  A window one token off, a lost penalty or temperature or a
    page that was given back and read all the same changes the result by far more than the tolerance."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, L, page = "cuda:0", 700, 16
    g = torch.Generator().manual_seed(dk * 100 + dv)
    q = 0.5 * torch.randn(L, heads, dk, generator=g)
    k = torch.randn(L, kv_heads, dk, generator=g)
    v = torch.randn(L, kv_heads, dv, generator=g)
    if cache_dtype == torch.bfloat16:
        k, v = k.bfloat16().float(), v.bfloat16().float()
    rep = heads // kv_heads
    aim = lambda row, col, f: q.__setitem__(row, f * k[col].repeat_interleave(rep, 0)
                                            / k[col].norm(dim=-1, keepdim=True).repeat_interleave(rep, 0))
    w = window or L
    pairs = [(L - 1, L - w), (L - 2, L - 2 - w), (L - 3, max(0, L - 3 - w + 1)), (650, 650 - min(w, 650) + 1), (651, 640), (40, 0), (600, 592)]
    for row, col in pairs:
        if col >= 0:
            aim(row, col, 6.0)
    temperature = torch.linspace(0.6, 2.2, heads)
    weight, rate = torch.linspace(0.3, 1.4, heads), torch.linspace(1.5, 0.1, heads)
    scale = 0.9
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    ref = torch.einsum("hij,jhd->ihd", P.masked_softmax(P.distance_scores(q, kk, scale, temperature, weight, rate),
                                                        P.visible(L, window or None)), vv.double())
    plain_scores = torch.einsum("hij,jhd->ihd", P.masked_softmax(P.distance_scores(q, kk, scale, None, None, None),
                                                                 P.visible(L, window or None)), vv.double())
    assert (ref - plain_scores).abs().max() > 0.05
    if window:
        off = torch.einsum("hij,jhd->ihd", P.masked_softmax(P.distance_scores(q, kk, scale, temperature, weight, rate),
                                                            P.visible(L, window + 1)), vv.double())
        assert (ref[L - 2] - off[L - 2]).abs().max() > 0.05          # the key just outside would be seen
    order = list(reversed(range(L // page + 2)))
    tol = 2e-5 if cache_dtype == torch.float32 else 2e-2
    for q_lens in ([L], [1], [2], [3], [33], [130]):             # a whole prompt, decoded tokens, portions
        n = q_lens[0]
        first_kept = max(0, L - n - w + 1) if window else 0          # what a window group still holds before this step
        k_pool, table = _paged(k, page, order, cache_dtype, dev, first_kept)
        v_pool = _paged(v, page, order, cache_dtype, dev, first_kept)[0]
        out = torch.zeros(n, heads * dv, dtype=torch.float32, device=dev)
        ops.paged_attention_general(_Ctx(q_lens, [L], dev), q[L - n:].reshape(n, -1).contiguous().to(dev), k_pool, v_pool,
                                    out, table, None, heads, kv_heads, dk, dv, scale, window,
                                    head_scale=temperature.to(dev), penalty=(weight.to(dev), rate.to(dev)))
        err = (out.cpu().double().view(n, heads, dv) - ref[L - n:]).abs().max() / ref.abs().max()
        assert err < tol, (q_lens, float(err))
        # the same with a gate per head on the way out: columns 3.. of a wider tensor of logits
        logits = 2 * torch.randn(n, heads + 5, generator=g)
        ops.paged_attention_general(_Ctx(q_lens, [L], dev), q[L - n:].reshape(n, -1).contiguous().to(dev), k_pool, v_pool,
                                    out, table, None, heads, kv_heads, dk, dv, scale, window,
                                    head_scale=temperature.to(dev), penalty=(weight.to(dev), rate.to(dev)),
                                    gate=(logits.to(dev), 3))
        gated = ref[L - n:] * torch.sigmoid(logits[:, 3:3 + heads].double())[:, :, None]
        err = (out.cpu().double().view(n, heads, dv) - gated).abs().max() / ref.abs().max()
        assert err < tol, ("gated", q_lens, float(err))
        ctx = _Ctx(q_lens, [L], dev)
        if cache_dtype == torch.bfloat16 and dk == dv and n > 4 and ops.sinks_on_tcgen05(ctx, cache_dtype, heads, kv_heads, dk, dv, page):
            # heads of 128: the tensor-memory kernel, queries in bfloat16
            out16 = torch.zeros(n, heads * dv, dtype=torch.bfloat16, device=dev)
            ops.paged_attention(ctx, q[L - n:].reshape(n, -1).contiguous().to(dev).bfloat16(), k_pool, v_pool, out16, table,
                                heads, kv_heads, dk, page, scale, window,
                                mods=(temperature.to(dev), weight.to(dev), rate.to(dev)))
            err = (out16.cpu().double().view(n, heads, dv) - ref[L - n:]).abs().max() / ref.abs().max()
            assert err < tol, ("tensor memory", q_lens, float(err))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unit_norm_and_append(dtype):
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(5)
    for T, nq, nkv, dk, dv, extra in ((7, 4, 2, 24, 40, 4), (3, 1, 1, 100, 7, 0), (40, 6, 2, 88, 72, 6)):
        proj = 3 * torch.randn(T, nq * dk + nkv * (dk + dv) + extra, generator=g)
        slots = torch.randperm(64, generator=g)[:T].to(torch.int32)
        kp = torch.zeros(4, nkv, 16, dk, dtype=dtype, device=dev)
        vp = torch.zeros(4, nkv, 16, dv, dtype=dtype, device=dev)
        q = torch.zeros(T, nq * dk, device=dev)
        ops.attention_unit_norm_append(proj.to(dev), 1e-3, q, kp, vp, slots.to(dev), nq, nkv, dk, dv)
        want_q = P.unit_rms(proj[:, :nq * dk].view(T, nq, dk), 1e-3)
        want_k = P.unit_rms(proj[:, nq * dk:(nq + nkv) * dk].view(T, nkv, dk), 1e-3)
        want_v = proj[:, (nq + nkv) * dk:(nq + nkv) * dk + nkv * dv].view(T, nkv, dv).double()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert (q.cpu().double().view(T, nq, dk) - want_q).abs().max() < 1e-5
        for t in range(T):
            page, off = int(slots[t]) // 16, int(slots[t]) % 16
            assert (kp[page, :, off].cpu().double() - want_k[t]).abs().max() < tol
            assert (vp[page, :, off].cpu().double() - want_v[t]).abs().max() < tol * 10


def test_router_choice_and_weights():
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(8)
    for T, E, top in ((9, 6, 2), (5, 3, 3), (33, 70, 8), (4, 2, 1), (3, 1, 1)):
        z, b = 2 * torch.randn(T, E, generator=g), torch.randn(E, generator=g)
        if E >= 6:
            z[0, 4] = z[0, 1] = 9.0 - b[1]          # a tie after the bias only if the biases agree: make them
            b[4] = b[1]
        choice = torch.zeros(T, top, dtype=torch.int32, device=dev)
        weight = torch.zeros(T, top, device=dev)
        ops.moe_route(z.to(dev), b.to(dev), top, choice, weight)
        val, idx = (z + b).double().topk(top, dim=-1)
        if E >= 6:
            assert choice[0, :2].tolist() == [1, 4]                   # a tie goes to the lower index
            idx[0, :2] = torch.tensor([1, 4])
        assert torch.equal(choice.cpu().long(), idx)
        assert (weight.cpu().double() - torch.softmax(val, -1)).abs().max() < 1e-6
        # the same from columns of a wider tensor, routed by the block that orders the pairs
        wide = torch.cat([torch.randn(T, 5, generator=g), z, torch.randn(T, 2, generator=g)], dim=1).to(dev)
        choice2, weight2 = torch.zeros_like(choice), torch.zeros_like(weight)
        heads = torch.zeros(2, E + 1, dtype=torch.int32, device=dev)
        por, rop = torch.zeros(T * top, dtype=torch.int32, device=dev), torch.zeros(T * top, dtype=torch.int32, device=dev)
        assert ops.moe_sort_routes(T, E)
        ops.moe_sort(choice2, E, heads[0], heads[1], por, rop, route=(wide, 5, b.to(dev), weight2))
        assert torch.equal(choice2, choice) and torch.equal(weight2, weight)
        assert heads[0].tolist() == [int((idx < e).sum()) for e in range(E + 1)]
        assert all(int(por[int(rop[i])]) == i for i in range(T * top))


@pytest.mark.parametrize("dtype,interleaved", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_grouped_products_of_the_experts(dtype, interleaved):
    """Pairs ordered by expert, both grouped products and the combination, against loops over tokens: experts that
    nobody chose, an expert with more rows than a tile, one token, sizes that are no multiple of anything; with the
    gate and up rows interleaved in blocks of eight the bfloat16 products run on tensor cores where the sizes fit."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(12)
    sizes = ((150, 5, 2, 40, 24), (1, 4, 4, 36, 9), (70, 9, 1, 64, 32), (33, 3, 3, 24, 130))
    if interleaved:
        sizes = ((150, 5, 2, 40, 24), (1, 4, 4, 72, 8), (300, 9, 1, 64, 200), (33, 3, 3, 264, 136), (70, 2, 2, 36, 16))
    for T, E, top, H, ff in sizes:
        x = torch.randn(T, H, generator=g).to(dtype)
        gu = (0.5 * torch.randn(E, 2 * ff, H, generator=g)).to(dtype)
        dn = (0.3 * torch.randn(E, H, ff, generator=g)).to(dtype)
        choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
        if E == 5:
            choice[choice == 3] = 0
            choice[:, 1] = torch.where(choice[:, 0] == 4, 1, 4)     # expert 3 unused, expert 4 in (almost) every token
        weight = torch.rand(T, top, generator=g)
        shared = torch.randn(T, H, generator=g).to(dtype)
        n = T * top
        d = lambda t: t.to(dev)
        offsets, tiles = torch.zeros(E + 1, dtype=torch.int32, device=dev), torch.zeros(E + 1, dtype=torch.int32, device=dev)
        por, rop = torch.zeros(n, dtype=torch.int32, device=dev), torch.zeros(n, dtype=torch.int32, device=dev)
        ops.moe_sort(d(choice), E, offsets, tiles, por, rop)
        assert offsets.tolist() == [int((choice < e).sum()) for e in range(E + 1)]
        assert sorted(por.tolist()) == list(range(n)) and all(int(por[int(rop[i])]) == i for i in range(n))
        y = torch.zeros(n, ff, dtype=dtype, device=dev)
        gu_dev = d(gu)
        if interleaved:        # blocks of 16 rows: 8 gate rows, then the 8 up rows of the same features
            gu_dev = torch.stack([gu_dev[:, :ff].reshape(E, ff // 8, 8, H), gu_dev[:, ff:].reshape(E, ff // 8, 8, H)],
                                 dim=2).reshape(E, 2 * ff, H).contiguous()
        ops.moe_grouped(d(x), por, top, gu_dev, y, offsets, tiles, glu=True, interleaved=interleaved, limit=1.2, alpha=1.702)
        rows = torch.zeros(n, H, device=dev)
        ops.moe_grouped(y, None, 1, d(dn), rows, offsets, tiles)
        out = torch.zeros(T, H, dtype=dtype, device=dev)
        ops.moe_combine(rows, rop, d(weight), d(shared), out)
        want = shared.double().clone()
        for t in range(T):
            for c in range(top):
                e = int(choice[t, c])
                W = {"gate": gu[e, :ff], "up": gu[e, ff:], "down": dn[e]}
                want[t] += weight[t, c].double() * P.expert(x[t:t + 1], W, "", 1.2)[0]
        err = (out.cpu().double() - want).abs().max() / want.abs().max()
        assert err < (2e-5 if dtype == torch.float32 else 2e-2), (T, E, top, float(err))


@pytest.mark.parametrize("tile", [128, 256])
def test_grouped_products_in_tiles_of_tensor_memory(tile):
    """Steps of many tokens: every expert's rows in whole tiles of 128 (one SM a tile) or 256 (a pair of SMs) of a
    gathered copy, both products on the persistent tensor-memory kernel.  An expert nobody chose, one with a single
    row, one with several tiles."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(14)
    for T, E, top, H, ff in ((700, 5, 2, 64, 48), (130, 3, 1, 136, 200), (512, 4, 4, 256, 128)):
        x = torch.randn(T, H, generator=g).bfloat16()
        gu = (0.4 * torch.randn(E, 2 * ff, H, generator=g)).bfloat16()
        dn = (0.3 * torch.randn(E, H, ff, generator=g)).bfloat16()
        choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
        if E == 5:
            choice[choice == 3] = 0
            choice[:, 1] = torch.where(choice[:, 0] == 4, 1, 4)
            choice[7, 0] = 2
            choice[choice[:, 0] == 2, 0] = 0
            choice[7, 0] = 2                                    # expert 2: one row; expert 3: none; expert 4: many tiles
        weight = torch.rand(T, top, generator=g)
        n = T * top
        n_tiles = n // tile + E
        d = lambda t: t.to(dev)
        heads = torch.zeros(2, E + 1, dtype=torch.int32, device=dev)
        got = torch.full((n_tiles,), -7, dtype=torch.int32, device=dev)
        por = torch.full((n_tiles * tile,), -7, dtype=torch.int32, device=dev)
        rop = torch.zeros(n, dtype=torch.int32, device=dev)
        ops.moe_sort(d(choice), E, heads[0], heads[1], por, rop, tile_rows=tile, group_of_tile=got)
        counts = [int((choice == e).sum()) for e in range(E)]
        assert all(int(heads[0][e]) % tile == 0 for e in range(E))
        want_groups = sum(([e] * -(-c // tile) for e, c in enumerate(counts)), [])
        assert got.tolist() == want_groups + [-1] * (n_tiles - len(want_groups))
        assert all(int(por[int(rop[i])]) == i for i in range(n)) and int((por >= 0).sum()) == n
        gu_dev = torch.stack([d(gu)[:, :ff].reshape(E, ff // 8, 8, H), d(gu)[:, ff:].reshape(E, ff // 8, 8, H)],
                             dim=2).reshape(E, 2 * ff, H).contiguous()
        xs = torch.empty(n_tiles * tile, H, dtype=torch.bfloat16, device=dev)
        ops.moe_gather_rows(d(x), por, top, xs)
        y = torch.zeros(n_tiles * tile, ff, dtype=torch.bfloat16, device=dev)
        ops.gemm_tn_tcgen05_grouped(xs, gu_dev, y, got, glu=True, limit=1.2, alpha=1.702, tile_rows=tile)
        rows = torch.zeros(n_tiles * tile, H, device=dev)
        ops.gemm_tn_tcgen05_grouped(y, d(dn), rows, got, tile_rows=tile)
        out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        ops.moe_combine(rows, rop, d(weight), None, out)
        assert ops.gemm_error_flag(torch.device(dev)) == 0
        want = torch.zeros(T, H, dtype=torch.float64)
        for t in range(T):
            for c in range(top):
                e = int(choice[t, c])
                W = {"gate": gu[e, :ff], "up": gu[e, ff:], "down": dn[e]}
                want[t] += weight[t, c].double() * P.expert(x[t:t + 1], W, "", 1.2)[0]
        err = (out.cpu().double() - want).abs().max() / want.abs().max()
        assert err < 2e-2, (T, E, top, float(err))


def test_cap_and_clamped_activation():
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(2)
    x = 30 * torch.randn(7, 333, generator=g)
    y = x.to(dev)
    ops.softcap(y, 11.0)
    assert (y.cpu().double() - P.softcap(x.double(), 11.0)).abs().max() < 1e-5
    gu = 4 * torch.randn(5, 2 * 77 + 9, generator=g)         # columns behind gate and up are not read
    out = torch.zeros(5, 77, device=dev)
    ops.clamped_glu(gu.to(dev), out, 2.5, 1.702)
    gt, up = gu[:, :77].double().clamp(max=2.5), gu[:, 77:154].double().clamp(-2.5, 2.5)
    assert (out.cpu().double() - gt * torch.sigmoid(1.702 * gt) * (up + 1)).abs().max() < 1e-5


# ---- as a user runs it: the command line and the trace replay ---------------------------------------------------

def test_command_line_and_trace_replay(tmp_path, tmp_path_factory):
    import subprocess
    import sys
    from conftest import ROOT
    folder, cfg, W = folder_of("stack", tmp_path_factory)
    env = dict(os.environ, PYTHONPATH=ROOT)
    cli = lambda *a: subprocess.run([sys.executable, "-m", "safetyraise_lmengine_b200", *a], env=env,
                                    capture_output=True, text=True, timeout=600)
    out = cli("inspect", "--model-path", folder, "--context", "64")
    assert out.returncode == 0, out.stderr
    info = json.loads(out.stdout)
    assert info["spec"]["architecture"] == "Tonanex" and len(info["cache_groups"]) >= 3
    svc, req = tmp_path / "svc.json", tmp_path / "req.json"
    svc.write_text(json.dumps({"model_path": folder, "model_name": "stack",
                               "engine": {"max_context": 128, "max_active": 2, "prefill_chunk": 4, "page_size": 4,
                                          "num_pages": 40, "dtype": "float32", "max_batch_tokens": 32}}))
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    req.write_text(json.dumps({"prompt_ids": prompt, "max_tokens": 6, "temperature": 0.0}))
    out = cli("run", "--config", str(svc), "--request", str(req))
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout)
    toks = list(prompt)
    for tok in res["tokens"]:
        row = P.forward(cfg, W, toks)[-1].numpy()
        assert row[tok] >= row.max() - 1e-5 * np.abs(row).max()
        toks.append(tok)
    assert len(res["tokens"]) == 6 and res["finish_reason"] == "length"

    rng = np.random.default_rng(2)
    a, b = random_tokens(rng, 50, cfg["vocab"]), random_tokens(rng, 40, cfg["vocab"])
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": [1]}, {"id": "b", "tokens": b[:39], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[39:], "want": [0]}, {"id": "a", "tokens": a[32:], "want": [17]}],
         "end": ["a", "b"]},
    ]
    out_dir = tmp_path / "out_float32"
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out",
                           str(out_dir), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    ra, rb = plain("stack", cfg, W, a), plain("stack", cfg, W, b)
    biggest = max(np.abs(ra).max(), np.abs(rb).max())
    for got, ref in ((read(0), ra[[0, 29]]), (read(1), ra[[31]]), (read(2), np.stack([rb[39], ra[49]]))):
        assert got.shape == ref.shape and np.abs(got - ref).max() <= TOL["float32"] * biggest


# ---- configurations drawn at random: layer order, sizes and constants that no other test chose -----------------

def random_config(seed):
    rng = np.random.default_rng(2000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = pick(40, 64, 96, 128, 160)
    layers = []
    for i in range(int(rng.integers(2, 7))):
        if layers and rng.random() < 0.3:
            j = int(rng.integers(len(layers)))
            layers.append(dict({k: v for k, v in layers[j].items() if k != "weights_of"}, weights_of=j))
            continue
        kv = pick(1, 2, 3)
        dim, vdim = pick((8, 8), (16, 40), (24, 16), (32, 64), (64, 64), (128, 128), (48, 128), (80, 56))
        kind = pick("dense", "moe", "moe", None)
        if kind == "moe":
            experts = pick(2, 3, 5, 8, 12)
            mlp = moe(experts=experts, top=int(rng.integers(1, min(experts, 4) + 1)), ff=pick(8, 16, 24, 40, 50),
                      limit=pick(0.8, 1.5, 3.0), shared=pick(0, 16, 36), shared_limit=pick(1.0, 2.5))
        else:
            mlp = {"kind": "dense", "ff": pick(32, 72, 100)} if kind else None
        layers.append(attn(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=vdim, window=pick(None, 1, 9, 16, 50, 129, 1000),
                           mlp=mlp))
    return config(layers, width=width, vocab=pick(97, 160, 301), eps=pick(1e-6, 1e-5, 1e-4), softcap=pick(None, 5.0, 30.0))


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Whatever the order of layers and the sizes: float32 within the tolerance at every position under a cutting
    with portions, decoded tokens and a second request beside it; bfloat16 by the rule of `check`."""
    from safetyraise_lmengine_b200.weights.random_init import write_model_folder
    from safetyraise_lmengine_b200.weights.safetensors_io import WeightFolder, write_safetensors
    cfg = random_config(seed)
    out = write_model_folder(cfg, 900 + seed, str(tmp_path / "m"))
    src = WeightFolder(out)
    W = sharpen({n: src.get(n).clone() for n in src.names()}, cfg, 50 + seed)
    del src
    write_safetensors(os.path.join(out, "model.safetensors"), W)
    rng = np.random.default_rng(seed)
    reqs = {"a": random_tokens(rng, 180, cfg["vocab"]), "b": random_tokens(rng, 37, cfg["vocab"])}
    a, b = reqs["a"], reqs["b"]
    steps = [{"entries": [("a", a[:61], list(range(61)))]},
             {"entries": [("b", b[:2], [0, 1]), ("a", a[61:64], [0, 1, 2])]},
             {"entries": [("a", a[64:150], list(range(86))), ("b", b[2:3], [0])]},
             {"entries": [("b", b[3:36], list(range(33))), ("a", a[150:151], [0])]}]
    steps += [{"entries": [("a", a[i:i + 1], [0])] + ([("b", b[36:], [0])] if i == 151 else [])} for i in range(151, 180)]
    model = (f"random {seed}", out, cfg, W)
    for dtype in DTYPES:
        eng = build(out, dtype, num_pages=20, page_size=16)
        check(replay(eng, steps), model, reqs, dtype)
        assert all_pages_free(eng, 20)
