"""The layered decoder (Nifunex) on the GPU against the plain numpy restatement in oracle/nifunex.py.

Small random configurations of the tests' own (never a shipped model's sizes); the product runs through the C ABI
(models.NifunexWithConfig / DeviceCache.forward_ragged), the oracle token by token in float64.  Two precisions: "f32" (every
product and the cache in 32-bit) against the exact oracle; "bf16" (the serving precision: tensor-core GEMMs over hi | lo activation
halves, bf16 latent cache) against the oracle that rounds what it caches to bf16.  What is left between the two in that mode is
the occasional cached element that lands on the other side of a bf16 rounding boundary (f32 against f64 arithmetic: one element
moves by 2^-8 of its value and the logits near it by ~1e-3), hence the wider bar there.
"""
import numpy as np
import pytest

from fastllm_b200 import models
from fastllm_b200._lib import FastllmError
from oracle import nifunex as O

pytestmark = pytest.mark.gpu

TOL = {"f32": 4e-5, "bf16": 1e-2}


# ---- configurations ---------------------------------------------------------------------------------------------------------
def gla(heads=2, dim=8, vdim=8, tau=8.0, rank=4, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}


def lat(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, window=None, scale=None, rot_dims=None, base=10000.0, yarn=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
         "rot": {"base": base, "dims": rot_dims if rot_dims is not None else rot_dim}}
    if yarn:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff=24, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff=16, experts=4, top=2, limit=1.0, shared=(24, 0.75)):
    c = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        c["shared"] = {"ff": shared[0], "limit": shared[1]}
    return c


def config(layers, vocab=48, width=32, eps=1e-5):
    return {"architecture": "Nifunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def hybrid_cfg(window=9, **kw):
    """every mechanism at once: recurrent + windowed latent attention + shared cache + dense + MoE"""
    return config([gla(mlp=dense()), lat(window=window, yarn=(4.0, 16, 8.0, 1.0), mlp=moe()), gla(heads=3, dim=4, vdim=12, tau=3.0, mlp=moe(shared=None, top=1)),
                   lat(window=window, yarn=(4.0, 16, 8.0, 1.0), kv_from=1, mlp=moe())], **kw)


# ---- helpers ----------------------------------------------------------------------------------------------------------------
def to_bits(a):
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


_built = {}


def build(cfg, seed=0, dtype="f32", tweak=None):
    """-> (oracle, product adapter); weights are bf16-representable, handed over as bf16 bit patterns"""
    key = (repr(cfg), seed, dtype, tweak.__name__ if tweak else None)
    if key not in _built:
        w = O.random_weights(cfg, seed)
        if tweak:
            tweak(w)
        model, _ = models.NifunexWithConfig.initialize_model(cfg, {k: to_bits(v) for k, v in w.items()}, dtype)
        _built[key] = (O.Nifunex(cfg, w, cache_round=O.bf16_round if dtype == "bf16" else None), model)
    return _built[key]


def relerr(got, ref, allow=0.0):
    """worst position's error: rms over the vocabulary of the logits' difference (means taken off) relative to the rms of the
    logits.  allow: share of positions left out, worst first (long serving-precision runs only: a 1e-3 change upstream of a random
    router can flip a near-tied expert pick; the exact mode never needs it)."""
    d = np.asarray(got, dtype=np.float64) - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    e = np.sort(np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1)))
    return float(e[len(e) - 1 - int(allow * len(e))])


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def all_places(toks):
    return [list(range(len(toks)))]


def run_whole(model, toks, slot=0, cache=None):
    cache = cache or model.new_device_cache(max_batch=4, max_seq=max(64, len(toks)))
    return cache.forward_ragged([slot], [toks], all_places(toks))


def run_cut(model, toks, cuts, slot=0, cache=None):
    """feed the tokens in portions of the given sizes (the rest one by one) and collect every position's logits"""
    cache = cache or model.new_device_cache(max_batch=4, max_seq=max(64, len(toks)))
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = min(sizes.pop(0) if sizes else 1, len(toks) - at)
        out.append(cache.forward_ragged([slot], [toks[at:at + n]], [list(range(n))]))
        at += n
    return np.concatenate(out)


# ---- each mechanism alone ---------------------------------------------------------------------------------------------------
MECHANISMS = {
    "gla": config([gla()]),
    "gla_wide_value": config([gla(heads=3, dim=12, vdim=40, tau=2.5, rank=5)], width=40),
    "latent": config([lat()]),
    "latent_window_yarn": config([lat(window=7, yarn=(8.0, 12, 4.0, 0.5), rot_dim=8, base=500.0)]),
    "latent_partial_rotation": config([lat(rot_dim=8, rot_dims=4, dim=4, vdim=12, kv_rank=20, heads=3)]),
    "latent_shared_cache": config([lat(window=5), lat(window=11, kv_from=0, heads=4, dim=4, vdim=4)]),
    "dense_ff": config([gla(mlp=dense(ff=40, limit=0.4))]),
    "moe_shared": config([gla(mlp=moe(experts=5, top=3, ff=12))]),
    "moe_top1_no_shared": config([lat(mlp=moe(experts=3, top=1, shared=None))]),
    "moe_one_expert": config([gla(mlp=moe(experts=1, top=1, shared=(8, 2.0)))]),
    "one_head": config([gla(heads=1, dim=16, vdim=16), lat(heads=1, dim=16, rot_dim=2, vdim=8, kv_rank=8)]),
}


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_alone(name, dtype):
    cfg = MECHANISMS[name]
    oracle, model = build(cfg, seed=3, dtype=dtype)
    toks = tokens(cfg, 37)
    assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL[dtype]


def test_odd_sizes_every_mechanism():
    """sizes that are no multiple of 4 / 8 / 32 anywhere, more than 32 value columns, 70 tokens across a page border"""
    cfg = config([gla(heads=3, dim=10, vdim=34, rank=3, mlp=moe(ff=10, experts=5, top=2, shared=(14, 1.0))),
                  lat(heads=5, dim=6, rot_dim=6, rot_dims=2, vdim=10, kv_rank=36, window=66, mlp=dense(ff=22)),
                  lat(heads=2, dim=18, rot_dim=6, rot_dims=2, vdim=6, kv_rank=36, window=3, kv_from=1, mlp=None)], vocab=37, width=50)
    oracle, model = build(cfg, seed=5)
    toks = tokens(cfg, 70)
    assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]


def tc_cfg():
    """widths in whole 64-column blocks: in the serving precision the projections run on the tensor-core GEMM (hi | lo activation
    halves), beside shapes that stay on the exact kernel (the 40-wide shared expert's down projection)"""
    return config([gla(heads=4, dim=16, vdim=16, rank=8, mlp=dense(ff=64)),
                   lat(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=40, mlp=moe(ff=64, experts=4, top=2, shared=(64, 1.0))),
                   gla(heads=2, dim=32, vdim=64, rank=8, mlp=moe(ff=32, experts=3, top=1, shared=(40, 1.0))),
                   lat(heads=8, dim=8, rot_dim=8, vdim=8, kv_rank=32, window=25, kv_from=1, mlp=dense(ff=128))], vocab=96, width=128)


def tc_cfg_partial_tiles():
    """192-wide: three 64-column k blocks, weight matrices that end inside a 128-row tile (grouped experts of 384 and 192 rows),
    five experts of which three are picked"""
    return config([lat(heads=3, dim=48, rot_dim=16, vdim=64, kv_rank=64, window=70, mlp=moe(ff=192, experts=5, top=3, shared=(128, 1.0))),
                   gla(heads=3, dim=64, vdim=64, rank=8, mlp=moe(ff=64, experts=2, top=2, shared=None)),
                   lat(heads=6, dim=24, rot_dim=16, vdim=32, kv_rank=64, kv_from=0, mlp=dense(ff=320))], vocab=200, width=192)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("make", [tc_cfg, tc_cfg_partial_tiles])
def test_tensor_core_projections(make, dtype):
    """1 row, a few rows, up to 128 rows (weights as the 128-row operand, split-K) and more (tokens as rows) through the same layers"""
    cfg = make()
    oracle, model = build(cfg, seed=21, dtype=dtype)
    toks = tokens(cfg, 333, seed=9)
    ref = oracle.run(toks)
    allow = 0.02 if dtype == "bf16" else 0.0
    assert relerr(run_whole(model, toks, cache=model.new_device_cache(4, 384)), ref, allow) < TOL[dtype]
    assert relerr(run_cut(model, toks, [5, 128, 129, 2, 60], cache=model.new_device_cache(4, 384)), ref, allow) < TOL[dtype]


# ---- schedules: whole prompt, token by token, portions, batches ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_prefill_equals_token_by_token(dtype):
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=7, dtype=dtype)
    toks = tokens(cfg, 90)
    ref = oracle.run(toks)
    whole, single = run_whole(model, toks), run_cut(model, toks, [])
    assert relerr(whole, ref) < TOL[dtype] and relerr(single, ref) < TOL[dtype]
    assert relerr(single, np.asarray(whole, dtype=np.float64)) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 2], [5, 64, 2, 17], [63, 2, 64], [1, 66, 2, 2, 2, 40]])
def test_portions(cuts):
    """a prompt cut into portions (down to two tokens, across page and window borders), the rest decoded one by one"""
    cfg = hybrid_cfg(window=33)
    oracle, model = build(cfg, seed=8)
    toks = tokens(cfg, 150, seed=4)
    assert relerr(run_cut(model, toks, cuts), oracle.run(toks)) < TOL["f32"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mixed_batch_equals_each_alone(dtype):
    """three requests of unequal length advance together: portions of one beside single tokens of another"""
    cfg = hybrid_cfg(window=20)
    oracle, model = build(cfg, seed=9, dtype=dtype)
    reqs = [tokens(cfg, n, seed=s) for n, s in ((75, 1), (9, 2), (40, 3))]
    cache = model.new_device_cache(max_batch=4, max_seq=128, pool_tokens=4 * 64)
    plan = [[(0, 3), (1, 1)], [(0, 30), (1, 1), (2, 2)], [(2, 38), (1, 7), (0, 1)], [(0, 41)]]
    at, got = [0, 0, 0], [[], [], []]
    slot = {0: 2, 1: 0, 2: 3}
    for step in plan:
        parts = [reqs[r][at[r]:at[r] + n] for r, n in step]
        lg = cache.forward_ragged([slot[r] for r, _ in step], parts, [list(range(len(p))) for p in parts])
        row = 0
        for (r, n), p in zip(step, parts):
            got[r].append(lg[row:row + len(p)])
            row += len(p)
            at[r] += len(p)
    for r in range(3):
        assert at[r] == len(reqs[r])
        alone = run_whole(model, reqs[r])
        together = np.concatenate(got[r])
        assert relerr(together, oracle.run(reqs[r])) < TOL[dtype]
        assert relerr(together, np.asarray(alone, dtype=np.float64)) < TOL[dtype]


def test_pages_and_slots_reused():
    """a pool of three pages and two slots serves five requests one after another and two at a time; what a finished request left
    in its pages and its state slot must not leak into the next one"""
    cfg = hybrid_cfg(window=70)
    oracle, model = build(cfg, seed=10)
    cache = model.new_device_cache(max_batch=2, max_seq=192, pool_tokens=192)
    assert cache.pool_stats() == (3, 3)
    for i, n in enumerate((130, 100, 64, 65, 3)):
        toks = tokens(cfg, n, seed=20 + i)
        slot = i % 2
        assert relerr(run_whole(model, toks, slot=slot, cache=cache), oracle.run(toks)) < TOL["f32"]
        assert cache.slot_len(slot) == n and cache.pool_stats()[1] == 3 - (n + 63) // 64
        cache.slot_reset(slot)
        assert cache.pool_stats() == (3, 3)
    a, b = tokens(cfg, 100, seed=31), tokens(cfg, 60, seed=32)
    lg = cache.forward_ragged([1, 0], [a, b], [list(range(100)), list(range(60))])
    assert cache.pool_stats()[1] == 0
    assert relerr(lg[:100], oracle.run(a)) < TOL["f32"] and relerr(lg[100:], oracle.run(b)) < TOL["f32"]
    with pytest.raises(FastllmError):          # b would need a second page: the pool is empty, nothing is changed
        cache.forward_ragged([0], [tokens(cfg, 10)], None)
    assert cache.slot_len(0) == 60
    cache.slot_reset(1)
    more = tokens(cfg, 10, seed=33)
    lg = cache.forward_ragged([0], [more], [list(range(10))])
    assert relerr(lg, oracle.run(b + more)[60:]) < TOL["f32"]


# ---- keys that must (not) be seen: made to stand out --------------------------------------------------------------------------
def _sharp(w):
    """queries and latents scaled up: the softmax is nearly one-hot, so a key that is wrongly admitted or dropped moves the logits"""
    for k in w:
        if k.endswith("mix.uk") or k.endswith("mix.dkv"):
            w[k] = O.bf16_round(w[k] * 4.0)


@pytest.mark.parametrize("window", [1, 2, 63, 64, 65, 130])
def test_window_edges_in_prompt_and_decoding(window):
    """peaky attention; windows of one key, around a page (64 tokens) and over two pages; every position of a 200-token
    sequence is checked in a whole prompt, in portions and decoded one by one"""
    cfg = config([lat(window=window, scale=2.0, mlp=None), lat(window=window + 3, scale=2.0, kv_from=0, mlp=dense())])
    oracle, model = build(cfg, seed=11, tweak=_sharp)
    toks = tokens(cfg, 200, seed=5)
    ref = oracle.run(toks)
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [window + 1, 2, 61]), ref) < TOL["f32"]


def test_window_one_off_would_show():
    """the oracle itself, with the window one key too long or too short, is far outside the bar: the test above has teeth"""
    cfg = config([lat(window=9, scale=2.0)])
    w = O.random_weights(cfg, 11)
    _sharp(w)
    toks = tokens(cfg, 60, seed=5)
    ref = O.Nifunex(cfg, w).run(toks)
    for wrong in (8, 10):
        bad = O.Nifunex(config([lat(window=wrong, scale=2.0)]), w).run(toks)
        assert relerr(bad, ref) > 100 * TOL["f32"]


def _long_memory(w):
    """decay bias high: the recurrent state forgets slowly, tokens hundreds of positions back still count"""
    for k in w:
        if k.endswith("a2.b"):
            w[k] = O.bf16_round(np.full_like(w[k], 6.0))


def test_far_tokens_reach_through_the_state():
    cfg = config([gla(tau=32.0, mlp=None), gla(heads=1, dim=24, vdim=8, tau=64.0, mlp=dense())])
    oracle, model = build(cfg, seed=12, tweak=_long_memory)
    toks = tokens(cfg, 400, seed=6)
    ref = oracle.run(toks)
    # the first token matters at the end: changing it alone moves the last logits well beyond the bar
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert relerr(oracle.run(other)[-1:], ref[-1:]) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [2, 300, 2]), ref) < TOL["f32"]


def test_first_tokens():
    cfg = hybrid_cfg(window=2)
    oracle, model = build(cfg, seed=13)
    for n in (1, 2, 3):
        toks = tokens(cfg, n, seed=n)
        assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]
        assert relerr(run_cut(model, toks, []), oracle.run(toks)) < TOL["f32"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_long_decoding(dtype):
    cfg = hybrid_cfg(window=50)
    oracle, model = build(cfg, seed=14, dtype=dtype)
    toks = tokens(cfg, 330, seed=7)
    assert relerr(run_cut(model, toks, [10]), oracle.run(toks), 0.02 if dtype == "bf16" else 0.0) < TOL[dtype]


# ---- the framework's own entry points -------------------------------------------------------------------------------------------
def oracle_greedy(oracle, prompt, n):
    st = oracle.new_state()
    logits = oracle.run(prompt, st)[-1]
    out = []
    for _ in range(n):
        tok = int(np.flatnonzero(logits == logits.max())[-1])       # last index among equal maxima, as the sampler does
        out.append(tok)
        logits = oracle.step(tok, st)
    return out


def test_greedy_generation_through_model_and_batcher():
    cfg = hybrid_cfg(window=12)
    oracle, model = build(cfg, seed=15)
    prompts = [tokens(cfg, n, seed=40 + n) for n in (5, 70, 23, 9, 31)]
    want = [oracle_greedy(oracle, p, 12) for p in prompts]
    # Model.generate: prompt in one forward, then token by token (the reference's loop)
    assert models.Model(model, None, eos_token_id=None).generate(prompts[0], 12) == want[0]
    # continuous batching: prompts alone, decode steps shared
    assert models.ContinuousBatcher(model, max_batch=3, eos_token_id=None).generate(prompts, 12) == want
    # mixed steps: prompt portions of 16 tokens beside the decode tokens of the others, slots reused by the waiting requests
    b = models.ContinuousBatcher(model, max_batch=2, eos_token_id=None, prefill_chunk=16)
    assert b.generate(prompts, 12) == want
    assert b.cache.pool_stats()[0] == b.cache.pool_stats()[1]


def test_uniform_entry_points_and_errors():
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=16)
    toks = tokens(cfg, 20)
    cache = model.new_device_cache(max_batch=2, max_seq=64)
    ref = oracle.run(toks)
    both = cache.forward(np.asarray([toks[:12], toks[:12]], dtype=np.uint32), 0)          # fl_forward: [b, t], last-position logits
    assert relerr(both, np.stack([ref[11], ref[11]])) < TOL["f32"]
    nxt = cache.forward_slots([1], np.asarray([toks[12:]], dtype=np.uint32), [12])      # fl_forward_slots
    assert relerr(nxt, ref[19:20]) < TOL["f32"]
    with pytest.raises(FastllmError):
        cache.forward(np.asarray([[1]], dtype=np.uint32), 5)                             # position differs from what the slot holds
    with pytest.raises(FastllmError):
        cache.forward_ragged([0, 0], [[1], [2]], None)                                   # a slot twice in one step
    with pytest.raises(FastllmError):
        cache.forward_ragged([0], [[cfg["vocab"]]], None)                                # token id out of range
    bad = config([lat(), lat(kv_from=0, kv_rank=8)])
    with pytest.raises(FastllmError):
        models.NifunexWithConfig.initialize_model(bad, {k: to_bits(v) for k, v in O.random_weights(bad).items()}, "f32")
    missing = {k: to_bits(v) for k, v in O.random_weights(cfg).items() if k != "l1.mix.uk"}
    with pytest.raises(FastllmError):
        models.NifunexWithConfig.initialize_model(cfg, missing, "f32")


def test_checkpoint_folder_through_the_registry(tmp_path):
    """config.json + model.safetensors -> the registry picks the class; the trace runner's own code path"""
    import json
    from fastllm_b200 import safetensors_io
    cfg = hybrid_cfg()
    w = O.random_weights(cfg, 17)
    file_cfg = json.loads(json.dumps(cfg))
    for l in file_cfg["layers"]:
        l["mixer"].pop("decay_rank", None)      # a checkpoint does not spell it out: it is the shape of the a1 tensor
    (tmp_path / "config.json").write_text(json.dumps(file_cfg))
    safetensors_io.write_safetensors(str(tmp_path / "model.safetensors"), {k: to_bits(v) for k, v in w.items()})
    model, _ = models.load_model(str(tmp_path), "f32")
    assert isinstance(model, models.NifunexWithConfig)
    toks = tokens(cfg, 30)
    assert relerr(run_whole(model, toks), O.Nifunex(cfg, w).run(toks)) < TOL["f32"]


def test_trace_runner_end_to_end(tmp_path):
    """bin/trace_run as a process: a checkpoint folder, steps on standard input (portions beside single tokens, a request that
    sits out a step, one that wants nothing, a fifth request that takes over a finished one's slot and pages), logits files out"""
    import json
    import os
    import subprocess
    from fastllm_b200 import safetensors_io
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = hybrid_cfg(window=30)
    w = O.random_weights(cfg, 23)
    file_cfg = json.loads(json.dumps(cfg))
    for l in file_cfg["layers"]:
        l["mixer"].pop("decay_rank", None)
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(file_cfg))
    safetensors_io.write_safetensors(str(model_dir / "model.safetensors"), {k: to_bits(v) for k, v in w.items()})
    reqs = {name: tokens(cfg, n, seed=50 + i) for i, (name, n) in enumerate((("a", 70), ("b", 5), ("c", 33), ("d", 64), ("e", 40)))}
    refs = {"float32": {k: O.Nifunex(cfg, w).run(v) for k, v in reqs.items()},
            "bfloat16": {k: O.Nifunex(cfg, w, cache_round=O.bf16_round).run(v) for k, v in reqs.items()}}
    plan = [[("a", 3, [0, 2]), ("b", 1, [0])],
            [("a", 60, [59]), ("c", 33, []), ("d", 2, [1])],
            [("b", 4, [0, 3]), ("d", 62, [0, 61])],                       # a sits this step out; b, c and d end here
            [("a", 1, [0]), ("e", 40, [39])],                             # e arrives after three requests left
            [("a", 6, [0, 5])]]
    at = {k: 0 for k in reqs}
    lines, places = [], {}
    for n, step in enumerate(plan):
        entries, rows, end = [], [], []
        for rid, cnt, want in step:
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + cnt], "want": want})
            rows += [(rid, at[rid] + p) for p in want]
            at[rid] += cnt
            if at[rid] == len(reqs[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
        places[n] = rows
    assert all(at[k] == len(reqs[k]) for k in reqs)
    for dtype, tol in (("float32", TOL["f32"]), ("bfloat16", TOL["bf16"])):
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "256"],
                           input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == ["done %d" % n for n in range(len(plan))]
        for n, rows in places.items():
            want = np.stack([refs[dtype][rid][p] for rid, p in rows])
            f = out_dir / ("%d.f32" % n)
            got = np.fromfile(f, dtype="<f4").reshape(-1, cfg["vocab"])
            assert got.shape == want.shape and relerr(got, want) < tol
            f.unlink()
