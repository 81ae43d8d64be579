"""The Rofetar decoder on the GPU against the plain numpy restatement in oracle/rofetar.py.

Small random configurations of the tests' own; the product runs through the C ABI (models.RofetarWithConfig /
DeviceCache.forward_ragged), the oracle token by token in float64.  Two precisions: "f32" (every product and the cache in 32-bit)
against the exact oracle; "bf16" (the serving precision: tensor-core GEMMs over hi | lo activation halves, bf16 key / value cache)
against the oracle that rounds the keys and values it caches to bf16.
"""
import json
import os
import subprocess

import numpy as np
import pytest

from fastllm_b200 import models
from fastllm_b200._lib import FastllmError
from oracle import rofetar as O

pytestmark = pytest.mark.gpu

TOL = {"f32": 4e-5, "bf16": 1e-2}


# ---- configurations ---------------------------------------------------------------------------------------------------------
def att(heads=4, kv_heads=2, dim=8, vdim=12, rot_dims=4, base=10000.0, yarn=None, scale=None, softcap=30.0, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "softcap": softcap, "rot": {"base": base, "dims": rot_dims}}
    if yarn:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def mamba(heads=4, vdim=6, state=10, groups=2, norm_groups=1, conv=3, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv},
            "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=6, vdim=10, conv=3, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def config(layers, vocab=48, width=32, eps=1e-5):
    return {"architecture": "Rofetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def hybrid_cfg(**kw):
    """every mechanism at once: both recurrent mixers, attention with its own cache and on a shared one, with / without feed-forward"""
    return config([delta(mlp=None), att(yarn=(4.0, 16, 8.0, 1.0), mlp=dense()), mamba(mlp=dense(ff=20)), delta(heads=3, kv_heads=3, dim=4, vdim=12, conv=2),
                   att(heads=2, kv_heads=2, yarn=(4.0, 16, 8.0, 1.0), kv_from=1, mlp=dense()), mamba(heads=2, groups=1, norm_groups=2, vdim=8, state=5, conv=4)], **kw)


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
        model, _ = models.RofetarWithConfig.initialize_model(cfg, {k: to_bits(v) for k, v in w.items()}, dtype)
        _built[key] = (O.Rofetar(cfg, w, cache_round=O.bf16_round if dtype == "bf16" else None), model)
    return _built[key]


def relerr(got, ref):
    """worst position's error: rms over the vocabulary of the logits' difference (means taken off) relative to the rms of the logits"""
    d = np.asarray(got, dtype=np.float64) - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))).max())


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def run_whole(model, toks, slot=0, cache=None):
    cache = cache or model.new_device_cache(max_batch=4, max_seq=max(64, len(toks)))
    return cache.forward_ragged([slot], [toks], [list(range(len(toks)))])


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
    "attention": config([att()]),
    "attention_full_rotation_plain": config([att(heads=3, kv_heads=3, dim=6, vdim=4, rot_dims=6, softcap=None, base=300.0)]),
    "attention_one_kv_head_yarn": config([att(heads=6, kv_heads=1, dim=12, vdim=20, rot_dims=8, yarn=(8.0, 12, 4.0, 0.5), base=500.0, softcap=2.0, scale=1.5)]),
    "attention_no_rotation": config([att(rot_dims=0)]),
    "attention_shared_cache": config([att(mlp=dense()), att(heads=2, kv_heads=2, kv_from=0, scale=0.9, softcap=5.0)]),
    "mamba2": config([mamba()]),
    "mamba2_wide": config([mamba(heads=6, vdim=40, state=37, groups=3, norm_groups=5, conv=5)], width=40),
    "mamba2_one_group_two_taps": config([mamba(heads=3, vdim=4, state=4, groups=1, norm_groups=3, conv=2)]),
    "delta": config([delta()]),
    "delta_wide_value": config([delta(heads=6, kv_heads=1, dim=12, vdim=40, conv=5)], width=40),
    "delta_equal_heads_one_tap": config([delta(heads=2, kv_heads=2, dim=16, vdim=8, conv=1)]),
    "dense_ff": config([delta(mlp=dense(ff=40))]),
    "one_head": config([att(heads=1, kv_heads=1, dim=16, vdim=8), mamba(heads=1, groups=1, vdim=16, state=16), delta(heads=1, kv_heads=1, dim=16, vdim=16)]),
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
    cfg = config([mamba(heads=3, vdim=34, state=11, groups=3, norm_groups=2, conv=3, mlp=dense(ff=22)),
                  att(heads=6, kv_heads=3, dim=10, vdim=14, rot_dims=6, mlp=dense(ff=10)),
                  delta(heads=5, kv_heads=5, dim=9, vdim=35, conv=4),
                  att(heads=3, kv_heads=3, dim=10, vdim=14, rot_dims=2, kv_from=1, softcap=None)], vocab=37, width=50)
    oracle, model = build(cfg, seed=5)
    toks = tokens(cfg, 70)
    assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]


def tc_cfg():
    """widths in whole 64-column blocks: in the serving precision the projections run on the tensor-core GEMM (hi | lo activation
    halves); the recurrent mixers' stacked input matrices end in a few per-head rows (padded to a multiple of 8)"""
    return config([delta(heads=4, kv_heads=2, dim=16, vdim=32, conv=4, mlp=dense(ff=64)),
                   att(heads=4, kv_heads=2, dim=32, vdim=16, rot_dims=16, mlp=dense(ff=128)),
                   mamba(heads=4, vdim=16, state=24, groups=2, norm_groups=2, conv=4),
                   att(heads=8, kv_heads=2, dim=32, vdim=16, rot_dims=16, kv_from=1, mlp=dense(ff=64))], vocab=96, width=128)


def tc_cfg_partial_tiles():
    """192-wide: three 64-column k blocks, matrices that end inside a 128-row tile, a feed-forward outside the tiles (ff = 100)"""
    return config([att(heads=3, kv_heads=1, dim=48, vdim=64, rot_dims=32, mlp=dense(ff=320)),
                   mamba(heads=3, vdim=64, state=16, groups=1, norm_groups=3, conv=3, mlp=dense(ff=100)),
                   delta(heads=3, kv_heads=3, dim=64, vdim=64, conv=4)], vocab=200, width=192)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("make", [tc_cfg, tc_cfg_partial_tiles])
def test_tensor_core_projections(make, dtype):
    """1 row, a few rows, up to 128 rows (weights as the 128-row operand, split-K) and more (tokens as rows) through the same layers"""
    cfg = make()
    oracle, model = build(cfg, seed=21, dtype=dtype)
    toks = tokens(cfg, 333, seed=9)
    ref = oracle.run(toks)
    assert relerr(run_whole(model, toks, cache=model.new_device_cache(4, 384)), ref) < TOL[dtype]
    assert relerr(run_cut(model, toks, [5, 128, 129, 2, 60], cache=model.new_device_cache(4, 384)), ref) < TOL[dtype]


def test_tensor_core_attention_long_portions():
    """serving precision, portions of 64 tokens and more: scores and weighted sums run as tensor-core GEMMs per key/value head
    (query heads of a group as extra rows).  Two sequences bring long portions in the same step, at positions past the start
    and across page borders; the cap and the sink both bite (sharp scores); a short tail falls to the per-row kernel."""
    cfg = config([att(heads=6, kv_heads=2, dim=24, vdim=40, rot_dims=8, softcap=6.0, scale=1.0, mlp=None),
                  att(heads=4, kv_heads=2, dim=24, vdim=40, rot_dims=24, softcap=None, scale=0.3, kv_from=0, mlp=dense(ff=64))], vocab=64, width=64)
    oracle, model = build(cfg, seed=31, dtype="bf16", tweak=_sharp)
    a, b = tokens(cfg, 300, seed=1), tokens(cfg, 200, seed=2)
    ra, rb = oracle.run(a), oracle.run(b)
    cache = model.new_device_cache(max_batch=2, max_seq=320)
    got_a, got_b = [], []
    for (na0, na1), (nb0, nb1) in (((0, 70), (0, 3)), ((70, 199), (3, 130)), ((199, 300), (130, 200))):
        lg = cache.forward_ragged([1, 0], [a[na0:na1], b[nb0:nb1]], [list(range(na1 - na0)), list(range(nb1 - nb0))])
        got_a.append(lg[:na1 - na0])
        got_b.append(lg[na1 - na0:])
    assert relerr(np.concatenate(got_a), ra) < TOL["bf16"] and relerr(np.concatenate(got_b), rb) < TOL["bf16"]
    # the same positions through the per-row kernel (token by token) agree with the GEMM path
    single = run_cut(model, b, [], cache=model.new_device_cache(max_batch=1, max_seq=256))
    assert relerr(single, rb) < TOL["bf16"]


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


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 2], [5, 64, 2, 17], [63, 2, 64], [1, 66, 2, 2, 2, 40], [3, 1, 1, 2, 1, 3, 1, 1, 1, 4]])
def test_portions(cuts):
    """a prompt cut into portions (down to two tokens and single ones: shorter than the convolutions reach back, so a row's taps
    come from this step, from the slot's carried inputs and from before the start at once), across page borders, the rest decoded"""
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=8)
    toks = tokens(cfg, 150, seed=4)
    assert relerr(run_cut(model, toks, cuts), oracle.run(toks)) < TOL["f32"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mixed_batch_equals_each_alone(dtype):
    """three requests of unequal length advance together: portions of one beside single tokens of another"""
    cfg = hybrid_cfg()
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
    in its pages, its state slot and its carried convolution inputs must not leak into the next one"""
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=10)
    cache = model.new_device_cache(max_batch=2, max_seq=192, pool_tokens=192)
    assert cache.pool_stats() == (3, 3)
    for i, n in enumerate((130, 100, 64, 65, 3, 1, 2)):
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
    # a request decoded token by token in a slot whose previous owner left a long state behind
    cache.slot_reset(0)
    short = tokens(cfg, 6, seed=34)
    assert relerr(run_cut(model, short, [], slot=0, cache=cache), oracle.run(short)) < TOL["f32"]


# ---- keys that must be seen, and the sink: made to stand out ------------------------------------------------------------------
def _sharp(w):
    """query and key norm weights scaled up: scores reach the cap, the softmax is nearly one-hot, so a key that is wrongly dropped
    or taken from a wrong page moves the logits"""
    for k in w:
        if k.endswith("q.norm") or k.endswith("k.norm"):
            w[k] = O.bf16_round(w[k] * 3.0)


def test_far_keys_across_pages():
    """peaky attention over 300 tokens (five pages): every position checked in a whole prompt, in portions and decoded one by one"""
    cfg = config([att(softcap=40.0, scale=1.0, mlp=None), att(heads=2, kv_heads=2, softcap=40.0, scale=1.0, kv_from=0, mlp=dense())])
    oracle, model = build(cfg, seed=11, tweak=_sharp)
    toks = tokens(cfg, 300, seed=5)
    ref = oracle.run(toks)
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [65, 2, 61, 128]), ref) < TOL["f32"]
    # the attention does look far back: hiding the first 200 keys from the last position changes its logits well beyond the bar
    st = oracle.new_state()
    oracle.run(toks[:-1], st)
    for i in st["kv"]:
        st["kv"][i] = ([np.zeros_like(k) if j < 200 else k for j, k in enumerate(st["kv"][i][0])], st["kv"][i][1])
    assert relerr(oracle.step(toks[-1], st)[None], ref[-1:]) > 100 * TOL["f32"]


def test_sink_and_cap_would_show():
    """the oracle itself without the extra one in the denominator, or without the score cap, is far outside the bar"""
    cfg = config([att(softcap=3.0, scale=1.0)])
    w = O.random_weights(cfg, 11)
    toks = tokens(cfg, 40, seed=5)
    ref = O.Rofetar(cfg, w).run(toks)
    no_cap = O.Rofetar(config([att(softcap=None, scale=1.0)]), w).run(toks)
    assert relerr(no_cap, ref) > 100 * TOL["f32"]
    saved = O.sink_softmax
    try:
        O.sink_softmax = lambda s: np.exp(s - s.max()) / np.exp(s - s.max()).sum()
        assert relerr(O.Rofetar(cfg, w).run(toks), ref) > 100 * TOL["f32"]
    finally:
        O.sink_softmax = saved
    _, model = build(cfg, seed=11)
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]


def _long_memory(w):
    """slow decays: the recurrent states forget slowly, tokens hundreds of positions back still count"""
    for k in w:
        if k.endswith("A_log"):
            w[k] = O.bf16_round(np.full_like(w[k], -6.0))
        if k.endswith("mix.dt_bias"):
            w[k] = O.bf16_round(np.full_like(w[k], -1.0))


@pytest.mark.parametrize("kind", ["mamba2", "delta"])
def test_far_tokens_reach_through_the_state(kind):
    # the delta rule overwrites what earlier tokens wrote along the keys that follow: 64 key channels leave room for 400 tokens
    layer = mamba(mlp=None) if kind == "mamba2" else delta(dim=64, mlp=None)
    cfg = config([layer, dict(layer, mlp=dense())])
    oracle, model = build(cfg, seed=12, tweak=_long_memory)
    toks = tokens(cfg, 400, seed=6)
    ref = oracle.run(toks)
    # the first token matters at the end: changing it alone moves the last logits well beyond the bar
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert relerr(oracle.run(other)[-1:], ref[-1:]) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [2, 300, 2]), ref) < TOL["f32"]


def test_first_tokens():
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=13)
    for n in (1, 2, 3, 5):
        toks = tokens(cfg, n, seed=n)
        assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]
        assert relerr(run_cut(model, toks, []), oracle.run(toks)) < TOL["f32"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_long_decoding(dtype):
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=14, dtype=dtype)
    toks = tokens(cfg, 330, seed=7)
    assert relerr(run_cut(model, toks, [10]), oracle.run(toks)) < TOL[dtype]


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
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=15)
    prompts = [tokens(cfg, n, seed=40 + n) for n in (5, 70, 23, 9, 31)]
    want = [oracle_greedy(oracle, p, 12) for p in prompts]
    assert models.Model(model, None, eos_token_id=None).generate(prompts[0], 12) == want[0]
    assert models.ContinuousBatcher(model, max_batch=3, eos_token_id=None).generate(prompts, 12) == want
    b = models.ContinuousBatcher(model, max_batch=2, eos_token_id=None, prefill_chunk=16)
    assert b.generate(prompts, 12) == want
    assert b.cache.pool_stats()[0] == b.cache.pool_stats()[1]


def test_uniform_entry_points_and_errors():
    cfg = hybrid_cfg()
    oracle, model = build(cfg, seed=16)
    toks = tokens(cfg, 20)
    cache = model.new_device_cache(max_batch=2, max_seq=64)
    ref = oracle.run(toks)
    both = cache.forward(np.asarray([toks[:12], toks[:12]], dtype=np.uint32), 0)
    assert relerr(both, np.stack([ref[11], ref[11]])) < TOL["f32"]
    nxt = cache.forward_slots([1], np.asarray([toks[12:]], dtype=np.uint32), [12])
    assert relerr(nxt, ref[19:20]) < TOL["f32"]
    bad = config([att(), att(kv_from=0, dim=4)])            # a shared cache needs equal key sizes
    with pytest.raises(FastllmError):
        models.RofetarWithConfig.initialize_model(bad, {k: to_bits(v) for k, v in O.random_weights(bad).items()}, "f32")
    missing = {k: to_bits(v) for k, v in O.random_weights(cfg).items() if k != "l2.mix.conv.b"}
    with pytest.raises(FastllmError):
        models.RofetarWithConfig.initialize_model(cfg, missing, "f32")
    clone = model.clone()
    assert relerr(run_whole(clone, toks), ref) < TOL["f32"]


def _write_checkpoint(folder, cfg, w):
    from fastllm_b200 import safetensors_io
    folder.mkdir(exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    safetensors_io.write_safetensors(str(folder / "model.safetensors"), {k: to_bits(v) for k, v in w.items()})


def test_checkpoint_folder_through_the_registry(tmp_path):
    cfg = hybrid_cfg()
    w = O.random_weights(cfg, 17)
    _write_checkpoint(tmp_path / "m", cfg, w)
    model, _ = models.load_model(str(tmp_path / "m"), "f32")
    assert isinstance(model, models.RofetarWithConfig)
    toks = tokens(cfg, 30)
    assert relerr(run_whole(model, toks), O.Rofetar(cfg, w).run(toks)) < TOL["f32"]


def test_command_line_generate(tmp_path):
    """python -m fastllm_b200 generate: registry, loader, continuous batcher with prompt portions, greedy sampling -- ids in, ids out"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = hybrid_cfg()
    w = O.random_weights(cfg, 29)
    _write_checkpoint(tmp_path / "m", cfg, w)
    prompts = [tokens(cfg, n, seed=60 + n) for n in (3, 40, 17)]
    cmd = ["python3", "-m", "fastllm_b200", "generate", "--model", str(tmp_path / "m"), "--dtype", "f32", "--max-tokens", "6", "--max-batch", "2",
           "--prefill-chunk", "16"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root, env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, r.stderr[-2000:]
    got = [json.loads(l)["generated"] for l in r.stdout.splitlines() if l.startswith("{")]
    oracle = O.Rofetar(cfg, w)
    assert got == [oracle_greedy(oracle, p, 6) for p in prompts]


def test_trace_runner_end_to_end(tmp_path):
    """bin/trace_run as a process: steps on standard input (portions beside single tokens, a request that sits out a step, one that
    wants nothing, a fifth request that takes over a finished one's slot and pages), logits files out"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = hybrid_cfg()
    w = O.random_weights(cfg, 23)
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    _write_checkpoint(model_dir, cfg, w)
    reqs = {name: tokens(cfg, n, seed=50 + i) for i, (name, n) in enumerate((("a", 70), ("b", 5), ("c", 33), ("d", 64), ("e", 40)))}
    refs = {"float32": {k: O.Rofetar(cfg, w).run(v) for k, v in reqs.items()},
            "bfloat16": {k: O.Rofetar(cfg, w, cache_round=O.bf16_round).run(v) for k, v in reqs.items()}}
    plan = [[("a", 3, [0, 2]), ("b", 1, [0])],
            [("a", 60, [59]), ("c", 33, []), ("d", 2, [1])],
            [("b", 4, [0, 3]), ("d", 62, [0, 61])],
            [("a", 1, [0]), ("e", 40, [39])],
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
