"""Host-side pieces of the layered decoder (Nifunex) that need no GPU: config.json -> layer descriptors, the registry, the mixed-step
scheduler over a stand-in cache, and closed-form checks of the plain restatement (oracle/nifunex.py) that the GPU tests lean on."""
import math

import numpy as np
import pytest

from fastllm_b200 import _lib, models
from oracle import nifunex as O


def _cfg():
    return {"architecture": "Nifunex", "vocab": 40, "width": 24, "norm": {"eps": 1e-6}, "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 6, "vdim": 10, "tau": 4.0}, "mlp": {"kind": "dense", "ff": 20, "limit": 1.25}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "rot_dim": 6, "vdim": 8, "kv_rank": 12, "scale": 0.3, "mask": {"size": 5},
                                                "rot": {"base": 777.0, "dims": 4, "scaling": {"factor": 2.0, "original": 64, "fast": 8.0, "slow": 2.0}}},
         "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 0.5}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 16, "limit": 2.0}}},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 4, "rot_dim": 6, "vdim": 8, "kv_rank": 12, "scale": 0.5, "kv_from": 1,
                                                "rot": {"base": 777.0, "dims": 4, "scaling": {"factor": 2.0, "original": 64, "fast": 8.0, "slow": 2.0}}},
         "mlp": None}]}


def test_config_to_layer_descs():
    d = models.nifunex_layer_descs(_cfg(), {0: 3})
    g, a, b = d[0], d[1], d[2]
    assert (g.mixer, g.heads, g.dim, g.vdim, g.decay_rank, g.tau) == (_lib.FL_MIXER["gla"], 2, 6, 10, 3, 4.0)
    assert (g.ffn, g.ff, g.limit, g.kv_from) == (_lib.FL_FFN["dense"], 20, 1.25, -1)
    assert (a.mixer, a.rot_dim, a.kv_rank, a.window, a.rot_dims, a.rot_base, a.kv_from) == (_lib.FL_MIXER["latent_attention"], 6, 12, 5, 4, 777.0, -1)
    assert (a.yarn_factor, a.yarn_original, a.yarn_fast, a.yarn_slow) == (2.0, 64.0, 8.0, 2.0) and abs(a.scale - 0.3) < 1e-7
    assert (a.ffn, a.ff, a.experts, a.top, a.shared_ff, a.shared_limit, a.limit) == (_lib.FL_FFN["moe"], 8, 6, 2, 16, 2.0, 0.5)
    assert (b.kv_from, b.window, b.ffn, b.heads) == (1, 0, _lib.FL_FFN["none"], 1)
    with pytest.raises(models.FastllmError):
        models.nifunex_layer_descs(_cfg(), {})          # the decay bottleneck's size must come from somewhere
    bad = _cfg()
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(models.FastllmError):
        models.nifunex_layer_descs(bad, {0: 3})


def test_registry_picks_by_architecture():
    assert models.model_class_for({"architecture": "Nifunex"}) is models.NifunexWithConfig
    assert models.model_class_for({"architectures": ["MistralForCausalLM"]}) is models.MistralWithConfig
    assert models.NifunexWithConfig.get_family() == "Nifunex" and not models.NifunexWithConfig.supports_architecture("LlamaForCausalLM")
    with pytest.raises(models.FastllmError):
        models.model_class_for({"architecture": "Unheard"})


class _FakeRagged:
    """stand-in for DeviceCache: the 'model' predicts (sum of all tokens the slot has seen) % vocab; records every step"""
    vocab = 11

    def __init__(self):
        self.seen, self.steps, self.resets = {}, [], 0

    def forward_ragged(self, slots, toks, want):
        self.steps.append([(s, len(t)) for s, t in zip(slots, toks)])
        rows = []
        for s, t, w in zip(slots, toks, want):
            base = self.seen.get(s, 0)
            for i, tok in enumerate(t):
                base += int(tok)
                if i in w:
                    r = np.zeros(self.vocab, dtype=np.float32)
                    r[base % self.vocab] = 1.0
                    rows.append(r)
            self.seen[s] = base
        return np.stack(rows) if rows else np.zeros((0, self.vocab), dtype=np.float32)

    def slot_reset(self, s):
        self.seen.pop(s, None)
        self.resets += 1


def test_mixed_step_scheduler(_built):
    class M:
        arch, position_per_call = "nifunex", False
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9], [3, 3, 3]]
    fake = _FakeRagged()
    b = models.ContinuousBatcher(M(), max_batch=2, eos_token_id=None, cache=fake, prefill_chunk=3)
    out = b.generate(prompts, 4)

    def expect(p):
        s, res = sum(p), []
        for _ in range(4):
            res.append(s % 11)
            s += s % 11
        return res
    assert out == [expect(p) for p in prompts]
    assert fake.steps[0] == [(0, 3), (1, 1)]                 # a prompt's first portion beside a one-token prompt
    assert any(len(st) == 2 and {n for _, n in st} == {3, 1} for st in fake.steps[1:])     # a portion beside a decoded token
    assert fake.resets == 3 and all(n <= 3 for st in fake.steps for _, n in st)


# ---- the plain restatement, checked in closed form ---------------------------------------------------------------------------
def test_oracle_recurrence_is_the_decayed_sum():
    """o_t = sum_{j<=t} (q_t . (prod_{j<i<=t} alpha_i) * k_j) v_j"""
    cfg = {"vocab": 8, "width": 12, "norm": {"eps": 1e-5}, "layers": [{"type": "gla", "mixer": {"heads": 1, "dim": 3, "vdim": 2, "tau": 2.0, "decay_rank": 2}, "mlp": None}]}
    w = O.random_weights(cfg, 1)
    m = O.Nifunex(cfg, w)
    st = m.new_state()
    rng = np.random.default_rng(0)
    hs = rng.normal(size=(6, 12))
    W = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    got = []
    for h in hs:
        m.gla(0, h, st)
        got.append(st["gla"][0][0].copy())
    alpha = [1.0 / (1.0 + np.exp(-(W["l0.mix.a2"] @ (W["l0.mix.a1"] @ h) + W["l0.mix.a2.b"]))) ** 0.5 for h in hs]
    S = np.zeros((3, 2))
    for t, h in enumerate(hs):
        S = sum(np.prod(np.stack(alpha[j + 1:t + 1] + [np.ones(3)]), axis=0)[:, None] * np.outer(W["l0.mix.k"] @ hs[j], W["l0.mix.v"] @ hs[j]) for j in range(t + 1))
        assert np.allclose(S, got[t], rtol=1e-10, atol=1e-12)


def test_oracle_rotation_and_yarn():
    f, mult = O.yarn_freqs(8, 100.0, None)
    assert mult == 1.0 and np.allclose(f, 100.0 ** (-np.arange(4) / 4.0))
    f2, mult2 = O.yarn_freqs(8, 100.0, {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0})
    corr = lambda t: 8 * math.log(32 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(corr(4.0)), 0), min(math.ceil(corr(1.0)), 7)
    ramp = np.clip((np.arange(4) - lo) / max(hi - lo, 0.001), 0, 1)
    assert np.allclose(f2, f / 4.0 * ramp + f * (1 - ramp)) and abs(mult2 - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    x = np.arange(6, dtype=np.float64) + 1.0
    y = O.rotate_pairs(x, 3, f[:2], 1.0, 4)
    a = 3 * f[:2]
    assert np.allclose(y[0:4:2], x[0:4:2] * np.cos(a) - x[1:4:2] * np.sin(a)) and np.allclose(y[1:4:2], x[1:4:2] * np.cos(a) + x[0:4:2] * np.sin(a))
    assert np.array_equal(y[4:], x[4:])         # channels past the rotated ones pass through


def test_oracle_router_and_clamped_glu():
    picks = O.route_topk(np.ones(3), np.array([[0.0, 0, 0], [1.0, 0, 0], [1.0, 0, 0], [-1.0, 0, 0]]), 2)
    assert [e for e, _ in picks] == [1, 2] and abs(sum(wt for _, wt in picks) - 1.0) < 1e-12       # equal scores: lower index first
    h = np.array([2.0, -3.0])
    eye = np.eye(2)
    y = O.glu_clamped(h, eye, eye, eye, 1.0)
    g, u = np.minimum(h, 1.0), np.clip(h, -1.0, 1.0)
    assert np.allclose(y, g / (1 + np.exp(-1.702 * g)) * (u + 1.0)) and g[1] == -3.0               # the gate is only clamped from above
