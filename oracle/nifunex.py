"""Plain, slow restatement of the Nifunex decoder (hybrid of gated-linear-attention layers and windowed latent-attention
layers, dense or mixture-of-experts feed-forward, a norm before AND after every sublayer).  Test infrastructure only: numpy,
one function per mechanism, token by token, float64 unless told otherwise.  Nothing of the product imports this file and this
file imports nothing of the product.

Notation: h is a sublayer's input row (already normed), W matrices are [out, in] and applied as W @ h.
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ----------------------------------------------------------------------------------------------------
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_offset(x, w, eps):
    """the layer norms and the final norm: zero-centred weight: the scale is 1 + w"""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    """the norms inside the mixers: ordinary weight"""
    return rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def glu_clamped(h, w_gate, w_up, w_down, limit):
    """g = min(Wg h, L); u = clamp(Wu h, -L, L); down((g * sigmoid(1.702 g)) * (u + 1))"""
    g = np.minimum(w_gate @ h, limit)
    u = np.clip(w_up @ h, -limit, limit)
    return w_down @ (g * sigmoid(1.702 * g) * (u + 1.0))


def route_topk(h, w_router, top):
    """softmax over ALL experts, the `top` largest (lower index first among equals), renormalised by their sum + 1e-20"""
    z = (w_router @ h).astype(np.float64)
    s = np.exp(z - z.max())
    s /= s.sum()
    picks = sorted(range(len(s)), key=lambda e: (-s[e], e))[:top]
    wsum = sum(s[e] for e in picks) + 1e-20
    return [(e, s[e] / wsum) for e in picks]


def yarn_freqs(dims, base, scaling):
    """-> (frequency per pair [dims/2], multiplier of cos and sin)"""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def corr(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(corr(float(scaling["fast"]))), 0)
    hi = min(math.ceil(corr(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, freqs, mult, dims):
    """interleaved rotary embedding on the first `dims` entries of the last axis; the rest pass through"""
    out = np.array(x, dtype=np.float64, copy=True)
    a = pos * freqs
    c, s = np.cos(a) * mult, np.sin(a) * mult
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- the model -------------------------------------------------------------------------------------------------------
class Nifunex:
    """weights: dict name -> float array (already holding the values the product sees, e.g. bf16-rounded).
    cache_round: optional function applied to what a latent-attention layer caches (latent and rotated key part) -- bf16_round
    restates a cache kept in bfloat16, so that a serving-precision run can be held to a tight bar."""

    def __init__(self, config: dict, weights: dict, cache_round=None):
        self.cache_round = cache_round
        self.cfg = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.layers = config["layers"]

    def new_state(self):
        st = {"pos": 0, "gla": {}, "kv": {}}
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "gla":
                st["gla"][i] = np.zeros((m["heads"], m["dim"], m["vdim"]))
            elif "kv_from" not in m:
                st["kv"][i] = []            # list of (latent, rotated key) per position
        return st

    # -- mixers --
    def gla(self, i, h, st):
        m, w, p = self.layers[i]["mixer"], self.w, f"l{i}.mix."
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        q = (w[p + "q"] @ h).reshape(H, D) * D ** -0.5
        k = (w[p + "k"] @ h).reshape(H, D)
        v = (w[p + "v"] @ h).reshape(H, Dv)
        z = w[p + "a2"] @ (w[p + "a1"] @ h) + w[p + "a2.b"]
        log_alpha = (-np.logaddexp(0.0, -z) / float(m["tau"])).reshape(H, D)      # log(sigmoid(z)) / tau
        S = st["gla"][i]
        S *= np.exp(log_alpha)[:, :, None]
        S += k[:, :, None] * v[:, None, :]
        o = np.einsum("hdv,hd->hv", S, q)
        o = norm_plain(o, w[p + "norm"], self.eps).reshape(-1)
        g = w[p + "g"] @ h
        return w[p + "o"] @ (o * (g * sigmoid(g)))

    def latent_attention(self, i, h, st):
        m, w, p = self.layers[i]["mixer"], self.w, f"l{i}.mix."
        H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        pos = st["pos"]
        freqs, mult = yarn_freqs(m["rot"]["dims"], float(m["rot"]["base"]), m["rot"].get("scaling"))
        q = (w[p + "q"] @ h).reshape(H, D + R)
        q_plain, q_rot = q[:, :D], rotate_pairs(q[:, D:], pos, freqs, mult, m["rot"]["dims"])
        src = m.get("kv_from")
        if src is None:
            ckv = w[p + "dkv"] @ h
            lat = norm_plain(ckv[:C], w[p + "dkv.norm"], self.eps)
            krot = rotate_pairs(ckv[C:], pos, freqs, mult, m["rot"]["dims"])
            if self.cache_round is not None:
                lat, krot = np.asarray(self.cache_round(lat), dtype=np.float64), np.asarray(self.cache_round(krot), dtype=np.float64)
            st["kv"][i].append((lat, krot))
            src = i
        hist = st["kv"][src]
        win = (m.get("mask") or {}).get("size")
        first = 0 if win is None else max(0, pos - int(win) + 1)
        lats = np.stack([hist[j][0] for j in range(first, pos + 1)])          # [n, C]
        krots = np.stack([hist[j][1] for j in range(first, pos + 1)])         # [n, R]
        uk = w[p + "uk"].reshape(H, D, C)
        uv = w[p + "uv"].reshape(H, Dv, C)
        out = np.zeros((H, Dv))
        for hd in range(H):
            kk = lats @ uk[hd].T                                               # [n, D]
            vv = lats @ uv[hd].T                                               # [n, Dv]
            s = (kk @ q_plain[hd] + krots @ q_rot[hd]) * float(m["scale"])
            pr = np.exp(s - s.max())
            pr /= pr.sum()
            out[hd] = pr @ vv
        return w[p + "o"] @ out.reshape(-1)

    # -- feed-forward --
    def ff(self, i, h):
        c, w, p = self.layers[i]["mlp"], self.w, f"l{i}.mlp."
        if c["kind"] == "dense":
            return glu_clamped(h, w[p + "gate"], w[p + "up"], w[p + "down"], float(c["limit"]))
        y = np.zeros(self.cfg["width"])
        lim = float(c["expert"]["limit"])
        for e, wt in route_topk(h, w[p + "router"], int(c["router"]["top"])):
            y += wt * glu_clamped(h, w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], lim)
        if c.get("shared"):
            sg = sigmoid(float((w[p + "shared.sg"] @ h).reshape(-1)[0]))
            y += sg * glu_clamped(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], float(c["shared"]["limit"]))
        return y

    # -- one token through every layer --
    def step(self, token, st, layer_trace=None):
        w, eps = self.w, self.eps
        x = w["embed"][int(token)].copy()
        for i, l in enumerate(self.layers):
            h = norm_offset(x, w[f"l{i}.norm1"], eps)
            y = self.gla(i, h, st) if l["type"] == "gla" else self.latent_attention(i, h, st)
            x = x + norm_offset(y, w[f"l{i}.norm1b"], eps)
            if l.get("mlp"):
                h = norm_offset(x, w[f"l{i}.norm2"], eps)
                x = x + norm_offset(self.ff(i, h), w[f"l{i}.norm2b"], eps)
            if layer_trace is not None:
                layer_trace.append(x.copy())
        st["pos"] += 1
        return w["head"] @ norm_offset(x, w["final.norm"], eps)

    def run(self, tokens, st=None, layer_trace=False):
        """-> logits [len(tokens), vocab] (and the residual stream [layers, tokens, width] if asked)"""
        st = st if st is not None else self.new_state()
        out, tr = [], []
        for t in tokens:
            lt = [] if layer_trace else None
            out.append(self.step(t, st, lt))
            if layer_trace:
                tr.append(lt)
        logits = np.stack(out)
        if layer_trace:
            return logits, np.transpose(np.asarray(tr), (1, 0, 2))
        return logits


# ---- random models for tests -----------------------------------------------------------------------------------------
def bf16_round(a):
    """round-to-nearest-even to bfloat16, returned as float32"""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32)


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor the configuration asks for"""
    W, V, out = cfg["width"], cfg["vocab"], {}
    out["embed"], out["head"], out["final.norm"] = (V, W), (V, W), (W,)
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        out[p + "norm1"], out[p + "norm1b"] = (W,), (W,)
        if l["type"] == "gla":
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            out[p + "mix.q"], out[p + "mix.k"] = (H * D, W), (H * D, W)
            out[p + "mix.v"], out[p + "mix.g"], out[p + "mix.o"] = (H * Dv, W), (H * Dv, W), (W, H * Dv)
            out[p + "mix.norm"] = (Dv,)
            out[p + "mix.a1"], out[p + "mix.a2"], out[p + "mix.a2.b"] = (m["decay_rank"], W), (H * D, m["decay_rank"]), (H * D,)
        else:
            H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out[p + "mix.q"], out[p + "mix.o"] = (H * (D + R), W), (W, H * Dv)
            out[p + "mix.uk"], out[p + "mix.uv"] = (H * D, C), (H * Dv, C)
            if "kv_from" not in m:
                out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = (C + R, W), (C,)
        c = l.get("mlp")
        if not c:
            continue
        out[p + "norm2"], out[p + "norm2b"] = (W,), (W,)
        if c["kind"] == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (c["ff"], W), (c["ff"], W), (W, c["ff"])
        else:
            F = c["expert"]["ff"]
            out[p + "mlp.router"] = (c["router"]["experts"], W)
            for e in range(c["router"]["experts"]):
                out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = (F, W), (F, W), (W, F)
            if c.get("shared"):
                Fs = c["shared"]["ff"]
                out[p + "mlp.shared.gate"], out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = (Fs, W), (Fs, W), (W, Fs)
                out[p + "mlp.shared.sg"] = (1, W)
    return out


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """bf16-representable random weights: matrices N(0, 1/in), norm weights and biases small"""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shp in tensor_shapes(cfg).items():
        if len(shp) == 1:
            a = rng.normal(0.0, 0.2, shp)
            if name.endswith("mix.norm") or name.endswith("dkv.norm"):
                a = 1.0 + a
            if name.endswith("a2.b"):
                a = rng.normal(2.0, 1.0, shp)
        else:
            a = rng.normal(0.0, 1.0, shp) / math.sqrt(shp[1])
            if name == "embed":
                a = rng.normal(0.0, 1.0, shp)
        w[name] = bf16_round(a)
    return w
