"""Plain, slow restatement of the Rofetar decoder: a hybrid of softmax attention with a sink, Mamba-2 state-space layers and
gated-delta-rule layers, each sublayer's OUTPUT normed before it joins the residual stream.  Test infrastructure only: numpy,
one function per mechanism, token by token, float64.  Nothing of the product imports this file and this file imports nothing
of the product.

Notation: x is the residual row a sublayer reads (not normed), W matrices are [out, in] and applied as W @ x.
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ----------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_w(x, w, eps):
    return rms_unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def glu_gelu(x, wg, bg, wu, bu, wd, bd):
    return wd @ (gelu_tanh(wg @ x + bg) * (wu @ x + bu)) + bd


def rotary_freqs(dims, base, scaling):
    """-> (angle per position for each of the dims/2 pairs, multiplier of cos and sin)"""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_index(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_index(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x, pos, freqs, mult, dims):
    """rotary embedding on the first `dims` entries of the last axis, entry i paired with entry i + dims/2; the rest pass"""
    out = np.array(x, dtype=np.float64, copy=True)
    half = dims // 2
    a = pos * freqs
    c, s = np.cos(a) * mult, np.sin(a) * mult
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def sink_softmax(s):
    """p_j = exp(s_j) / (1 + sum_k exp(s_k)): one more, valueless, entry of score 0 in the denominator"""
    m = max(float(s.max()), 0.0)
    e = np.exp(s - m)
    return e / (math.exp(-m) + e.sum())


def conv_step(hist, x, w, b=None):
    """causal per-channel convolution: hist [taps-1, channels] holds the previous inputs (oldest first, zeros before the start);
    w [channels, taps], the last column meets the current input.  -> (output [channels], new hist)"""
    full = np.concatenate([hist, x[None, :]], axis=0)           # [taps, channels]
    y = np.einsum("tc,ct->c", full, w)
    if b is not None:
        y = y + b
    return y, full[1:]


# ---- the model -------------------------------------------------------------------------------------------------------
class Rofetar:
    """weights: dict name -> float array holding the values the product sees (bf16-representable).
    cache_round: optional function applied to the keys and values an attention layer caches."""

    def __init__(self, config: dict, weights: dict, cache_round=None):
        self.cfg = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.layers = config["layers"]
        self.cache_round = cache_round

    def new_state(self):
        st = {"pos": 0, "kv": {}, "S": {}, "conv": {}}
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "attention":
                if m.get("kv_from") is None:
                    st["kv"][i] = ([], [])
            elif l["type"] == "mamba2":
                ch = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
                st["S"][i] = np.zeros((m["heads"], m["state"], m["vdim"]))
                st["conv"][i] = np.zeros((m["conv"] - 1, ch))
            elif l["type"] == "delta":
                st["S"][i] = np.zeros((m["heads"], m["dim"], m["vdim"]))
                st["conv"][i] = {"q": np.zeros((m["conv"] - 1, m["kv_heads"] * m["dim"])),
                                 "k": np.zeros((m["conv"] - 1, m["kv_heads"] * m["dim"])),
                                 "v": np.zeros((m["conv"] - 1, m["heads"] * m["vdim"]))}
            else:
                raise ValueError(l["type"])
        return st

    # -- mixers --
    def attention(self, i, x, st):
        m, w, p = self.layers[i]["mixer"], self.w, f"l{i}.mix."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        pos = st["pos"]
        rot = m.get("rot") or {}
        rd = int(rot.get("dims", 0))
        freqs, mult = rotary_freqs(rd, float(rot.get("base", 10000.0)), rot.get("scaling")) if rd else (None, 1.0)
        q = norm_w((w[p + "q"] @ x).reshape(H, D), w[p + "q.norm"], self.eps)
        if rd:
            q = rotate_halves(q, pos, freqs, mult, rd)
        src = m.get("kv_from")
        if src is None:
            k = norm_w((w[p + "k"] @ x).reshape(G, D), w[p + "k.norm"], self.eps)
            if rd:
                k = rotate_halves(k, pos, freqs, mult, rd)
            v = (w[p + "v"] @ x).reshape(G, Dv)
            if self.cache_round is not None:
                k, v = np.asarray(self.cache_round(k), dtype=np.float64), np.asarray(self.cache_round(v), dtype=np.float64)
            st["kv"][i][0].append(k)
            st["kv"][i][1].append(v)
            src = i
        K = np.stack(st["kv"][src][0][:pos + 1])           # [n, G, D]
        V = np.stack(st["kv"][src][1][:pos + 1])           # [n, G, Dv]
        cap = m.get("softcap")
        out = np.zeros((H, Dv))
        for hd in range(H):
            g = hd // (H // G)
            s = (K[:, g, :] @ q[hd]) * float(m["scale"])
            if cap:
                s = float(cap) * np.tanh(s / float(cap))
            out[hd] = sink_softmax(s) @ V[:, g, :]
        return w[p + "o"] @ out.reshape(-1)

    def mamba2(self, i, x, st):
        m, w, p = self.layers[i]["mixer"], self.w, f"l{i}.mix."
        H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
        inner = H * P
        u = w[p + "in"] @ x
        z, xbc, dt = u[:inner], u[inner:2 * inner + 2 * G * N], u[2 * inner + 2 * G * N:]
        xbc, st["conv"][i] = conv_step(st["conv"][i], xbc, w[p + "conv"], w[p + "conv.b"])
        xbc = silu(xbc)
        xs = xbc[:inner].reshape(H, P)
        B = xbc[inner:inner + G * N].reshape(G, N)
        Cc = xbc[inner + G * N:].reshape(G, N)
        dt = softplus(dt + w[p + "dt_bias"])
        decay = np.exp(-np.exp(w[p + "A_log"]) * dt)
        S = st["S"][i]
        y = np.zeros((H, P))
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[hd] * S[hd] + dt[hd] * np.outer(B[g], xs[hd])
            y[hd] = S[hd].T @ Cc[g] + w[p + "D"][hd] * xs[hd]
        y = y.reshape(-1) * silu(z)
        ng = int(m.get("norm_groups", 1))
        y = rms_unit(y.reshape(ng, inner // ng), self.eps).reshape(-1) * w[p + "norm"]
        return w[p + "o"] @ y

    def delta(self, i, x, st):
        m, w, p = self.layers[i]["mixer"], self.w, f"l{i}.mix."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        cs = st["conv"][i]
        q, cs["q"] = conv_step(cs["q"], w[p + "q"] @ x, w[p + "q.conv"])
        k, cs["k"] = conv_step(cs["k"], w[p + "k"] @ x, w[p + "k.conv"])
        v, cs["v"] = conv_step(cs["v"], w[p + "v"] @ x, w[p + "v.conv"])
        q, k, v = silu(q).reshape(G, D), silu(k).reshape(G, D), silu(v).reshape(H, Dv)
        q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * D ** -0.5
        k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
        beta = sigmoid(w[p + "b"] @ x)
        decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(w[p + "a"] @ x + w[p + "dt_bias"]))
        S = st["S"][i]
        o = np.zeros((H, Dv))
        for hd in range(H):
            g = hd // (H // G)
            S[hd] *= decay[hd]
            upd = beta[hd] * (v[hd] - S[hd].T @ k[g])
            S[hd] += np.outer(k[g], upd)
            o[hd] = S[hd].T @ q[g]
        o = norm_w(o, w[p + "norm"], self.eps).reshape(-1) * silu(w[p + "g"] @ x)
        return w[p + "o"] @ o

    def ff(self, i, x):
        c, w, p = self.layers[i]["mlp"], self.w, f"l{i}.mlp."
        if c["kind"] != "dense":
            raise ValueError(c["kind"])
        return glu_gelu(x, w[p + "gate"], w[p + "gate.b"], w[p + "up"], w[p + "up.b"], w[p + "down"], w[p + "down.b"])

    # -- one token through every layer --
    def step(self, token, st, layer_trace=None):
        w, eps = self.w, self.eps
        x = w["embed"][int(token)].copy()
        for i, l in enumerate(self.layers):
            y = getattr(self, l["type"])(i, x, st)
            x = x + norm_w(y, w[f"l{i}.norm1"], eps)
            if l.get("mlp"):
                x = x + norm_w(self.ff(i, x), w[f"l{i}.norm2"], eps)
            if layer_trace is not None:
                layer_trace.append(x.copy())
        st["pos"] += 1
        return w["head"] @ norm_w(x, w["final.norm"], eps)

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
        out[p + "norm1"] = (W,)
        if l["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[p + "mix.q"], out[p + "mix.q.norm"], out[p + "mix.o"] = (H * D, W), (D,), (W, H * Dv)
            if m.get("kv_from") is None:
                out[p + "mix.k"], out[p + "mix.v"], out[p + "mix.k.norm"] = (G * D, W), (G * Dv, W), (D,)
        elif l["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            ch = H * P + 2 * G * N
            out[p + "mix.in"] = (2 * H * P + 2 * G * N + H, W)
            out[p + "mix.conv"], out[p + "mix.conv.b"] = (ch, m["conv"]), (ch,)
            out[p + "mix.dt_bias"], out[p + "mix.A_log"], out[p + "mix.D"] = (H,), (H,), (H,)
            out[p + "mix.norm"], out[p + "mix.o"] = (H * P,), (W, H * P)
        else:
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                out[p + "mix." + n], out[p + "mix." + n + ".conv"] = (rows, W), (rows, m["conv"])
            out[p + "mix.b"], out[p + "mix.a"] = (H, W), (H, W)
            out[p + "mix.A_log"], out[p + "mix.dt_bias"], out[p + "mix.norm"] = (H,), (H,), (Dv,)
            out[p + "mix.g"], out[p + "mix.o"] = (H * Dv, W), (W, H * Dv)
        c = l.get("mlp")
        if not c:
            continue
        out[p + "norm2"] = (W,)
        F = c["ff"]
        out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (F, W), (F, W), (W, F)
        out[p + "mlp.gate.b"], out[p + "mlp.up.b"], out[p + "mlp.down.b"] = (F,), (F,), (W,)
    return out


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """bf16-representable random weights: matrices N(0, 1/in); norm weights around 1; decays spread over fast and slow heads"""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shp in tensor_shapes(cfg).items():
        if name.endswith("A_log"):
            a = rng.uniform(-3.0, 1.0, shp)
        elif name.endswith("dt_bias"):
            a = rng.uniform(-3.0, 0.5, shp)
        elif name.endswith(".conv"):
            a = rng.normal(0.0, 0.5, shp)
        elif name.endswith(".D"):
            a = rng.normal(1.0, 0.3, shp)
        elif len(shp) == 1:
            a = rng.normal(0.0, 0.2, shp)
            if "norm" in name:
                a = 1.0 + a
        elif name == "embed":
            a = rng.normal(0.0, 1.0, shp)
        else:
            a = rng.normal(0.0, 1.0, shp) / math.sqrt(shp[1])
        w[name] = bf16_round(a)
    return w
