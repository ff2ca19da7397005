"""Galirax in plain float64 numpy, one function per mechanism, written from the equations and sharing no code with the product
path.  Everything is token by token or dense and slow on purpose.

Notation: x is the residual stream [T, W]; a layer computes h = LN(x) and x <- x + (mixer(h) + experts(h)).
"""
from __future__ import annotations

import math

import numpy as np


def bf16_round(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


# ------------------------------------------------------------------------------------------------ rotation
def rotation_freqs(rot):
    """f_i = base^(-2i/n) for i < n/2; with scaling {factor, low, high, original} a frequency whose wavelength L = 2 pi / f is
    shorter than original / high stays, longer than original / low becomes f / factor, and in between the two are mixed with
    weight s = (original / L - low) / (high - low) on the unscaled one."""
    n = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / n) for i in range(n // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f
    out = []
    for fi in f:
        wl = 2.0 * math.pi / fi
        if wl < sc["original"] / sc["high"]:
            out.append(fi)
        elif wl > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * fi / sc["factor"] + s * fi)
    return np.array(out)


def rotate_pairs(x, pos, rot):
    """x [T, heads, dim]; entries (2i, 2i+1), i < dims/2, turn by pos * f_i; the rest of a head is left alone."""
    n = rot["dims"]
    if n == 0:
        return x.copy()
    ang = np.asarray(pos, dtype=np.float64)[:, None] * rotation_freqs(rot)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    y = x.copy()
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    y[..., 0:n:2] = a * c - b * s
    y[..., 1:n:2] = b * c + a * s
    return y


# ------------------------------------------------------------------------------------------------ attention
def visible(i, j, window=0, keep_first=0):
    """May position i look at position j?"""
    return j <= i and (window <= 0 or i - j < window or j < keep_first)


def sink_attention(q, k, v, scale, sink, window=0, keep_first=0):
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence, H a multiple of G.  Row by row:
    p_j = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j')), out = sum_j p_j v_j: the sink takes weight and gives nothing."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[-1]))
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, window, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = np.array([scale * (q[i, h] @ k[j, g]) for j in js])
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            den = e.sum() + math.exp(sink[h] - m)
            out[i, h] = (e / den) @ np.stack([v[j, g] for j in js])
    return out


def attention_mixer(h, W, pre, mx, eps, with_bias_and_norm, pos0=0):
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q, k, v = h @ W[pre + "q"].T, h @ W[pre + "k"].T, h @ W[pre + "v"].T
    if with_bias_and_norm:
        q, k, v = q + W[pre + "q.b"], k + W[pre + "k.b"], v + W[pre + "v.b"]
        q, k = rms_norm(q, W[pre + "q.norm"], eps), rms_norm(k, W[pre + "k.norm"], eps)  # over all heads at once
    pos = np.arange(pos0, pos0 + T)
    rot = mx.get("rot") or {"dims": 0}
    q, k = rotate_pairs(q.reshape(T, H, D), pos, rot), rotate_pairs(k.reshape(T, G, D), pos, rot)
    mask = mx.get("mask") or {}
    o = sink_attention(q, k, v.reshape(T, G, V), mx["scale"], W[pre + "sink"], mask.get("size", 0), mask.get("keep_first", 0))
    return o.reshape(T, H * V) @ W[pre + "o"].T


# ------------------------------------------------------------------------------------------------ linear attention
def decayed_outer_product_scan(q, k, v, decay, S0=None):
    """Per head: S <- decay_h S + k_t v_t^T, o_t = S^T q_t.  q, k [T, H, D], v [T, H, V]; returns o [T, H, V] and the last S [H, D, V]."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = np.zeros((H, D, V)) if S0 is None else S0.copy()
    o = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def lightning_mixer(h, W, pre, mx, eps):
    T = h.shape[0]
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    q, k, v = (silu(h @ W[pre + n].T) for n in "qkv")
    o, _ = decayed_outer_product_scan(q.reshape(T, H, D), k.reshape(T, H, D), v.reshape(T, H, V), mx["decay"])
    o = rms_norm(o.reshape(T, H * V), W[pre + "norm"], eps) * sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


# ------------------------------------------------------------------------------------------------ experts
def route(z, correction, top, n_group, n_keep, scale):
    """z [E] router logits of one token -> (chosen experts, their weights).  s = sigmoid(z) weighs, c = s + correction chooses;
    groups of E / n_group neighbours are ranked by the sum of their two largest c, all but the n_keep best are out (their c
    counts as -inf); the top c win, lowest index first among equals; weights s / (sum of the chosen s + 1e-20) * scale."""
    E = len(z)
    s = sigmoid(z)
    c = s + correction
    if n_group > 1 and n_keep < n_group:
        per = E // n_group
        score = [np.sort(c[g * per:(g + 1) * per])[-2:].sum() for g in range(n_group)]
        kept = sorted(range(n_group), key=lambda g: (-score[g], g))[:n_keep]
        c = np.array([c[e] if e // per in kept else -np.inf for e in range(E)])
    chosen = sorted(range(E), key=lambda e: (-c[e], e))[:top]
    w = s[chosen]
    return chosen, w / (w.sum() + 1e-20) * scale


def experts_ff(h, W, pre, mlp):
    r = mlp["router"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, w = route(W[pre + "router"] @ h[t], W[pre + "correction"], r["top"], gr["count"], gr["keep"], r["scale"])
        for e, we in zip(chosen, w):
            p = f"{pre}e{e}."
            out[t] += we * (W[p + "down"] @ (silu(W[p + "gate"] @ h[t]) * (W[p + "up"] @ h[t])))
    return out


# ------------------------------------------------------------------------------------------------ the model
def run_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def forward(cfg, W, tokens, residuals=None):
    """Logits [T, vocab] of one sequence from its first token on."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    for il in run_order(cfg):
        layer, pre = cfg["layers"][il], f"l{il}."
        h = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        if layer["type"] == "lightning":
            y = lightning_mixer(h, W, pre + "mix.", layer["mixer"], eps)
        else:
            y = attention_mixer(h, W, pre + "mix.", layer["mixer"], eps, layer["type"] == "attention_2")
        if layer.get("mlp") is not None:
            y = y + experts_ff(h, W, pre + "mlp.", layer["mlp"])
        x = x + y
        if residuals is not None:
            residuals.append(x.copy())
    z = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap") or 0.0
    return cap * np.tanh(z / cap) if cap > 0 else z


# ------------------------------------------------------------------------------------------------ small configurations and weights
def moe(ff=24, experts=6, top=2, groups=3, keep=2, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}}


def attn_layer(kind="attention", heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=1000.0, scaling=True, window=0, keep_first=0, scale=None, mlp="moe"):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale if scale is not None else 1.3 / math.sqrt(dim)}
    if window:
        mx["mask"] = {"size": window, "keep_first": keep_first}
    return {"type": kind, "mixer": mx, "mlp": moe() if mlp == "moe" else mlp}


def lightning_layer(heads=3, dim=8, vdim=12, decay=None, mlp="moe"):
    decay = decay if decay is not None else [0.5 + 0.49 * (i + 1) / heads for i in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": moe() if mlp == "moe" else mlp}


def make_config(layers, width=40, vocab=61, eps=1e-5, softcap=12.0, loop=None):
    cfg = {"architecture": "Galirax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_softcap": softcap, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0, gain=1.0):
    """bf16-representable float32 values, so that the served (bf16) and the exact (f32) modes read the same model."""
    rng = np.random.default_rng(seed)
    Wd, vocab = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, rows, cols, g=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)) * g * gain / math.sqrt(cols))

    def vec(name, n, mean=0.0, spread=0.3):
        W[name] = bf16_round(mean + spread * rng.standard_normal(n))

    W["embed"] = bf16_round(rng.standard_normal((vocab, Wd)))
    mat("head", vocab, Wd, 3.0)
    vec("final.norm", Wd, 1.0, 0.1); vec("final.norm.b", Wd, 0.0, 0.1)
    for il, layer in enumerate(cfg["layers"]):
        p, mx = f"l{il}.", layer["mixer"]
        vec(p + "norm1", Wd, 1.0, 0.1); vec(p + "norm1.b", Wd, 0.0, 0.1)
        if layer["type"] == "lightning":
            H, D, V = mx["heads"], mx["dim"], mx["vdim"]
            mat(p + "mix.q", H * D, Wd, 2.0); mat(p + "mix.k", H * D, Wd, 2.0); mat(p + "mix.v", H * V, Wd, 2.0); mat(p + "mix.g", H * V, Wd, 2.0)
            mat(p + "mix.o", Wd, H * V)
            vec(p + "mix.norm", H * V, 1.0, 0.2)
        else:
            H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            mat(p + "mix.q", H * D, Wd, 2.0); mat(p + "mix.k", G * D, Wd, 2.0); mat(p + "mix.v", G * V, Wd, 2.0)
            mat(p + "mix.o", Wd, H * V)
            vec(p + "mix.sink", H, 0.5, 1.0)
            if layer["type"] == "attention_2":
                vec(p + "mix.q.b", H * D); vec(p + "mix.k.b", G * D); vec(p + "mix.v.b", G * V)
                vec(p + "mix.q.norm", H * D, 1.0, 0.2); vec(p + "mix.k.norm", G * D, 1.0, 0.2)
        mlp = layer.get("mlp")
        if mlp is not None:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            mat(p + "mlp.router", E, Wd, 3.0)
            vec(p + "mlp.correction", E, 0.0, 0.3)
            for e in range(E):
                mat(f"{p}mlp.e{e}.gate", F, Wd, 2.0); mat(f"{p}mlp.e{e}.up", F, Wd, 2.0); mat(f"{p}mlp.e{e}.down", Wd, F, 2.0)
    return W


def as_tensors(W):
    """name -> (dtype, shape, raw bytes), the form the loader takes: matrices and vectors as bf16 bits."""
    out = {}
    for name, a in W.items():
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
        out[name] = ("BF16", tuple(a.shape), bits.view(np.uint8).reshape(-1))
    return out
