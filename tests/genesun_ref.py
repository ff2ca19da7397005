"""A plain, slow statement of the Genesun equations in numpy float64: one function per mechanism, token-by-token loops, no
caches, no fusion.  It shares no code with the package; the tests compare the library against it.

Notation: x [T, W] activations of one sequence, W_* matrices stored [out, in] and applied as x @ W.T.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return np.minimum(z, 0.0) - np.log1p(np.exp(-np.abs(z)))


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def polynorm(z, coef, eps):
    a, b, c, e = [float(v) for v in coef]
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def rotation_table(dims, base, scaling, positions):
    """cos, sin [len(positions), dims / 2] of the angles position * f_i, with the YaRN blend and magnitude when scaling is given."""
    i = np.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    if scaling:
        def turns_to_dim(t):
            return dims * math.log(scaling["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(turns_to_dim(scaling["fast"])), 0)
        hi = min(math.ceil(turns_to_dim(scaling["slow"])), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / scaling["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(scaling["factor"]) + 1.0
    ang = np.asarray(positions, dtype=F)[:, None] * f[None, :]
    return np.cos(ang) * mag, np.sin(ang) * mag


def rotate_interleaved(x, cos, sin, dims):
    """x [T, ..., n]: pairs (2i, 2i+1) of the first `dims` entries are rotated, the rest pass."""
    out = x.copy()
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = cos.reshape(shape), sin.reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, scale, sink, window=0):
    """q, k [T, H, n], v [T, H, m]; causal; the denominator also holds exp(sink[h]).  Token by token, head by head."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[-1]), dtype=F)
    for t in range(T):
        lo = 0 if window <= 0 else max(0, t - window + 1)
        for h in range(H):
            s = (k[lo:t + 1, h] @ q[t, h]) * scale
            mx = max(s.max(), sink[h]) if sink is not None else s.max()
            e = np.exp(s - mx)
            den = e.sum() + (math.exp(sink[h] - mx) if sink is not None else 0.0)
            out[t, h] = (e / den) @ v[lo:t + 1, h]
    return out


def latent_attention(W, p, mx, h, eps, shared):
    """h [T, width].  shared: dict layer -> (latent, rotated key part); this layer adds or reads its entry."""
    H, D, R, V, KR = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    rot = mx.get("rot") or {}
    dims = rot.get("dims", R)
    cos, sin = rotation_table(dims, rot.get("base", 10000.0), rot.get("scaling"), np.arange(T)) if dims else (None, None)
    cq = unit_rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    if dims:
        q_rot = rotate_interleaved(q_rot, cos, sin, dims)
    if mx.get("kv_from") is None:
        dkv = h @ W[p + "dkv"].T
        lat = unit_rms(dkv[:, :KR], eps) * W[p + "dkv.norm"]
        k_rot = dkv[:, KR:]
        if dims:
            k_rot = rotate_interleaved(k_rot, cos, sin, dims)
        shared[p] = (lat, k_rot)
    else:
        lat, k_rot = shared["l%d.mix." % mx["kv_from"]]
    k_plain = (lat @ W[p + "uk"].T).reshape(T, H, D)
    v = (lat @ W[p + "uv"].T).reshape(T, H, V)
    k = np.concatenate([k_plain, np.broadcast_to(k_rot[:, None, :], (T, H, R))], -1)
    o = sink_softmax_attention(np.concatenate([q_plain, q_rot], -1), k, v, mx["scale"], W[p + "sink"], mx.get("window") or 0)
    o = o.reshape(T, H * V) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def mlstm_recurrence(q, k, v, i_pre, f_pre, cap, state=None):
    """q, k [T, H, D] (q already scaled), v [T, H, V], gate pre-activations [T, H].  Returns o [T, H, V] and the final state."""
    T, H, D = q.shape
    V = v.shape[-1]
    if state is None:
        state = (np.zeros((H, D, V), F), np.zeros((H, D), F), np.zeros(H, F))
    S, n, m = [a.copy() for a in state]
    out = np.zeros((T, H, V), F)
    for t in range(T):
        li = cap * np.tanh(i_pre[t] / cap)
        lf = log_sigmoid(cap * np.tanh(f_pre[t] / cap))
        m_new = np.maximum(lf + m, li)
        a, b = np.exp(lf + m - m_new), np.exp(li - m_new)
        for hd in range(H):
            S[hd] = a[hd] * S[hd] + b[hd] * np.outer(k[t, hd], v[t, hd])
            n[hd] = a[hd] * n[hd] + b[hd] * k[t, hd]
            den = max(abs(n[hd] @ q[t, hd]), math.exp(-m_new[hd])) + 1e-6
            out[t, hd] = (S[hd].T @ q[t, hd]) / den
        m = m_new
    return out, (S, n, m)


def mlstm(W, p, mx, h, eps):
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    o, _ = mlstm_recurrence(q, k, v, h @ W[p + "i"].T + W[p + "i.b"], h @ W[p + "f"].T + W[p + "f.b"], mx["gate_cap"])
    o = unit_rms(o, eps).reshape(T, H * V) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def forward(cfg, W, tokens):
    """Logits [T, vocab] of one sequence."""
    W = {k: np.asarray(v, dtype=F) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    results, shared = [x], {}
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = layer_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention(W, p + "mix.", layer["mixer"], h, eps, shared)
        else:
            y = mlstm(W, p + "mix.", layer["mixer"], h, eps)
        y = y * sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + layer_norm(y, W[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            h = layer_norm(x, W[p + "norm2"], eps)
            y = polynorm(h @ W[p + "mlp.up"].T, W[p + "mlp.act"], eps) @ W[p + "mlp.down"].T
            y = y * sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + layer_norm(y, W[p + "norm2b"], eps)
        results.append(x)
        x = sum(W[p + "dwa"][j] * results[j] for j in range(i + 2))
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T


# ------------------------------------------------------------------------------------------------ random models
def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return u.view(np.float32)


def attn_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=32, q_rank=24, ff=48, kv_from=None, rot_dims=None, scaling=True, base=10000.0, window=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": 1.0 / math.sqrt(dim + rot_dim),
          "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if scaling:
        mx["rot"]["scaling"] = {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    if window:
        mx["window"] = window
    return {"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mlstm_layer(heads=2, dim=16, vdim=24, gate_cap=10.0, ff=0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, width=64, vocab=96, eps=1e-5):
    return {"architecture": "Genesun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def random_weights(cfg, seed=0, gain=1.0):
    """bf16-representable f32 weights under the design's tensor names."""
    rng = np.random.default_rng(seed)
    Wd, vocab = cfg["width"], cfg["vocab"]
    W = {}

    def mat(o, i, g=1.0):
        return bf16_round(rng.standard_normal((o, i)) * g * gain / math.sqrt(i))

    def vec(n, mean=1.0, sd=0.1):
        return bf16_round(mean + sd * rng.standard_normal(n))

    W["embed"] = bf16_round(rng.standard_normal((vocab, Wd)))
    W["head"] = mat(vocab, Wd)
    W["final.norm"] = vec(Wd)
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        mx = layer["mixer"]
        H, D, V = mx["heads"], mx["dim"], mx["vdim"]
        W[p + "norm1"], W[p + "norm1b"] = vec(Wd), vec(Wd)
        W[p + "rg1"], W[p + "rg1.b"] = mat(Wd, Wd), vec(Wd, 0.0, 0.5)
        W[p + "dwa"] = bf16_round(rng.uniform(0.2, 0.9, i + 2))
        if layer["type"] == "latent_attention":
            R, KR, QR = mx["rot_dim"], mx["kv_rank"], mx["q_rank"]
            W[p + "mix.dq"], W[p + "mix.dq.norm"], W[p + "mix.uq"] = mat(QR, Wd), vec(QR), mat(H * (D + R), QR, 2.0)
            if mx.get("kv_from") is None:
                W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = mat(KR + R, Wd), vec(KR)
            W[p + "mix.uk"], W[p + "mix.uv"] = mat(H * D, KR, 2.0), mat(H * V, KR)
            W[p + "mix.sink"] = bf16_round(rng.standard_normal(H))
            W[p + "mix.g"], W[p + "mix.o"] = mat(H * V, Wd), mat(Wd, H * V)
        else:
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * D, Wd), mat(H * D, Wd), mat(H * V, Wd)
            W[p + "mix.g"], W[p + "mix.o"], W[p + "mix.norm"] = mat(H * V, Wd), mat(Wd, H * V), vec(H * V)
            W[p + "mix.i"], W[p + "mix.i.b"] = mat(H, Wd, 2.0), vec(H, 0.0, 1.0)
            W[p + "mix.f"], W[p + "mix.f.b"] = mat(H, Wd, 2.0), vec(H, 2.0, 1.0)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            W[p + "norm2"], W[p + "norm2b"] = vec(Wd), vec(Wd)
            W[p + "rg2"], W[p + "rg2.b"] = mat(Wd, Wd), vec(Wd, 0.0, 0.5)
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(ff, Wd), mat(Wd, ff)
            W[p + "mlp.act"] = bf16_round(np.array([0.6, 0.3, 0.2, 0.05]) + 0.05 * rng.standard_normal(4))
    return W


def as_tensors(W):
    """The loader's input: name -> (dtype, shape, raw bytes)."""
    return {k: ("F32", tuple(v.shape), np.ascontiguousarray(v, dtype=np.float32).view(np.uint8).reshape(-1)) for k, v in W.items()}
