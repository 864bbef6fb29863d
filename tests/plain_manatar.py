"""A plain, slow statement of the Manatar decoder in NumPy: whole sequences, no cache, one function per mechanism.

It shares nothing with the engine: its own reader of config.json and model.safetensors, its own arithmetic
(float64, so that it is the sharper side of every comparison).

Notation.  T tokens of one sequence at positions 0..T-1; W the width; m the residual multiplier.  A layer is
x += m rms(mixer(x)) w1, then (unless its configuration says null) x += m rms(ff(x)) w2: the sublayers read x as it is and
the norm sits on what they give.

  embedding     x_t = E[id_t] + B[(id_(t-1) a + id_t b) mod n]   (B[n] for t = 0)
  attention     two score maps a head over shared values: q, k, v = conv(W h + b) (short causal convolution a channel);
                q, k per head and map: rms with a shared weight, then pairs (2i, 2i+1) of the first `dims` values turned by
                p f_i; softmax(scale q.k) v for each map; o = a1 - lambda a2, lambda = exp(lq1.lk1) - exp(lq2.lk2) + diff;
                o / rms(o) (1 - diff); times sigmoid(W_g h); W_o (+ b).  A layer may read another layer's k and v.
  mlstm         per head a matrix S and a vector n with a running maximum of the gates' logarithms; see mlstm().
  feed-forward  dense: g = min(W_g h, L), u = clamp(W_u h, -L, L), W_d (g sigmoid(1.702 g) (u + 1));
                experts: the `top` largest router logits choose, softmax over the chosen, each expert W_d (silu(W_g h) W_u h),
                plus a shared expert of the same form for every token.
  output        head (rms(x) w)
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_tensors(path):
    """name -> array (float64 for floating tensors, int64 for integer ones)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    directory = json.loads(raw[8:8 + n].decode("utf-8"))
    out = {}
    for name, d in directory.items():
        if name == "__metadata__":
            continue
        lo, hi = d["data_offsets"]
        blob = raw[8 + n + lo:8 + n + hi]
        if d["dtype"] == "BF16":
            a = (np.frombuffer(blob, "<u2").astype(np.uint32) << 16).view("<f4").astype(np.float64)
        elif d["dtype"] == "F32":
            a = np.frombuffer(blob, "<f4").astype(np.float64)
        elif d["dtype"] == "I32":
            a = np.frombuffer(blob, "<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {d['dtype']}")
        out[name] = a.reshape(d["shape"])
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_tensors(os.path.join(model_dir, "model.safetensors"))


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def embed(cfg, w, ids):
    x = w["embed"][ids].copy()
    big = (cfg.get("embedding") or {}).get("bigram")
    if big is None:
        return x
    n = big["buckets"]
    for t, tok in enumerate(ids):
        row = n if t == 0 else (int(ids[t - 1]) * big["mul_prev"] + int(tok) * big["mul_cur"]) % n
        x[t] += w["bigram"][row]
    return x


def short_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    if taps_w is None:
        return u
    T, C = u.shape
    taps = taps_w.shape[1]
    y = np.zeros_like(u)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            y[shift:] += u[:T - shift] * taps_w[:, j]
    return y


def frequencies(rot):
    """(f [dims/2], factor on cos and sin)."""
    dims, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = sc["factor"], sc["original"]
    where = lambda t: dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, rot):
    """x [T, n, d]: the first rot.dims values of every row turned pairwise (2i, 2i+1) by position * f_i."""
    if not rot or not rot["dims"]:
        return x
    f, mag = frequencies(rot)
    dims = rot["dims"]
    T = x.shape[0]
    ang = np.arange(T)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def attention_kv(w, p, m, h, eps):
    """The layer's keys (after convolution, norm and rotation) [T, G, 2, dim] and values (after convolution) [T, G, vdim]."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = short_conv(h @ w[p + "k"].T + w[p + "k.b"], w.get(p + "k.conv")).reshape(T, G * 2, dim)
    v = short_conv(h @ w[p + "v"].T + w[p + "v.b"], w.get(p + "v.conv")).reshape(T, G, vdim)
    k = rotate(rms(k, eps) * w[p + "k.norm"], m.get("rot")).reshape(T, G, 2, dim)
    return k, v


def attention(w, p, m, h, eps, kv):
    T = h.shape[0]
    H, G, dim, vdim, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    q = short_conv(h @ w[p + "q"].T + w[p + "q.b"], w.get(p + "q.conv")).reshape(T, H * 2, dim)
    q = rotate(rms(q, eps) * w[p + "q.norm"], m.get("rot")).reshape(T, H, 2, dim)
    k, v = kv
    lam = math.exp(float(w[p + "lq1"] @ w[p + "lk1"])) - math.exp(float(w[p + "lq2"] @ w[p + "lk2"])) + diff
    mask = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, vdim))
    for hh in range(H):
        g = hh // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hh, mp] @ k[:, g, mp].T) * m["scale"]
            s = np.where(mask, s, -np.inf)
            e = np.exp(s - s.max(axis=1, keepdims=True))
            a.append((e / e.sum(axis=1, keepdims=True)) @ v[:, g])
        out[:, hh] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    out = out.reshape(T, H * vdim) * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T + w[p + "o.b"]


def mlstm(w, p, m, h, eps):
    T = h.shape[0]
    H, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dim)
    v = (h @ w[p + "v"].T).reshape(T, H, vdim)
    ig = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    z = cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap)
    fg = -np.logaddexp(0.0, -z)                      # log sigmoid
    out = np.zeros((T, H, vdim))
    for hh in range(H):
        S, n, mx = np.zeros((dim, vdim)), np.zeros(dim), 0.0
        for t in range(T):
            m_new = max(fg[t, hh] + mx, ig[t, hh])
            a, b = math.exp(fg[t, hh] + mx - m_new), math.exp(ig[t, hh] - m_new)
            S = a * S + b * np.outer(k[t, hh], v[t, hh])
            n = a * n + b * k[t, hh]
            mx = m_new
            out[t, hh] = (S.T @ q[t, hh]) / (max(abs(float(n @ q[t, hh])), math.exp(-mx)) + 1e-6)
    out = rms(out, eps).reshape(T, H * vdim) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def dense_ff(w, p, mlp, h):
    L = mlp["limit"]
    g = np.minimum(h @ w[p + "gate"].T, L)
    u = np.clip(h @ w[p + "up"].T, -L, L)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def expert(w, p, h):
    g = h @ w[p + "gate"].T
    return (g * sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe_ff(w, p, mlp, h):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = np.argsort(-z[t], kind="stable")[:top]
        e = np.exp(z[t, chosen] - z[t, chosen].max())
        e /= e.sum()
        for wt, ex in zip(e, chosen):
            out[t] += wt * expert(w, f"{p}e{ex}.", h[t:t + 1])[0]
    if mlp.get("shared") is not None:
        out += expert(w, p + "shared.", h)
    return out


def forward(cfg, w, ids, layers_out=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the residual stream after every layer."""
    ids = np.asarray(ids, dtype=np.int64)
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = embed(cfg, w, ids)
    kvs = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kvs[i] = attention_kv(w, p, m, x, eps)
            y = attention(w, p, m, x, eps, kvs[i if m.get("kv_from") is None else m["kv_from"]])
        elif layer["type"] == "mlstm":
            y = mlstm(w, p, m, x, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms(y, eps) * w[f"l{i}.norm1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(w, f"l{i}.mlp.", mlp, x) if mlp["kind"] == "dense" else moe_ff(w, f"l{i}.mlp.", mlp, x)
            x = x + mult * rms(y, eps) * w[f"l{i}.norm2"]
        if layers_out is not None:
            layers_out.append(x.copy())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T
