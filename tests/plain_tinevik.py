"""A plain, slow statement of the Tinevik decoder in NumPy: whole sequences, no cache, one function per mechanism.

It shares nothing with the engine: its own reader of config.json and model.safetensors, its own arithmetic
(float64, so that it is the sharper side of every comparison).

Notation.  T tokens of one sequence at positions 0..T-1; W the width.  LN(x; w, b) = (x - mean) / sqrt(var + eps) w + b and
rms(x) = x / sqrt(mean(x^2) + eps), eps = norm.eps.  A layer is

    x += LN1b(mixer(LN1(x)))        then (unless its configuration says null)        x += LN2b(ff(LN2(x)))

and a layer whose entry names `weights_of: j` runs with layer j's tensors.

  embedding     x_t = s E[id_t]
  gla           per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q scaled by dim^-1/2 and
                a = sigmoid(W_a2 W_a1 h + b)^(1/tau) per key channel; rms(o) w per head, times silu(W_g h), then W_o
  attention     q, k per head: rms with a shared weight, then the first `dims` values turned in pairs (i, i + dims/2) by
                p f_i / factor, f_i = base^(-2i/dims); v_j turned over all its pairs (m, m + vdim/2) by j base^(-2m/vdim);
                z = cap tanh(scale q.k / cap); the heads' scores mixed by a matrix, z'_h = sum_g M[h, g] z_g; causal softmax;
                the weighted sum of the turned values turned back by the query's position; W_o
  latent        c_q = rms(W_dq h) w, q = W_uq c_q; c = rms(W_dkv h) w; k = W_uk c, v = W_uv c per head; softmax(scale q.k) over
                the last `size` positions; heads side by side times sigmoid(W_g h); W_o
  feed-forward  dense: W_d f(W_u h), f(z) = softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (e^z - 1 - z) + z/2 otherwise;
                experts: a table gives each token id its `top` experts, each weighted 1/top; an expert is
                W_d (g sigmoid(1.702 g) (u + 1)), g = min(W_g h, L), u = clamp(W_u h, -L, L)
  output        logits = c E LN(x)
"""
from __future__ import annotations

import json
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


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    d = x - mu
    return d / np.sqrt(np.mean(d * d, axis=-1, keepdims=True) + eps) * w + b


def turn_halves(x, pos, freq, sign=1.0):
    """x [..., T, n]; pairs (i, i + len(freq)) of the first 2 len(freq) values are turned by sign * pos * freq_i."""
    r = len(freq)
    ang = sign * np.asarray(pos, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang), np.sin(ang)
    out = x.copy()
    u, v = x[..., :r], x[..., r:2 * r]
    out[..., :r] = u * c - v * s
    out[..., r:2 * r] = v * c + u * s
    return out


def frequencies(base, dims):
    return base ** (-2.0 * np.arange(dims // 2) / dims)


def gla(w, p, m, h, eps):
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    a = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, dk)
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = rms(o, eps) * w[p + "norm"]
    g = h @ w[p + "g"].T
    return (o.reshape(T, H * dv) * (g * sigmoid(g))) @ w[p + "o"].T


def attention(w, p, m, h, eps):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = np.arange(T)
    q = rms((h @ w[p + "q"].T).reshape(T, H, dk), eps) * w[p + "q.norm"]
    k = rms((h @ w[p + "k"].T).reshape(T, G, dk), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    rot = m.get("rot")
    q, k, v = q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2)            # [heads, T, n]
    vf = None
    if rot is not None:
        f = frequencies(rot["base"], rot["dims"])
        if rot.get("scaling") is not None:
            f = f / rot["scaling"]["factor"]
        q, k = turn_halves(q, pos, f), turn_halves(k, pos, f)
        vf = frequencies(rot["base"], dv)
        v = turn_halves(v, pos, vf)
    z = np.stack([q[hh] @ k[hh // (H // G)].T for hh in range(H)]) * m["scale"]         # [H, T, T]
    if m.get("softcap") is not None:
        z = m["softcap"] * np.tanh(z / m["softcap"])
    if p + "talk" in w:
        z = np.einsum("hg,gij->hij", w[p + "talk"], z)
    mask = pos[None, :] <= pos[:, None]
    z = np.where(mask[None], z, -np.inf)
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    pr = e / e.sum(axis=-1, keepdims=True)
    o = np.stack([pr[hh] @ v[hh // (H // G)] for hh in range(H)])                         # [H, T, dv]
    if vf is not None:
        o = turn_halves(o, pos, vf, sign=-1.0)
    return o.transpose(1, 0, 2).reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(w, p, m, h, eps):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = np.arange(T)
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dk)
    c = rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).reshape(T, H, dk)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    z = np.einsum("ihd,jhd->hij", q, k) * m["scale"]
    d = pos[:, None] - pos[None, :]
    mask = d >= 0
    if m.get("mask") is not None:
        mask &= d < m["mask"]["size"]
    z = np.where(mask[None], z, -np.inf)
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    pr = e / e.sum(axis=-1, keepdims=True)
    o = np.einsum("hij,jhd->ihd", pr, v).reshape(T, H * dv)
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def xielu(z, p, q):
    neg = np.minimum(z, 0.0)
    return np.where(z > 0, softplus(p) * z * z + z / 2, (0.5 + softplus(q)) * (np.expm1(neg) - neg) + z / 2)


def dense_ff(w, p, h):
    a = w[p + "act"]
    return xielu(h @ w[p + "up"].T, a[0], a[1]) @ w[p + "down"].T


def expert(w, p, L, h):
    g = np.minimum(h @ w[p + "gate"].T, L)
    u = np.clip(h @ w[p + "up"].T, -L, L)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def table_experts(w, p, mlp, h, ids):
    top, L = mlp["router"]["top"], mlp["expert"]["limit"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in w[p + "table"][ids[t]][:top]:
            out[t] += expert(w, f"{p}e{int(e)}.", L, h[t:t + 1])[0] / top
    return out


MIXERS = {"gla": gla, "attention": attention, "latent_attention": latent_attention}


def forward(cfg, w, ids, layers_out=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the residual stream after every layer."""
    ids = np.asarray(ids, dtype=np.int64)
    eps = cfg["norm"]["eps"]
    scale = (cfg.get("embedding") or {}).get("scale", 1.0)
    x = w["embed"][ids] * scale
    for i, layer in enumerate(cfg["layers"]):
        j = layer.get("weights_of", i)
        n = lambda name, v: layer_norm(v, w[f"l{j}.{name}"], w[f"l{j}.{name}.b"], eps)
        x = x + n("norm1b", MIXERS[layer["type"]](w, f"l{j}.mix.", layer["mixer"], n("norm1", x), eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            h = n("norm2", x)
            y = dense_ff(w, f"l{j}.mlp.", h) if mlp["kind"] == "dense" else table_experts(w, f"l{j}.mlp.", mlp, h, ids)
            x = x + n("norm2b", y)
        if layers_out is not None:
            layers_out.append(x.copy())
    xn = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return xn @ w["embed"].T * cfg.get("logit_scale", 1.0)
