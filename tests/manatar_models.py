"""Small Manatar models for the tests: configurations of the tests' own, random weights of the tests' own making.

None of the configurations is anybody's model.  Between them they vary what a single model would make equal or 1: query against
key-value heads (1:1, 2:1, 3:1), key against value sizes, fewer turned values than a head has, rotations with and without rescaled
frequencies, taps (none, 2, 3, 4), layers that read another layer's cached keys and values, mLSTM key sizes that are no multiple of
four, experts of which one, some or all are chosen, with and without the shared one, layers without a feed-forward, a residual
multiplier of 1 and others, models without the hashed second embedding row, sizes the tensor-core kernels take and sizes they refuse.
"""
import json
import os

import numpy as np
import torch


def rot(base, dims, scaling=None):
    r = dict(base=base, dims=dims)
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def att(heads, kv, dim, vdim, conv, diff, scale, rotation, kv_from=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, diff=diff, scale=scale)
    if conv:
        m["conv"] = conv
    if rotation is not None:
        m["rot"] = rotation
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mem(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(ff, experts, top, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared is not None:
        d["shared"] = dict(ff=shared)
    return d


def layer(kind, mixer, mlp=None):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def config(vocab, width, layers, *, eps=1e-5, mult=1.0, bigram=(53, 7, 3)):
    c = dict(architecture="Manatar", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, layers=layers)
    if bigram is not None:
        c["embedding"] = dict(bigram=dict(zip(("buckets", "mul_prev", "mul_cur"), bigram)))
    return c


ROT_A = rot(10000.0, 8, (4.0, 64, 8.0, 1.0))
ROT_B = rot(300.0, 16, (1.5, 40, 16.0, 2.0))
# every kind of layer, a layer that reads the rows of layer 0 and one that reads those of layer 3, grouped heads
CFG_ALL = config(97, 64, [layer("attention", att(4, 2, 16, 24, 3, 0.25, 0.3, ROT_A), dense(96, 1.5)),
                          layer("mlstm", mem(2, 16, 32, 8.0), moe(24, 5, 2, 40)),
                          layer("attention", att(2, 2, 16, 24, 3, 0.25, 0.3, ROT_A, kv_from=0), moe(16, 4, 1)),
                          layer("attention", att(6, 2, 8, 16, 2, 0.4, 0.5, rot(500.0, 8)), None),
                          layer("mlstm", mem(4, 8, 16, 3.0), dense(72, 0.8)),
                          layer("attention", att(2, 2, 8, 16, 4, 0.1, 0.35, rot(500.0, 8), kv_from=3), moe(24, 3, 3, 24))],
                 mult=0.4, bigram=(101, 31, 17))
# odd sizes that only the general kernels take; no rescaling, fewer turned values than a head has, one layer with neither
# convolution nor rotation, no second embedding row, a multiplier of 1
CFG_ODD = config(61, 40, [layer("mlstm", mem(3, 10, 7, 15.0)),
                          layer("attention", att(3, 3, 10, 14, 2, 0.3, 0.4, rot(50.0, 4)), moe(12, 7, 3)),
                          layer("attention", att(3, 1, 6, 10, 0, 0.5, 0.6, None), dense(56, 3.0)),
                          layer("mlstm", mem(1, 22, 12, 2.0), moe(20, 2, 2, 8))], eps=1e-6, bigram=None)
# wider heads, tensor-core sizes, several layers reading one layer's rows
CFG_WIDE = config(83, 128, [layer("attention", att(4, 1, 64, 64, 4, 0.2, 0.125, ROT_B), moe(64, 8, 2, 128)),
                            layer("attention", att(2, 1, 64, 64, 2, 0.35, 0.125, ROT_B, kv_from=0)),
                            layer("mlstm", mem(2, 64, 128, 15.0), dense(256, 2.0)),
                            layer("attention", att(8, 1, 64, 64, 3, 0.2, 0.2, ROT_B, kv_from=0), dense(128, 1.0))],
                  mult=0.3, bigram=(257, 5, 11))

CONFIGS = {"all": CFG_ALL, "odd": CFG_ODD, "wide": CFG_WIDE}


def make_tensors(cfg, seed, sharp=1.0):
    """name -> float32 array, drawn so that every mechanism matters: biases and norm weights away from 0 and 1, scores of order one
    and more, the feed-forwards' clamps reached by a good part of the values, router logits apart, gates on both sides of their
    caps, the two lambda vectors large enough to move lambda away from `diff`."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    n = lambda *shape, std=1.0: (rng.standard_normal(shape) * std).astype(np.float32)
    t = {"embed": n(cfg["vocab"], W, std=0.8), "head": n(cfg["vocab"], W, std=1.5 * W ** -0.5), "final.norm": 1 + n(W, std=0.15)}
    big = (cfg.get("embedding") or {}).get("bigram")
    if big is not None:
        t["bigram"] = n(big["buckets"] + 1, W, std=0.6)

    def gated(p, ff, std):
        t[p + "gate"], t[p + "up"], t[p + "down"] = n(ff, W, std=std * W ** -0.5), n(ff, W, std=std * W ** -0.5), n(W, ff, std=ff ** -0.5)

    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        t[p + "norm1"] = 1 + n(W, std=0.2)
        if l["type"] == "attention":
            H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            names = [("q", H * 2 * dim)] + ([("k", G * 2 * dim), ("v", G * vdim)] if "kv_from" not in m else [])
            for name, rows in names:
                t[f"{p}mix.{name}"] = n(rows, W, std=sharp * 1.5 * W ** -0.5)
                t[f"{p}mix.{name}.b"] = n(rows, std=0.3)
                if m.get("conv"):
                    t[f"{p}mix.{name}.conv"] = n(rows, m["conv"], std=0.7)
            t[p + "mix.q.norm"] = sharp * (1.5 + n(dim, std=0.2))
            if "kv_from" not in m:
                t[p + "mix.k.norm"] = 1.5 + n(dim, std=0.2)
            for name in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + name] = n(dim, std=0.6 * dim ** -0.25)
            t[p + "mix.g"] = n(H * vdim, W, std=2 * W ** -0.5)
            t[p + "mix.o"] = n(W, H * vdim, std=(H * vdim) ** -0.5)
            t[p + "mix.o.b"] = n(W, std=0.2)
        else:
            H, dim, vdim = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = n(H * dim, W, std=2 * W ** -0.5), n(H * dim, W, std=2 * W ** -0.5)
            t[p + "mix.v"], t[p + "mix.g"] = n(H * vdim, W, std=W ** -0.5), n(H * vdim, W, std=2 * W ** -0.5)
            t[p + "mix.i"], t[p + "mix.f"] = n(H, W, std=3 * W ** -0.5), n(H, W, std=3 * W ** -0.5)
            t[p + "mix.i.b"], t[p + "mix.f.b"] = n(H, std=1.0), 2.0 + n(H, std=1.5)
            t[p + "mix.norm"] = 1 + n(H * vdim, std=0.15)
            t[p + "mix.o"] = n(W, H * vdim, std=(H * vdim) ** -0.5)
        ff = l["mlp"]
        if ff is None:
            continue
        t[p + "norm2"] = 1 + n(W, std=0.2)
        if ff["kind"] == "dense":
            gated(p + "mlp.", ff["ff"], 2.0)
        else:
            for e in range(ff["router"]["experts"]):
                gated(f"{p}mlp.e{e}.", ff["expert"]["ff"], 1.5)
            t[p + "mlp.router"] = n(ff["router"]["experts"], W, std=2 * W ** -0.5)
            t[p + "mlp.router.b"] = n(ff["router"]["experts"], std=0.5)
            if ff.get("shared") is not None:
                gated(p + "mlp.shared.", ff["shared"]["ff"], 1.5)
    return t


def write_model(model_dir, cfg, tensors, dtype=torch.bfloat16):
    """config.json and model.safetensors; tensors are stored in `dtype` (the values a bfloat16 checkpoint holds are what
    both the engine and the plain implementation then read)."""
    from vitna_anchor_b200.weights import write_model_folder
    os.makedirs(model_dir, exist_ok=True)
    write_model_folder(str(model_dir), cfg, {k: torch.from_numpy(v).to(dtype) for k, v in tensors.items()})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return str(model_dir)


def make_model(model_dir, name, seed=0, **kw):
    return write_model(model_dir, CONFIGS[name], make_tensors(CONFIGS[name], seed, **kw))
