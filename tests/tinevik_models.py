"""Small Tinevik models for the tests: configurations of the tests' own, random weights of the tests' own making.

None of the configurations is anybody's model.  Between them they vary what a single model would make equal or 1: query against
key-value heads (1:1, 2:1, 3:1, 4:1), key against value sizes, fewer turned values than a head has, rotations with and without
divided frequencies, attention without a cap or without a rotation, windows shorter and longer than a page and than a prompt, latent
ranks above and below the heads' sizes, decays' ranks, experts of which one, some or all are a token's, layers without a feed-forward,
layers that run with another layer's tensors (an earlier and a later one), scales of the embedding and the logits of 1 and others,
sizes the tensor-core kernels take and sizes they refuse.
"""
import json
import os

import numpy as np
import torch


def gla(heads, dim, vdim, tau):
    return dict(heads=heads, dim=dim, vdim=vdim, tau=tau)


def att(heads, kv, dim, vdim, scale, softcap=None, rot=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = rot
    return m


def rot(base, dims, factor=None):
    r = dict(base=base, dims=dims)
    if factor is not None:
        r["scaling"] = dict(factor=factor)
    return r


def lat(heads, dim, vdim, kv_rank, q_rank, scale, window=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale)
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, limit, experts, top):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


def layer(kind, mixer, mlp=None, weights_of=None):
    d = dict(type=kind, mixer=mixer, mlp=mlp)
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def config(vocab, width, layers, *, eps=1e-5, embed_scale=1.0, logit_scale=1.0):
    return dict(architecture="Tinevik", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=embed_scale),
                logit_scale=logit_scale, layers=layers)


_G1, _A1, _L1 = gla(2, 16, 24, 4.0), att(4, 2, 16, 24, 0.3, 20.0, rot(10000.0, 8, 4.0)), lat(3, 8, 12, 16, 24, 0.4, 21)
# every kind of layer and of feed-forward; layers 4 and 5 run with the tensors of layers 0 and 2, layer 3's window is longer than a page
CFG_ALL = config(97, 64, [layer("gla", _G1, dense(96)),
                          layer("latent_attention", _L1, moe(24, 1.2, 5, 2)),
                          layer("attention", _A1, moe(16, 0.8, 4, 1)),
                          layer("latent_attention", lat(2, 16, 8, 8, 8, 0.3, 5), None),
                          layer("gla", _G1, dense(96), weights_of=0),
                          layer("attention", _A1, moe(16, 0.8, 4, 1), weights_of=2)],
                 embed_scale=1.7, logit_scale=0.6)
# odd sizes that only the general kernels take; an attention without cap, one without a rotation, a latent layer without a window, a
# layer that runs with a LATER layer's tensors, scales of 1
CFG_ODD = config(61, 40, [layer("gla", gla(3, 10, 7, 1.0), moe(12, 2.0, 7, 3), weights_of=3),
                          layer("attention", att(3, 3, 10, 14, 0.4, None, rot(50.0, 4)), dense(56)),
                          layer("attention", att(3, 1, 6, 10, 0.6, 7.0, None), None),
                          layer("gla", gla(3, 10, 7, 1.0), moe(12, 2.0, 7, 3)),
                          layer("latent_attention", lat(5, 6, 10, 12, 20, 0.5), moe(20, 1.0, 2, 2))], eps=1e-6)
# wider heads, tensor-core sizes, a window of several pages, the whole head turned
CFG_WIDE = config(83, 128, [layer("attention", att(4, 1, 64, 64, 0.125, 30.0, rot(200000.0, 64, 8.0)), moe(64, 1.25, 8, 2)),
                            layer("gla", gla(2, 64, 128, 12.0), dense(256)),
                            layer("latent_attention", lat(4, 32, 64, 64, 96, 0.18, 50), dense(128)),
                            layer("gla", gla(4, 32, 32, 8.0), moe(64, 1.25, 8, 2))],
                  embed_scale=11.3, logit_scale=2.0)

CONFIGS = {"all": CFG_ALL, "odd": CFG_ODD, "wide": CFG_WIDE}


def make_tensors(cfg, seed, rank=5):
    """name -> float32 array (int32 for the experts' tables), drawn so that every mechanism matters: biases and norm weights away
    from 0 and 1, scores of order one and more (so the cap bends them), a mixing matrix that is far from the identity, decays spread
    between fast and slow, the experts' clamps reached by a good part of the values, activations on both sides of zero."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    n = lambda *shape, std=1.0: (rng.standard_normal(shape) * std).astype(np.float32)
    scale = (cfg.get("embedding") or {}).get("scale", 1.0)
    t = {"embed": n(V, W, std=0.8 / scale), "final.norm": 1 + n(W, std=0.15), "final.norm.b": n(W, std=0.1)}
    for i, l in enumerate(cfg["layers"]):
        if l.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", l["mixer"]
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if l["mlp"] is not None else ()):
            t[p + name] = (0.6 if name.endswith("b") else 1.0) + n(W, std=0.2)
            t[p + name + ".b"] = n(W, std=0.1)
        if l["type"] == "gla":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = n(H * dk, W, std=2 * W ** -0.5), n(H * dk, W, std=2 * W ** -0.5)
            t[p + "mix.v"], t[p + "mix.g"] = n(H * dv, W, std=W ** -0.5), n(H * dv, W, std=2 * W ** -0.5)
            t[p + "mix.a1"], t[p + "mix.a2"] = n(rank, W, std=2 * W ** -0.5), n(H * dk, rank, std=2 * rank ** -0.5)
            t[p + "mix.a2.b"] = 1.0 + n(H * dk, std=2.0)
            t[p + "mix.norm"] = 1 + n(dv, std=0.15)
            t[p + "mix.o"] = n(W, H * dv, std=(H * dv) ** -0.5)
        elif l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = n(H * dk, W, std=W ** -0.5), n(G * dk, W, std=W ** -0.5)
            t[p + "mix.v"] = n(G * dv, W, std=1.5 * W ** -0.5)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = 1.5 + n(dk, std=0.2), 1.5 + n(dk, std=0.2)
            t[p + "mix.talk"] = (np.eye(H) * 0.8 + rng.standard_normal((H, H)) * 0.4).astype(np.float32)
            t[p + "mix.o"] = n(W, H * dv, std=(H * dv) ** -0.5)
        else:
            H, dk, dv, rk, rq = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = n(rq, W, std=W ** -0.5), 1 + n(rq, std=0.2)
            t[p + "mix.uq"] = n(H * dk, rq, std=2 * rq ** -0.5)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = n(rk, W, std=W ** -0.5), 1 + n(rk, std=0.2)
            t[p + "mix.uk"], t[p + "mix.uv"] = n(H * dk, rk, std=2 * rk ** -0.5), n(H * dv, rk, std=1.5 * rk ** -0.5)
            t[p + "mix.g"] = n(H * dv, W, std=2 * W ** -0.5)
            t[p + "mix.o"] = n(W, H * dv, std=(H * dv) ** -0.5)
        ff = l["mlp"]
        if ff is None:
            continue
        if ff["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = n(ff["ff"], W, std=2 * W ** -0.5), n(W, ff["ff"], std=ff["ff"] ** -0.5)
            t[p + "mlp.act"] = n(2, std=1.0)
        else:
            E, top, f = ff["router"]["experts"], ff["router"]["top"], ff["expert"]["ff"]
            for e in range(E):
                q = f"{p}mlp.e{e}."
                t[q + "gate"], t[q + "up"], t[q + "down"] = n(f, W, std=1.5 * W ** -0.5), n(f, W, std=1.5 * W ** -0.5), n(W, f, std=f ** -0.5)
            t[p + "mlp.table"] = np.stack([rng.permutation(E)[:top] for _ in range(V)]).astype(np.int32)
    return t


def write_model(model_dir, cfg, tensors, dtype=torch.bfloat16):
    """config.json and model.safetensors; floating tensors are stored in `dtype` (the values a bfloat16 checkpoint holds are what
    both the engine and the plain implementation then read), tables as int32."""
    from vitna_anchor_b200.weights import write_model_folder
    os.makedirs(model_dir, exist_ok=True)
    write_model_folder(str(model_dir), cfg, {k: torch.from_numpy(v) if v.dtype == np.int32 else torch.from_numpy(v).to(dtype)
                                             for k, v in tensors.items()})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return str(model_dir)


def make_model(model_dir, name, seed=0, **kw):
    return write_model(model_dir, CONFIGS[name], make_tensors(CONFIGS[name], seed, **kw))
