"""Manatar on the CPU: the configuration reader, the manifest, which run reads whose cache, and the plain implementation's own pieces."""
import copy
import math

import numpy as np
import pytest

import manatar_models as MM
import plain_manatar as PM
from vitna_anchor_b200.config import ConfigError, resolve
from vitna_anchor_b200.config.manatar import DiffAttentionSpec, ManatarConfig
from vitna_anchor_b200.models.manatar import manatar_manifest
from vitna_anchor_b200.parts.diff_attention import DiffAttention
from vitna_anchor_b200.parts.rotary import blended_frequencies


@pytest.mark.parametrize("name", sorted(MM.CONFIGS))
def test_config_reads_back_and_names_every_tensor(name):
    cj = MM.CONFIGS[name]
    arch = resolve(cj)
    assert arch.name == "Manatar"
    cfg = arch.parse_config(cj)
    assert ManatarConfig.from_dict(cfg.to_dict()) == cfg
    made = MM.make_tensors(cj, 0)
    specs = {w.name: w for w in manatar_manifest(cfg)}
    assert set(specs) == set(made)
    for n, t in made.items():
        assert specs[n].fits(t.shape), n


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(window=7), "window"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),         # layer 1 is no attention layer
    (lambda c: c["layers"][5]["mixer"].update(kv_from=2), "kv_from"),         # layer 2 has no keys of its own
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),         # a later layer
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "vdim"),               # rows are read as the other layer wrote them
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=40), "dims"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
])
def test_what_the_engine_does_not_have_is_refused_by_name(change, word):
    cj = copy.deepcopy(MM.CONFIGS["all"])
    change(cj)
    with pytest.raises(ConfigError, match=word):
        ManatarConfig.from_dict(cj)


def test_sizes_that_may_be_left_out():
    cj = copy.deepcopy(MM.CONFIGS["odd"])
    m = cj["layers"][1]["mixer"]
    del m["kv_heads"], m["vdim"]
    del cj["residual_mult"]
    cfg = ManatarConfig.from_dict(cj)
    a = cfg.layers[1].mixer
    assert isinstance(a, DiffAttentionSpec) and (a.kv_heads, a.vdim) == (a.heads, a.dim)
    assert cfg.residual_mult == 1.0 and cfg.bigram is None
    assert cfg.layers[2].mixer.conv == 0 and cfg.layers[2].mixer.rot is None and cfg.layers[0].mlp is None


def test_frequencies_of_a_rescaled_rotation():
    """The rescaled frequencies against the recipe worked out by hand for one case, and against the plain implementation for the
    tests' rotations; without rescaling they are the powers of the base."""
    f, mag = blended_frequencies(100.0, 8, (4.0, 50, 4.0, 1.0))
    at = lambda turns: 8 * math.log(50 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(at(4.0)), 0), min(math.ceil(at(1.0)), 7)
    assert (lo, hi) == (0, 2)
    plain = [100.0 ** (-2 * i / 8) for i in range(4)]
    ramp = [0.0, 0.5, 1.0, 1.0]
    assert np.allclose(f, [p / 4.0 * r + p * (1 - r) for p, r in zip(plain, ramp)], rtol=1e-6)
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    for rot in (MM.ROT_A, MM.ROT_B, MM.rot(500.0, 8)):
        sc = rot.get("scaling")
        f, mag = blended_frequencies(rot["base"], rot["dims"], None if sc is None else (sc["factor"], sc["original"], sc["fast"], sc["slow"]))
        pf, pmag = PM.frequencies(rot)
        assert np.allclose(f, pf, rtol=1e-6) and mag == pytest.approx(pmag)
    f, mag = blended_frequencies(500.0, 8)
    assert mag == 1.0 and np.allclose(f, [1.0, 500 ** -0.25, 500 ** -0.5, 500 ** -0.75], rtol=1e-6)
    # a ramp whose ends meet: the step from kept to divided frequencies
    f, _ = blended_frequencies(100.0, 8, (2.0, 50, 1.0, 1.0))
    assert np.allclose(f[:2], plain[:2], rtol=1e-6) and np.allclose(f[2:], [p / 2 for p in plain[2:]], rtol=1e-6)


def test_lambda_of_a_layer():
    rng = np.random.default_rng(0)
    import torch
    a, b, c, d = (rng.standard_normal(12) * 0.4 for _ in range(4))
    got = DiffAttention.lambda_of(*(torch.tensor(v) for v in (a, b, c, d)), 0.3)
    assert got == pytest.approx(math.exp(a @ b) - math.exp(c @ d) + 0.3, rel=1e-5)


def test_plain_short_convolution_and_embedding():
    u = np.arange(10, dtype=np.float64).reshape(5, 2) + 1
    w = np.array([[1.0, 10.0, 100.0], [0.5, 0.0, 2.0]])
    y = PM.short_conv(u, w)
    assert y[0].tolist() == [100.0 * u[0, 0], 2.0 * u[0, 1]]                          # zeros before the start
    assert y[3, 0] == u[1, 0] + 10 * u[2, 0] + 100 * u[3, 0] and y[3, 1] == 0.5 * u[1, 1] + 2 * u[3, 1]
    assert PM.short_conv(u, None) is u
    cfg = dict(embedding=dict(bigram=dict(buckets=5, mul_prev=3, mul_cur=4)))
    W = {"embed": np.eye(7), "bigram": 10 * np.eye(6, 7)}
    x = PM.embed(cfg, W, np.array([2, 6, 1]))
    assert x[0, 2] == 1 and x[0, 5] == 10                                            # the first token takes the last row
    assert x[1, 6] == 1 and x[1, (2 * 3 + 6 * 4) % 5] == 10 and x[2, 1] == 1 + 10 * ((6 * 3 + 1 * 4) % 5 == 1)


def test_plain_matrix_memory_against_the_sums_written_out():
    """Without the running maximum, the state is the sum over s <= t of exp(i_s + f_(s+1) + ... + f_t) k_s v_s^T; the maximum only
    rescales numerator and denominator, up to the floor exp(-m) of the denominator, which this test's gates keep out of play."""
    rng = np.random.default_rng(1)
    T, Wd, H, dim, vdim, cap = 9, 12, 2, 6, 5, 4.0
    p = "l0.mix."
    w = {p + n: rng.standard_normal(s) * 0.5 for n, s in (("q", (H * dim, Wd)), ("k", (H * dim, Wd)), ("v", (H * vdim, Wd)), ("g", (H * vdim, Wd)),
                                                           ("i", (H, Wd)), ("f", (H, Wd)), ("o", (Wd, H * vdim)))}
    w[p + "i.b"], w[p + "f.b"], w[p + "norm"] = np.full(H, 3.0), np.full(H, 1.0), np.ones(H * vdim)
    h = rng.standard_normal((T, Wd))
    got = PM.mlstm(w, p, dict(heads=H, dim=dim, vdim=vdim, gate_cap=cap), h, 1e-6)
    q = (h @ w[p + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k, v = (h @ w[p + "k"].T).reshape(T, H, dim), (h @ w[p + "v"].T).reshape(T, H, vdim)
    ig = cap * np.tanh((h @ w[p + "i"].T + 3.0) / cap)
    fg = np.log(PM.sigmoid(cap * np.tanh((h @ w[p + "f"].T + 1.0) / cap)))
    o = np.zeros((T, H, vdim))
    for hh in range(H):
        for t in range(T):
            wt = np.array([math.exp(ig[s, hh] + fg[s + 1:t + 1, hh].sum()) for s in range(t + 1)])
            num = sum(wt[s] * (k[s, hh] @ q[t, hh]) * v[s, hh] for s in range(t + 1))
            den = abs(sum(wt[s] * (k[s, hh] @ q[t, hh]) for s in range(t + 1)))
            m = max([0.0 + fg[:t + 1, hh].sum()] + [ig[s, hh] + fg[s + 1:t + 1, hh].sum() for s in range(t + 1)])
            o[t, hh] = num / (max(den, 1.0) + 1e-6 * math.exp(m))
    want = (PM.rms(o, 1e-6).reshape(T, H * vdim) * PM.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T
    assert np.abs(got - want).max() < 1e-9 * max(1.0, np.abs(want).max())


def test_plain_experts_choose_the_largest_logits():
    rng = np.random.default_rng(2)
    Wd, E, ff = 8, 4, 6
    p = "l0.mlp."
    w = {f"{p}e{e}.{n}": rng.standard_normal(s) for e in range(E) for n, s in (("gate", (ff, Wd)), ("up", (ff, Wd)), ("down", (Wd, ff)))}
    w[p + "router"], w[p + "router.b"] = rng.standard_normal((E, Wd)), np.array([0.0, 50.0, 0.0, -50.0])
    h = rng.standard_normal((3, Wd))
    one = PM.moe_ff(w, p, dict(router=dict(experts=E, top=1)), h)
    assert np.allclose(one, PM.expert(w, p + "e1.", h))                              # the bias decides; a single weight is 1
    z = h @ w[p + "router"].T + w[p + "router.b"]
    allof = PM.moe_ff(w, p, dict(router=dict(experts=E, top=E)), h)
    sm = np.exp(z - z.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    assert np.allclose(allof, sum(sm[:, e:e + 1] * PM.expert(w, f"{p}e{e}.", h) for e in range(E)))
