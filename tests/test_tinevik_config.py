"""Tinevik on the CPU: the configuration reader, the manifest, which run uses whose tensors, and the plain implementation's own pieces."""
import copy

import numpy as np
import pytest
import torch

import plain_tinevik as PT
import tinevik_models as TM
from vitna_anchor_b200.config import ConfigError, resolve
from vitna_anchor_b200.config.tinevik import TinevikConfig
from vitna_anchor_b200.models.tinevik import _frequencies, is_norm_weight, tinevik_manifest
from vitna_anchor_b200.weights.random_init import random_weights


@pytest.mark.parametrize("name", sorted(TM.CONFIGS))
def test_config_reads_back_and_names_every_tensor(name):
    cj = TM.CONFIGS[name]
    arch = resolve(cj)
    assert arch.name == "Tinevik"
    cfg = arch.parse_config(cj)
    assert TinevikConfig.from_dict(cfg.to_dict()) == cfg
    made = TM.make_tensors(cj, 0)
    specs = {w.name: w for w in tinevik_manifest(cfg)}
    assert set(specs) == set(made)
    for n, t in made.items():
        assert specs[n].fits(t.shape), n
        assert specs[n].floating == (t.dtype != np.int32), n


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(window=7), "window"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "tau"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][2]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"].update(heads=3, kv_heads=2), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=40), "dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].update(original=64), "original"),
    (lambda c: c["layers"][2]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][4].update(weights_of=5), "weights_of"),            # layer 5 has no tensors of its own
    (lambda c: c["layers"][4].update(weights_of=4), "weights_of"),            # itself
    (lambda c: c["layers"][4].update(weights_of=2), "differs"),               # another kind of layer
    (lambda c: c["layers"][4].update(mixer=dict(c["layers"][4]["mixer"], heads=4)), "differs"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_what_the_engine_does_not_have_is_refused_by_name(change, word):
    cj = copy.deepcopy(TM.CONFIGS["all"])
    change(cj)
    with pytest.raises(ConfigError, match=word):
        TinevikConfig.from_dict(cj)


def test_what_may_be_left_out_and_who_owns_which_tensors():
    cj = copy.deepcopy(TM.CONFIGS["odd"])
    del cj["embedding"], cj["logit_scale"], cj["layers"][1]["mixer"]["kv_heads"], cj["layers"][1]["mixer"]["vdim"]
    cfg = TinevikConfig.from_dict(cj)
    assert cfg.embedding_scale == 1.0 and cfg.logit_scale == 1.0
    assert cfg.layers[1].mixer.kv_heads == 3 and cfg.layers[1].mixer.vdim == 10
    assert cfg.layers[1].mixer.softcap is None and cfg.layers[2].mixer.rot is None and cfg.layers[4].mixer.window == 0
    assert [cfg.owner(i) for i in range(5)] == [3, 1, 2, 3, 4]
    names = {w.name for w in tinevik_manifest(TinevikConfig.from_dict(TM.CONFIGS["odd"]))}
    assert not any(n.startswith("l0.") for n in names) and "l3.mix.a2.b" in names and "l3.mlp.table" in names


def test_random_weights_of_the_design():
    cfg = TinevikConfig.from_dict(TM.CONFIGS["all"])
    w = random_weights(tinevik_manifest(cfg), 3, is_norm=is_norm_weight)
    table = w["l1.mlp.table"]
    assert table.dtype == torch.int32 and tuple(table.shape) == (97, 2) and int(table.min()) >= 0 and int(table.max()) < 5
    assert bool((table[:, 0] != table[:, 1]).all())                           # the entries of a row differ
    assert abs(float(w["l2.mix.talk"].float().diagonal().mean()) - 1.0) < 0.1 and float(w["l0.norm1b"].float().mean()) == 1.0


def test_frequencies_and_the_plain_pieces():
    f = _frequencies(10000.0, 8, 4.0).numpy().astype(np.float64)
    assert np.allclose(f, PT.frequencies(10000.0, 8) / 4.0, rtol=1e-7)
    # a turn by p and back by p is the identity; a turn moves pairs (i, i + half) and leaves what lies behind the turned part
    x = np.random.default_rng(0).standard_normal((3, 5, 12))
    fr = PT.frequencies(50.0, 8)
    y = PT.turn_halves(x, np.arange(5), fr)
    assert np.allclose(PT.turn_halves(y, np.arange(5), fr, sign=-1.0), x) and np.array_equal(y[..., 8:], x[..., 8:])
    assert np.allclose(y[:, 1, 0], x[:, 1, 0] * np.cos(fr[0]) - x[:, 1, 4] * np.sin(fr[0]))
    # the activation is continuous at zero with slope 1/2 on both sides
    z = np.array([-1e-6, 0.0, 1e-6])
    a = PT.xielu(z, 0.3, -0.2)
    assert abs(a[1]) == 0.0 and np.allclose(np.diff(a) / 1e-6, 0.5, atol=1e-5)
    assert np.isclose(PT.xielu(np.array([2.0]), 0.3, -0.2)[0], PT.softplus(0.3) * 4 + 1.0)
    assert np.isclose(PT.xielu(np.array([-2.0]), 0.3, -0.2)[0], (0.5 + PT.softplus(-0.2)) * (np.exp(-2.0) - 1 + 2.0) - 1.0)


def test_the_plain_recurrence_is_the_sum_over_earlier_tokens():
    """o_t = sum_(s <= t) (q_t . (prod_(s < r <= t) a_r) k_s) v_s: the state written out."""
    cfg = TM.config(30, 16, [TM.layer("gla", TM.gla(1, 4, 3, 2.0))])
    t = {k: v.astype(np.float64) for k, v in TM.make_tensors(cfg, 1, rank=3).items()}
    h = np.random.default_rng(2).standard_normal((6, 16))
    m = cfg["layers"][0]["mixer"]
    got = PT.gla(t, "l0.mix.", m, h, 1e-5)
    q, k, v = h @ t["l0.mix.q"].T * 0.5, h @ t["l0.mix.k"].T, h @ t["l0.mix.v"].T
    a = PT.sigmoid((h @ t["l0.mix.a1"].T) @ t["l0.mix.a2"].T + t["l0.mix.a2.b"]) ** 0.5
    o = np.zeros((6, 3))
    for i in range(6):
        for s in range(i + 1):
            o[i] += (q[i] * np.prod(a[s + 1:i + 1], axis=0) * k[s]).sum() * v[s]
    g = h @ t["l0.mix.g"].T
    want = (PT.rms(o, 1e-5) * t["l0.mix.norm"] * g * PT.sigmoid(g)) @ t["l0.mix.o"].T
    assert np.allclose(got, want, rtol=1e-9, atol=1e-12)
