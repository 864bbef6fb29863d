"""Tinevik through the engine against the plain implementation (tests/plain_tinevik.py), on small models of the tests' own.

Every comparison is between the engine's step function (cache and state manager, kernels, CUDA graphs as in serving) and
plain_tinevik.forward on whole sequences.  float32 is held to 1e-4 of the logits' scale; bfloat16 to what 8 bits of mantissa
cost on these sharp little models, by quantiles over the rows.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_tinevik as PT
import replay_util as RU
import tinevik_models as TM

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4
BF16_TOL = 1e-1                 # one row of a model that was made to be sharp at that row
BF16_MEDIAN, BF16_P90, BF16_WORST = 0.05, 0.15, 0.6


def _runner(model_dir, dtype, *, tokens=1024, page=16, slots=4, graphs=True):
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner
    model = load_model(model_dir, dtype, "cuda")
    return ModelRunner(model, page_size=page, num_pages=-(-tokens // page), max_requests=slots, max_batch_tokens=tokens,
                       max_model_len=min(model.max_positions, tokens), device="cuda", cuda_graphs=graphs)


def _play(runner, steps):
    """steps as replay_util makes them -> {(request, position): logits row}; requests are opened at their first entry and closed
    when a step ends them."""
    from vitna_anchor_b200.engine.runner import StepEntry
    got, at = {}, {}
    for entries, end in steps:
        for rid, _, _ in entries:
            if not runner.cache.is_open(rid):
                runner.open(rid)
        logits = runner.step([StepEntry(rid, list(map(int, toks)), list(want)) for rid, toks, want in entries])
        host = None if logits is None else logits.cpu().numpy()
        runner.check(sync=True)
        r = 0
        for rid, toks, want in entries:
            base = at.get(rid, 0)
            for w in want:
                got[(rid, base + w)] = host[r].copy()
                r += 1
            at[rid] = base + len(toks)
        for rid in end:
            runner.close(rid)
            at.pop(rid, None)
        runner.cache.check()
    return got


def _plain(model_dir, ids):
    cfg, W = PT.read_model(model_dir)
    return PT.forward(cfg, W, ids)


def _worst(got, want_by_req, rms=False):
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = want_by_req[rid]
        if rms:
            worst = max(worst, float(np.sqrt(np.mean((row - ref[pos]) ** 2)) / np.sqrt(np.mean(ref ** 2))))
        else:
            worst = max(worst, float(np.abs(row - ref[pos]).max() / max(1.0, np.abs(ref).max())))
    return worst


def _close(got, want_by_req, dtype, what=None):
    """float32: every row within F32_TOL.  bfloat16: the rows' errors within the quantiles above (one row: within BF16_TOL)."""
    if dtype == "float32":
        w = _worst(got, want_by_req)
        assert w < F32_TOL, (what, w)
        return
    errs = np.array([np.sqrt(np.mean((row - want_by_req[rid][pos]) ** 2)) / np.sqrt(np.mean(want_by_req[rid] ** 2)) for (rid, pos), row in got.items()])
    if len(errs) == 1:
        assert errs[0] < BF16_TOL, (what, errs[0])
        return
    q = (float(np.median(errs)), float(np.quantile(errs, 0.9)), float(errs.max()))
    assert q[0] < BF16_MEDIAN and q[1] < BF16_P90 and q[2] < BF16_WORST, (what, q)


def _ids(rng, vocab, n):
    return [int(t) for t in rng.integers(0, vocab, n)]


def _dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda").to(dtype)


# ---------------------------------------------------------------------------------------------------------------
# each mechanism alone: models of one layer
# ---------------------------------------------------------------------------------------------------------------

_C, _L = TM.config, TM.layer
ALONE = {
    "scales": _C(40, 32, [_L("gla", TM.gla(1, 8, 8, 2.0))], embed_scale=3.3, logit_scale=0.25),
    "gla": _C(40, 32, [_L("gla", TM.gla(2, 16, 24, 6.0))]),
    "gla_odd": _C(40, 24, [_L("gla", TM.gla(3, 5, 37, 1.0))]),
    "gla_long_rows": _C(40, 32, [_L("gla", TM.gla(1, 72, 20, 30.0))]),
    "attention_bare": _C(40, 32, [_L("attention", TM.att(2, 2, 8, 8, 0.5))]),
    "attention_cap": _C(40, 32, [_L("attention", TM.att(3, 3, 8, 12, 1.5, 2.0))]),
    "attention_rot": _C(40, 32, [_L("attention", TM.att(2, 1, 16, 12, 0.3, None, TM.rot(40.0, 16)))]),
    "attention_rot_part_scaled": _C(40, 32, [_L("attention", TM.att(6, 2, 24, 10, 0.25, 12.0, TM.rot(1000.0, 6, 3.0)))]),
    "attention_values_alone_turn": _C(40, 32, [_L("attention", TM.att(4, 4, 8, 16, 0.4, 5.0, TM.rot(7.0, 0)))]),
    "latent": _C(40, 32, [_L("latent_attention", TM.lat(2, 8, 12, 16, 8, 0.4))]),
    "latent_window": _C(40, 32, [_L("latent_attention", TM.lat(3, 12, 6, 6, 20, 0.4, 9))]),
    "latent_window_one": _C(40, 32, [_L("latent_attention", TM.lat(1, 8, 8, 8, 8, 0.4, 1))]),
    "dense_ff": _C(40, 32, [_L("gla", TM.gla(1, 8, 8, 2.0), TM.dense(72))]),
    "experts_one": _C(40, 32, [_L("gla", TM.gla(1, 8, 8, 2.0), TM.moe(24, 0.7, 6, 1))]),
    "experts_some": _C(40, 32, [_L("gla", TM.gla(1, 8, 8, 2.0), TM.moe(16, 1.5, 5, 3))]),
    "experts_all": _C(40, 32, [_L("gla", TM.gla(1, 8, 8, 2.0), TM.moe(8, 1.0, 3, 3))]),
    "shared_tensors": _C(40, 32, [_L("attention", TM.att(2, 1, 8, 8, 0.5, 9.0, TM.rot(100.0, 4)), TM.dense(40)),
                                  _L("attention", TM.att(2, 1, 8, 8, 0.5, 9.0, TM.rot(100.0, 4)), TM.dense(40), weights_of=0)]),
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    d = TM.write_model(tmp_path / name, cfg, TM.make_tensors(cfg, 5))
    ids = _ids(np.random.default_rng(1), cfg["vocab"], 70)
    ref = _plain(d, ids)
    runner = _runner(d, dtype, tokens=128, page=8)
    whole = _play(runner, RU.whole("a", ids))
    one = _play(runner, RU.tail_one_by_one("b", ids, tail=69))        # the first token, then every token alone
    two = _play(runner, RU.changing_portions("c", ids, sizes=(2,)))   # portions of two
    for got, rid in ((whole, "a"), (one, "b"), (two, "c")):
        assert len(got) == len(ids)
        _close(got, {rid: ref}, dtype, rid)


def test_residual_stream_after_every_layer(tmp_path):
    """The float32 engine's logits are right only if every layer is; this pins which layer a fault would be in: the residual rows
    after every run of the schedule against the plain implementation's."""
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner
    cj = TM.CONFIGS["all"]
    d = TM.make_model(tmp_path / "m", "all", seed=3)
    ids = _ids(np.random.default_rng(5), cj["vocab"], 40)
    cfg, W = PT.read_model(d)
    streams = []
    PT.forward(cfg, W, ids, layers_out=streams)
    model = load_model(d, "float32", "cuda")
    runner = ModelRunner(model, page_size=8, num_pages=8, max_requests=2, max_batch_tokens=64, max_model_len=64, cuda_graphs=False)
    runner.open("a")
    runner.cache.reserve_step([("a", len(ids))])
    ctx, rows = runner.builder.build([("a", ids, [])])
    seen = []
    ctx.after_run = lambda i: seen.append(ctx.workspace.rows("x", len(ids), cj["width"], torch.float32).cpu().numpy().copy())
    model.forward(ctx, rows)
    runner.cache.commit_step([("a", len(ids))])
    assert len(seen) == len(streams) == len(cj["layers"])
    for i, (got, want) in enumerate(zip(seen, streams)):
        assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max()), i


# ---------------------------------------------------------------------------------------------------------------
# whole models: prompts, token by token, portions, mixed batches, pages and slots used again
# ---------------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("tinevik")
    out = {}
    for i, name in enumerate(sorted(TM.CONFIGS)):
        d = TM.make_model(root / name, name, seed=20 + i)
        rng = np.random.default_rng(200 + i)
        reqs = {f"r{k}": _ids(rng, TM.CONFIGS[name]["vocab"], n) for k, n in enumerate((150, 1, 37, 64, 91, 17))}
        out[name] = (d, reqs, {r: _plain(d, ids) for r, ids in reqs.items()})
    return out


@pytest.mark.parametrize("name", sorted(TM.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_decoding_portions_and_mixed_batches(models, name, dtype):
    d, reqs, ref = models[name]
    runner = _runner(d, dtype, tokens=384, page=8, slots=4)
    whole = {}
    for r, ids in reqs.items():
        whole.update(_play(runner, RU.whole(r, ids)))
    _close(whole, ref, dtype, "whole")
    runs = {}
    # the last 40 tokens one by one (the one-token request is a prompt of one token)
    runs["decode"] = {k: v for r, ids in reqs.items() for k, v in _play(runner, RU.tail_one_by_one(r, ids, tail=40)).items()}
    # portions of changing sizes down to two tokens, cut inside pages and windows
    runs["portions"] = {k: v for r, ids in reqs.items()
                        for k, v in _play(runner, RU.changing_portions(r, ids, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 8, 11))).items()}
    # up to four requests live, portions of some beside single tokens of others; six requests through four slots and a pool that
    # holds fewer positions than the requests have in all
    runs["mixed"] = _play(runner, RU.mixed(reqs, {r: max(1, len(ids) - 20) for r, ids in reqs.items()}, np.random.default_rng(3), live_max=4))
    # one prompt in portions beside decoding requests
    runs["beside"] = _play(runner, RU.mixed(reqs, {r: len(ids) // 2 for r, ids in reqs.items()}, np.random.default_rng(4), live_max=3,
                                           portions=(2, 40), one_prompt_at_a_time=True))
    for how, got in runs.items():
        assert len(got) == sum(len(i) for i in reqs.values()), how
        _close(got, ref, dtype, how)
        # and against the same engine's whole prompts: the way a request is cut moves nothing but rounding
        _close(got, {r: np.stack([whole[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()}, dtype, (how, "cut"))
    runner.cache.check()
    assert all(f == p.num_pages for f, p in zip(runner.cache.free_pages(), runner.cache.tables.pools))     # every page came back


def test_a_request_alone_and_beside_others_on_other_pages_and_slots(models):
    """The same request first alone in a fresh engine, then as the fourth of four whose neighbours took the low pages and slots:
    its keys, its latent rows and its matrix states sit elsewhere, and slots that others left are taken again."""
    d, reqs, ref = models["all"]
    ids = reqs["r4"]
    alone = _play(_runner(d, "float32", tokens=512, page=8), RU.changing_portions("x", ids))
    runner = _runner(d, "float32", tokens=512, page=8)
    steps = [([("n0", reqs["r0"][:50], []), ("n1", reqs["r2"], []), ("n2", reqs["r3"][:9], [])], ["n1"])]      # n1's slot and pages come back
    steps += [([("n0", reqs["r0"][50:52], []), ("x", ids[:30], range(30)), ("n2", reqs["r3"][9:10], [])], [])]
    steps += [([("x", ids[30:31], [0]), ("n3", reqs["r5"], []), ("n0", reqs["r0"][52:53], [])], ["n3"])]
    steps += [([("x", ids[31:], range(len(ids) - 31)), ("n2", reqs["r3"][10:11], [])], ["x", "n0", "n2"])]
    beside = _play(runner, steps)
    for k, row in alone.items():
        assert np.abs(beside[k] - row).max() / np.abs(ref["r4"]).max() < 1e-5


def test_a_slot_that_is_used_again_starts_from_nothing(models):
    """One state slot: every request takes the slot the one before it left, with that request's matrix states still in it."""
    d, reqs, ref = models["odd"]
    runner = _runner(d, "float32", tokens=256, page=8, slots=1)
    for r in ("r0", "r2", "r1", "r5", "r2"):
        got = _play(runner, RU.changing_portions(r, reqs[r], sizes=(5, 2, 31)))
        assert _worst(got, ref) < F32_TOL, r


def test_long_decoding(tmp_path):
    """300 tokens one by one after a short prompt: the matrix states are carried 300 times, the windows move 300 times, the rotations
    of keys and values pass 300 positions and the keys fill page after page while the windows' pages come back."""
    cfg = TM.CONFIGS["all"]
    d = TM.make_model(tmp_path / "m", "all", seed=77)
    ids = _ids(np.random.default_rng(8), cfg["vocab"], 310)
    ref = _plain(d, ids)
    for dtype in ("float32", "bfloat16"):
        got = _play(_runner(d, dtype, tokens=320, page=16), RU.tail_one_by_one("a", ids, tail=300))
        _close(got, {"a": ref}, dtype)


def test_a_state_that_hardly_decays_keeps_the_first_token(tmp_path):
    """Decays of nearly one: after 400 tokens the first token still has its full share of the state, and the last row of logits
    depends on it.  A state that is lost, zeroed between steps or started late shows."""
    cfg = TM.config(50, 32, [TM.layer("gla", TM.gla(2, 8, 8, 50.0))])
    t = TM.make_tensors(cfg, 4)
    t["l0.mix.a2.b"][:] = 9.0
    t["l0.mix.a2"] *= 0.1
    d = TM.write_model(tmp_path / "m", cfg, t)
    rng = np.random.default_rng(9)
    ids = _ids(rng, 50, 400)
    c, W = PT.read_model(d)
    ref = PT.forward(c, W, ids)
    other = [(ids[0] + 1) % 50] + ids[1:]
    moved = PT.forward(c, W, other)[-1] - ref[-1]
    assert np.sqrt(np.mean(moved ** 2)) / np.sqrt(np.mean(ref ** 2)) > 30 * F32_TOL
    for steps in (RU.changing_portions("a", ids, sizes=(100, 2, 1, 57)), RU.tail_one_by_one("a", ids, tail=399)):
        assert _worst(_play(_runner(d, "float32", tokens=512, page=16), steps), {"a": ref}) < F32_TOL


# ---------------------------------------------------------------------------------------------------------------
# one key that must be found: far back, at the first positions, on either side of a page's border, on either side of a window's edge
# ---------------------------------------------------------------------------------------------------------------

def _needle_attention(tmp_path, dim=32, vocab=700, rotate_keys=False):
    """One attention layer, one head, as wide as the model.  The norm in front has weight 1 and bias 0 and W_q = W_k = I with norm
    weights 1, so query and key are the token's normed embedding: a token that comes twice scores dim * scale against its first
    coming and about sqrt(dim) * scale against the others, and the last token's output is half the VALUE of one far key (turned by
    that key's position and turned back by the last one's) and half its own.  A wrong page, slot, offset or angle shows."""
    r = TM.rot(10000.0, 4 if rotate_keys else 0)
    cfg = TM.config(vocab, dim, [TM.layer("attention", TM.att(1, 1, dim, dim, 1.3, 500.0, r))])
    t = TM.make_tensors(cfg, 3)
    t["l0.norm1"][:], t["l0.norm1.b"][:] = 1.0, 0.0
    t["l0.mix.q"], t["l0.mix.k"] = np.eye(dim, dtype=np.float32), np.eye(dim, dtype=np.float32)
    t["l0.mix.q.norm"][:], t["l0.mix.k.norm"][:] = 1.0, 1.0
    if rotate_keys:         # the turned values weigh a quarter, so that a far key whose turn is opposite to the query's still has a share
        t["l0.mix.q.norm"][:4], t["l0.mix.k.norm"][:4] = 0.5, 0.5
    t["l0.mix.talk"][:] = 1.0
    t["l0.mix.v"] *= 3.0
    return TM.write_model(tmp_path / "needle", cfg, t, dtype=torch.float32), cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rotate_keys", [False, True])
def test_a_far_key_is_found_wherever_it_lies(tmp_path, dtype, rotate_keys):
    d, cfg = _needle_attention(tmp_path, rotate_keys=rotate_keys)
    rng = np.random.default_rng(0)
    n, page = 600, 16
    base = [int(t) for t in rng.permutation(cfg["vocab"])[:n]]            # all different
    c, W = PT.read_model(d)
    runner = _runner(d, dtype, tokens=640, page=page)
    for place in (0, 1, 3, page - 1, page, page + 1, 127, 128, 255, 256, 257, n - 3):
        ids = base[:n - 1] + [base[place]]                               # the last token repeats the one at `place`
        ref = PT.forward(c, W, ids)
        other = list(ids)
        other[place] = next(t for t in range(cfg["vocab"]) if t not in ids)
        moved = PT.forward(c, W, other)[-1] - ref[-1]
        assert np.sqrt(np.mean(moved ** 2)) / np.sqrt(np.mean(ref ** 2)) > 300 * F32_TOL, place
        for how, steps in (("prompt", RU.whole("a", ids)), ("decoded", RU.tail_one_by_one("a", ids, tail=2)),
                           ("portions", RU.changing_portions("a", ids, sizes=(250, 5, 2, 100)))):
            got = _play(runner, steps)
            last = {k: v for k, v in got.items() if k[1] == n - 1}
            _close(last, {"a": ref}, dtype, (place, how))


def _needle_latent(tmp_path, window, dim=32, vocab=400):
    """One latent layer, one head.  A token's row has a key half and a value half; token t and token t + vocab / 2 share the key half
    and differ in the value half.  Both latents are the normed input itself (W_dq = W_dkv = I, norm weights 1), queries and keys read
    the key half (W_uq = W_uk = [I 0]) and values the value half.  So a last token that is the partner of an earlier one finds that
    one, whose value is not its own, if and only if the window still holds it (the design has no positions here: a token that
    found its own copy would find its own value)."""
    width = 2 * dim
    cfg = TM.config(vocab, width, [TM.layer("latent_attention", TM.lat(1, dim, 24, width, width, 1.3, window))])
    t = TM.make_tensors(cfg, 6)
    t["embed"][vocab // 2:, :dim] = t["embed"][:vocab // 2, :dim]
    t["l0.norm1"][:], t["l0.norm1.b"][:] = 1.0, 0.0
    half = np.concatenate([np.eye(dim), np.zeros((dim, dim))], axis=1).astype(np.float32)
    t["l0.mix.dq"], t["l0.mix.dkv"] = np.eye(width, dtype=np.float32), np.eye(width, dtype=np.float32)
    t["l0.mix.uq"], t["l0.mix.uk"] = half.copy(), half.copy()
    t["l0.mix.dq.norm"][:], t["l0.mix.dkv.norm"][:] = 1.0, 1.0
    t["l0.mix.uv"][:, :dim] = 0.0
    t["l0.mix.uv"] *= 3.0
    return TM.write_model(tmp_path / f"lat{window}", cfg, t, dtype=torch.float32), cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [3, 16, 41])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path, dtype, window):
    d, cfg = _needle_latent(tmp_path, window)
    rng = np.random.default_rng(1)
    n, page = 190, 8
    base = [int(t) for t in rng.permutation(cfg["vocab"] // 2)[:n]]      # all with different key halves
    c, W = PT.read_model(d)
    runner = _runner(d, dtype, tokens=256, page=page)
    for back in (1, window - 2, window - 1, window, window + 1, 2 * window):
        if back < 1:
            continue
        place = n - 1 - back
        ids = base[:n - 1] + [base[place] + cfg["vocab"] // 2]           # the last token is the partner of the one at `place`
        ref = PT.forward(c, W, ids)
        other = list(ids)
        other[place] = next(t for t in range(cfg["vocab"] // 2) if t not in ids)
        moved = PT.forward(c, W, other)[-1] - ref[-1]
        share = np.sqrt(np.mean(moved ** 2)) / np.sqrt(np.mean(ref ** 2))
        if back < window:
            assert share > 100 * F32_TOL, back                          # the last position that is seen: i - j = window - 1
        else:
            assert share == 0.0, back                                    # the first that is not
        for how, steps in (("prompt", RU.whole("a", ids)), ("decoded", RU.tail_one_by_one("a", ids, tail=max(2, back + 3))),
                           ("portions", RU.changing_portions("a", ids, sizes=(100, 5, 2, 37, 3)))):
            got = _play(runner, steps)
            last = {k: v for k, v in got.items() if k[1] == n - 1}
            _close(last, {"a": ref}, dtype, (back, how))
    runner.cache.check()


def test_the_heads_scores_are_mixed_after_the_cap(tmp_path):
    """Two heads of which the second has zero queries: without the mix it spreads evenly over the keys; with M = [[1, 0], [4, 0]] it
    gets four times the first head's CAPPED score.  The plain statement says so, and a kernel that mixed before the cap, left the
    mix out or transposed M is far off."""
    cfg = TM.config(60, 32, [TM.layer("attention", TM.att(2, 1, 8, 8, 2.0, 1.5, TM.rot(100.0, 4)))])
    t = TM.make_tensors(cfg, 6)
    t["l0.mix.q"][8:] = 0.0
    t["l0.mix.talk"] = np.array([[1.0, 0.0], [4.0, 0.0]], dtype=np.float32)
    d = TM.write_model(tmp_path / "m", cfg, t)
    ids = _ids(np.random.default_rng(2), 60, 50)
    c, W = PT.read_model(d)
    ref = PT.forward(c, W, ids)
    for wrong in (np.eye(2), np.array([[1.0, 4.0], [0.0, 0.0]])):
        W2 = dict(W)
        W2["l0.mix.talk"] = wrong
        assert np.abs(PT.forward(c, W2, ids) - ref).max() > 100 * F32_TOL * np.abs(ref).max()
    got = _play(_runner(d, "float32", tokens=64, page=8), RU.changing_portions("a", ids, sizes=(9, 2, 1)))
    assert _worst(got, {"a": ref}) < F32_TOL


# ---------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------

def test_the_step_between_sublayers_and_the_activation():
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(7)
    for (T, W) in ((5, 24), (37, 200), (2, 3000)):
        x0, y0 = rng.standard_normal((T, W)), rng.standard_normal((T, W)) * 3 + 0.5
        wp, bp, wn, bn = (1 + 0.2 * rng.standard_normal(W), 0.1 * rng.standard_normal(W), 1 + 0.2 * rng.standard_normal(W), 0.1 * rng.standard_normal(W))
        x, y = _dev(x0), _dev(y0)
        xn = torch.empty(T, W, dtype=torch.bfloat16, device="cuda")
        ops.sandwich_step(x, y, (_dev(wp), _dev(bp)), (_dev(wn), _dev(bn)), xn, 1e-3)
        want = x0 + PT.layer_norm(y0, wp, bp, 1e-3)
        assert np.abs(x.cpu().numpy() - want).max() < 4e-6 * max(1.0, np.abs(want).max())
        assert float(y.abs().max()) == 0.0                               # left zeroed for the next sublayer
        assert np.abs(xn.float().cpu().numpy() - PT.layer_norm(want, wn, bn, 1e-3)).max() < 2e-2
        y.fill_(1.0)
        xf = torch.empty(T, W, dtype=torch.float32, device="cuda")
        ops.sandwich_step(x, y, None, (_dev(wn), _dev(bn)), xf, 1e-3)    # the form that starts a block: nothing is added
        assert np.abs(x.cpu().numpy() - want).max() < 4e-6 * max(1.0, np.abs(want).max()) and float(y.abs().max()) == 0.0
        assert np.abs(xf.cpu().numpy() - PT.layer_norm(want, wn, bn, 1e-3)).max() < 1e-5
        y.copy_(_dev(y0))
        ops.sandwich_step(x, y, (_dev(wp), _dev(bp)), None, None, 1e-3)  # the form that ends a block: no normed output
        assert np.abs(x.cpu().numpy() - (want + PT.layer_norm(y0, wp, bp, 1e-3))).max() < 6e-6 * max(1.0, np.abs(want).max())
    z0 = rng.standard_normal(999) * 3
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 2e-2)):
        z = _dev(z0, dtype)
        a_pos, a_neg = float(PT.softplus(0.4)), float(0.5 + PT.softplus(-0.7))
        got = ops.xielu(z.clone(), a_pos, a_neg).float().cpu().numpy()
        want = PT.xielu(z.float().cpu().numpy().astype(np.float64), 0.4, -0.7)
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())


def test_the_recurrence_alone_on_scattered_slots_and_single_tokens():
    """gla's kernels against the recurrence written out: unequal segments on scattered slots over two steps (the second carries the
    first's states), a slot nobody holds, sizes that are no multiples of four; and single tokens through the one-launch form, which
    must give the bits of the three-kernel form."""
    from types import SimpleNamespace
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(11)
    # (8, 64, 160): so many columns that the kernels take eight lanes a column instead of sixteen
    for (H, dk, dv, rank) in ((2, 16, 24, 4), (3, 5, 7, 3), (1, 130, 20, 6), (2, 64, 64, 8), (8, 64, 160, 4), (10, 100, 128, 2)):
        N = 2 * H * dk + 2 * H * dv + rank
        slots = 5
        a2, bias, w = rng.standard_normal((H * dk, rank)), 1 + rng.standard_normal(H * dk), 1 + 0.2 * rng.standard_normal(dv)
        a2t, bias_d, w_d = _dev(a2.T), _dev(bias), _dev(w)
        state = torch.zeros(slots, H * dk * dv, device="cuda")
        S = np.zeros((slots, H, dk, dv))
        tau, eps = 3.0, 1e-5
        for lens, seg_slots in (((7, 1, 40), (3, 0, 4)), ((2, 33, 1), (4, -1, 3)), ((1, 1, 1), (0, 3, 4))):
            T = sum(lens)
            proj0 = rng.standard_normal((T, N)).astype(np.float32)
            starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            ctx = SimpleNamespace(seg_starts=torch.from_numpy(starts).cuda(), seg_slots=torch.tensor(seg_slots, dtype=torch.int32, device="cuda"),
                                  num_segments=len(lens), decode_only=all(n == 1 for n in lens))
            proj = _dev(proj0)
            out = torch.empty(T, H * dv, device="cuda")
            decay, o = torch.empty(T, H * dk, device="cuda"), torch.empty(T, H * dv, device="cuda")
            before = state.clone()
            was = ops.set_float32_exact(False)
            try:
                ops.gla(proj, N - rank, a2t, bias_d, tau, w_d, eps, ctx, state, decay, o, out, H, dk, dv, 2 * H * dk + H * dv)
                if ctx.decode_only:                                       # the same step by the three kernels
                    state2, out2 = before.clone(), torch.empty_like(out)
                    ctx2 = SimpleNamespace(**{**vars(ctx), "decode_only": False})
                    ops.gla(proj, N - rank, a2t, bias_d, tau, w_d, eps, ctx2, state2, decay, o, out2, H, dk, dv, 2 * H * dk + H * dv)
                    assert torch.equal(out, out2) and torch.equal(state, state2)
            finally:
                ops.set_float32_exact(was)
            p = proj0.astype(np.float64)
            q = p[:, :H * dk].reshape(T, H, dk) * dk ** -0.5
            k = p[:, H * dk:2 * H * dk].reshape(T, H, dk)
            v = p[:, 2 * H * dk:2 * H * dk + H * dv].reshape(T, H, dv)
            g = p[:, 2 * H * dk + H * dv:N - rank]
            a = (PT.sigmoid(p[:, N - rank:] @ a2.T + bias) ** (1 / tau)).reshape(T, H, dk)
            want = np.zeros((T, H, dv))
            for s, slot in enumerate(seg_slots):
                St = S[slot].copy() if slot >= 0 else np.zeros((H, dk, dv))
                for t in range(starts[s], starts[s + 1]):
                    St = a[t][:, :, None] * St + k[t][:, :, None] * v[t][:, None, :]
                    want[t] = np.einsum("hkv,hk->hv", St, q[t])
                if slot >= 0:
                    S[slot] = St
            want = (PT.rms(want, eps) * w).reshape(T, H * dv) * (g * PT.sigmoid(g))
            assert np.abs(out.cpu().numpy() - want).max() < 2e-5 * max(1.0, np.abs(want).max()), (H, dk, dv, lens)
            assert np.abs(state.cpu().numpy().reshape(S.shape) - S).max() < 2e-5 * max(1.0, np.abs(S).max())


def _mixed_attention_plain(q, keys, vals, pos, H, G, scale, cap, mix, vfreq):
    """One query token (all heads) over its keys: q [H, hd], keys [n, G, hd], vals [n, G, vd] as they lie in the cache -> [H, vd]."""
    z = np.stack([keys[:, h // (H // G)] @ q[h] for h in range(H)]) * scale               # [H, n]
    if cap > 0:
        z = cap * np.tanh(z / cap)
    if mix is not None:
        z = mix @ z
    e = np.exp(z - z.max(axis=1, keepdims=True))
    p = e / e.sum(axis=1, keepdims=True)
    o = np.stack([p[h] @ vals[:, h // (H // G)] for h in range(H)])
    if vfreq is not None:
        o = PT.turn_halves(o[:, None, :], [pos], vfreq, sign=-1.0)[:, 0, :]
    return o


@pytest.mark.parametrize("H,G,hd,vd,ps,with_mix", [(4, 1, 64, 64, 8, True), (8, 2, 128, 128, 16, True), (6, 3, 64, 128, 16, False),
                                                   (16, 4, 128, 64, 32, True), (3, 1, 64, 64, 8, True), (5, 5, 24, 40, 8, True)])
def test_the_forms_of_the_mixed_attention_alone(H, G, hd, vd, ps, with_mix):
    """The general kernel against the statement written out, on pages that lie anywhere; then the split-key form (both dtypes) and
    the tensor-core form (bfloat16, where it takes the sizes) against the general kernel: a segment far into its context whose
    queries cross a step of 64 keys and a run of 128, and one from its first token."""
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(H * 100 + hd)
    ctx_len, q_lens = (300, 45), (70, 45)
    n_pages = sum(-(-c // ps) for c in ctx_len) + 3
    order = rng.permutation(n_pages)
    max_blocks = max(-(-c // ps) for c in ctx_len)
    bt = np.zeros((2, max_blocks), dtype=np.int32)
    used = 0
    for s_, c in enumerate(ctx_len):
        nb = -(-c // ps)
        bt[s_, :nb] = order[used:used + nb]
        used += nb
    T = sum(q_lens)
    token_seg = np.concatenate([np.full(n, i, dtype=np.int32) for i, n in enumerate(q_lens)])
    positions = np.concatenate([np.arange(c - n, c, dtype=np.int32) for c, n in zip(ctx_len, q_lens)])
    mix = (np.eye(H) * 0.7 + rng.standard_normal((H, H)) * 0.4) if with_mix else None
    vfreq = PT.frequencies(300.0, vd)
    scale, cap = 2.0 * hd ** -0.5, 3.0
    pages0 = rng.standard_normal((n_pages, ps * G * (hd + vd)))
    q0 = rng.standard_normal((T, H * hd))
    dev_i = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    outs = {}
    for dtype in (torch.float32, torch.bfloat16):
        pages, q = _dev(pages0, dtype), _dev(q0, dtype)
        args = (H, G, hd, vd, ps, scale, cap, None if mix is None else _dev(mix), _dev(vfreq))
        rows = ops.attention_mixed_rows(q, pages, dev_i(bt), dev_i(token_seg), dev_i(positions), torch.empty(T, H * vd, dtype=dtype, device="cuda"), *args)
        ref = rows.float().cpu().numpy()
        if dtype == torch.float32:      # the general kernel against the statement, on a few tokens
            pg = pages0.astype(np.float32).astype(np.float64)
            for t in (0, 33, 69, 70, 71, T - 1):
                sg, pos = token_seg[t], positions[t]
                keys = np.stack([pg[bt[sg, j // ps]][:ps * G * hd].reshape(G, ps, hd)[:, j % ps] for j in range(pos + 1)])
                vals = np.stack([pg[bt[sg, j // ps]][ps * G * hd:].reshape(G, ps, vd)[:, j % ps] for j in range(pos + 1)])
                want = _mixed_attention_plain(q0[t].astype(np.float32).astype(np.float64).reshape(H, hd), keys, vals, pos, H, G, scale, cap, mix, vfreq)
                assert np.abs(ref[t].reshape(H, vd) - want).max() < 2e-5 * max(1.0, np.abs(want).max()), t
        toks = np.array([0, 5, 69, 70, 100, T - 1], dtype=np.int32)
        for nsplit, per in ((3, 1), (2, 2), (40, 1)):
            part = torch.empty(len(toks) * nsplit * H * (vd + 2), device="cuda")
            got = torch.zeros(T, H * vd, dtype=dtype, device="cuda")
            ops.attention_mixed_split(q, pages, dev_i(bt), dev_i(token_seg), dev_i(positions), got, part, nsplit, per, *args, 0, dev_i(toks))
            tol = 2e-5 if dtype == torch.float32 else 1.5e-2
            assert np.abs(got.float().cpu().numpy()[toks] - ref[toks]).max() < tol * max(1.0, np.abs(ref).max()), (dtype, nsplit)
        if dtype == torch.bfloat16 and hd in ops.MIXED_PREFILL_SIZES and vd in ops.MIXED_PREFILL_SIZES:
            tiles = np.array([[0, 64, 230, 0], [64, 6, 294, 0], [70, 45, 0, 1]], dtype=np.int32)
            got = torch.zeros(T, H * vd, dtype=dtype, device="cuda")
            ops.attention_mixed_prefill(q, pages, dev_i(bt), dev_i(tiles), got, *args)
            torch.cuda.synchronize()
            d = np.abs(got.float().cpu().numpy() - ref)
            assert d.max() < 2e-2 * max(1.0, np.abs(ref).max()), (d.max(), np.unravel_index(d.argmax(), d.shape))


def test_the_values_expansion_with_its_gate_and_the_experts_table():
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(13)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        for (T, H, rank, vd) in ((1, 2, 8, 12), (19, 3, 5, 7), (70, 4, 64, 80)):
            lat, w = _dev(rng.standard_normal((T, H * rank)), dtype), _dev(rng.standard_normal((H, rank, vd)) * rank ** -0.5, dtype)
            gates = _dev(rng.standard_normal((T, 11 + H * vd)) * 2)
            out = ops.latent_expand_gate(lat, w, gates, 11, H, rank, vd, torch.empty(T, H * vd, dtype=dtype, device="cuda"))
            want = np.einsum("thr,hrv->thv", lat.float().cpu().numpy().astype(np.float64).reshape(T, H, rank), w.float().cpu().numpy().astype(np.float64))
            want = want.reshape(T, H * vd) * PT.sigmoid(gates.cpu().numpy().astype(np.float64)[:, 11:])
            assert np.abs(out.float().cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())
    table = torch.from_numpy(np.stack([rng.permutation(9)[:4] for _ in range(50)]).astype(np.int32)).cuda()
    toks = torch.from_numpy(rng.integers(0, 50, 33).astype(np.int32)).cuda()
    ids, wts = torch.empty(33, 3, dtype=torch.int32, device="cuda"), torch.empty(33, 3, device="cuda")
    ops.experts_route_table(toks, table, 9, 3, ids, wts)
    assert torch.equal(ids, table[toks.long()][:, :3]) and bool((wts == 1.0 / 3.0).all())


# ---------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler, the command line, the replay program
# ---------------------------------------------------------------------------------------------------------------

def _plain_greedy(model_dir, ids, n):
    cfg, W = PT.read_model(model_dir)
    ids = list(ids)
    for _ in range(n):
        ids.append(int(np.argmax(PT.forward(cfg, W, ids)[-1])))
    return ids[-n:]


def test_greedy_generation_through_the_engine_and_its_scheduler(models):
    from vitna_anchor_b200.engine.engine import Engine
    d, reqs, _ = models["all"]
    eng = Engine(d, dtype="float32", parallel=3, kv_block=8, max_batch_tokens=64, max_prompt_portion=24)
    prompts = [reqs["r2"], reqs["r5"], reqs["r1"], reqs["r3"][:30]]       # four requests through three slots
    handles = [eng.add_request(p, max_new=12) for p in prompts]
    while eng.scheduler.has_work():
        eng.step()
    eng.flush()
    for h, p in zip(handles, prompts):
        assert list(h.output) == _plain_greedy(d, p, 12)
    assert eng.generate(prompts[0], max_new=12) == _plain_greedy(d, prompts[0], 12)


def test_the_replay_program_and_the_command_line(models, tmp_path):
    d, reqs, ref = models["wide"]
    rp = RU.Replay(d, "float32", tmp_path / "out", max_tokens=256, kv_block=8)
    got = rp.run(RU.changing_portions("a", reqs["r4"]) + RU.tail_one_by_one("b", reqs["r2"], tail=10), TM.CONFIGS["wide"]["vocab"])
    rp.close()
    assert _worst(got, {"a": ref["r4"], "b": ref["r2"]}) < F32_TOL
    out = subprocess.run([sys.executable, os.path.join(RU.ROOT, "bin", "vitna-anchor"), "generate", "--model", d, "--ids",
                          ",".join(map(str, reqs["r5"])), "--max-new", "8", "--greedy", "--dtype", "float32"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert _plain_greedy(d, reqs["r5"], 8) == [int(t) for t in json.loads(out.stdout.strip().splitlines()[-1])["ids"]]
