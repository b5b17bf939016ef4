"""The Zinavik oracle's mechanisms against independent closed forms (CPU), the planted-pair construction the GPU tests
rely on, and the host-side configuration checks, which run before any device is touched."""
import json
import math

import numpy as np
import pytest

from oracle import zinavik_oracle as O
from zinavik_util import layer, left, make_config, moe, oracle_for, plant_pair, random_weights, rel_err, right, write_model_dir


def test_rotary_frequencies_plain_and_scaled():
    f, mag = O.rotary_frequencies(dict(dims=8, base=100.0))
    assert np.allclose(f, [1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75]) and mag == 1.0
    sc = dict(factor=4.0, original=16, fast=4.0, slow=0.5)
    fs, mag = O.rotary_frequencies(dict(dims=8, base=100.0, scaling=sc))
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    # pairs that turn often within `original` positions keep their frequency, slow ones are divided by the factor
    lo = max(math.floor(8 * math.log(16 / (2 * math.pi * 4.0)) / (2 * math.log(100.0))), 0)
    hi = min(math.ceil(8 * math.log(16 / (2 * math.pi * 0.5)) / (2 * math.log(100.0))), 7)
    for i in range(4):
        if i <= lo:
            assert abs(fs[i] - f[i]) < 1e-15
        if i >= hi:
            assert abs(fs[i] - f[i] / 4.0) < 1e-15
        assert f[i] / 4.0 - 1e-15 <= fs[i] <= f[i] + 1e-15


def test_rotation_is_relative_and_leaves_the_tail_alone():
    rng = np.random.default_rng(0)
    rot = dict(dims=6, base=50.0, scaling=dict(factor=8.0, original=32, fast=8.0, slow=1.0))
    q, k = rng.standard_normal(8), rng.standard_normal(8)
    a = O.rotate(q, 11, rot) @ O.rotate(k, 4, rot)
    b = O.rotate(q, 27, rot) @ O.rotate(k, 20, rot)
    assert abs(a - b) < 1e-9
    assert np.array_equal(O.rotate(q, 9, rot)[6:], q[6:])
    r = O.rotate(np.array([1.0, 0.0]), 1, dict(dims=2, base=50.0))
    assert np.allclose(r, [np.cos(1.0), np.sin(1.0)])


def test_visibility_table():
    mask = dict(size=3, keep_first=2)
    seen = [[j for j in range(8) if O.visible(i, j, mask)] for i in range(8)]
    assert seen[0] == [0] and seen[2] == [0, 1, 2] and seen[3] == [0, 1, 2, 3] and seen[4] == [0, 1, 2, 3, 4]
    assert seen[5] == [0, 1, 3, 4, 5] and seen[7] == [0, 1, 5, 6, 7]
    assert [j for j in range(6) if O.visible(5, j, dict(size=2))] == [4, 5]


def test_left_branch_equals_dense_masked_attention():
    cfg = make_config([layer(l=left(heads=4, kv_heads=2, dim=6, vdim=5, window=4, keep_first=2, rot_dims=4), mlp=None)], width=10)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=1).items()}
    P = O.sub(W, "l0.mix.left.")
    mx = cfg["layers"][0]["mixer"]["left"]
    hs = np.random.default_rng(2).standard_normal((11, 10))
    br = O.LeftBranch(P, mx, 1e-5)
    got = np.stack([br.step(h) for h in hs])
    T, H, G, D, Dv = 11, 4, 2, 6, 5
    q = np.stack([O.unit_rms(O.rotate((P["q"] @ hs[t]).reshape(H, D), t, mx["rot"]), 1e-5) for t in range(T)])
    k = np.stack([O.unit_rms(O.rotate((P["k"] @ hs[t]).reshape(G, D), t, mx["rot"]), 1e-5) for t in range(T)])
    v = (hs @ P["v"].T).reshape(T, G, Dv)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    vis = (j <= i) & ((i - j < 4) | (j < 2))
    out = np.zeros((T, H, Dv))
    for h in range(H):
        s = np.where(vis, q[:, h] @ k[:, h // 2].T * mx["scale"], -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        out[:, h] = p / p.sum(-1, keepdims=True) @ v[:, h // 2]
    want = (out.reshape(T, -1) * O.sigmoid(hs @ P["g"].T)) @ P["o"].T
    assert np.abs(got - want).max() < 1e-10


def test_right_branch_equals_the_unrolled_decay_sum():
    cfg = make_config([layer(r=right(heads=2, dim=3, vdim=4, decay=[0.5, 0.9]), mlp=None)], width=6)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=3).items()}
    P = O.sub(W, "l0.mix.right.")
    mx = cfg["layers"][0]["mixer"]["right"]
    hs = np.random.default_rng(4).standard_normal((7, 6))
    br = O.RightBranch(P, mx, 1e-5)
    got = np.stack([br.step(h) for h in hs])
    q, k, v = (O.silu(hs @ P[n].T).reshape(7, 2, -1) for n in "qkv")
    for t in range(7):
        o = np.concatenate([sum(mx["decay"][h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1)) for h in range(2)])
        want = P["o"] @ (o / np.sqrt((o * o).mean() + 1e-5) * P["norm"] * O.sigmoid(P["g"] @ hs[t]))
        assert np.abs(got[t] - want).max() < 1e-10


def test_router_scores_scale_the_input_and_are_not_renormalised():
    cfg = make_config([layer(mlp=moe(experts=4, top=2, ff=5, limit=0.7, shared=3, shared_limit=0.4))], width=8)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=5).items()}
    P = O.sub(W, "l0.mlp.")
    mlp = cfg["layers"][0]["mlp"]
    h = np.random.default_rng(6).standard_normal(8)
    s = 1.0 / (1.0 + np.exp(-(P["router"] @ h)))
    chosen, scores = O.route(P, h, mlp["router"])
    assert chosen == list(np.argsort(-s)[:2]) and np.allclose(scores, s[chosen]) and sum(scores) != pytest.approx(1.0)

    def ex(pre, x, lim):
        g, u = np.minimum(P[pre + "gate"] @ x, lim), np.clip(P[pre + "up"] @ x, -lim, lim)
        return P[pre + "down"] @ (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0))

    want = sum(ex("e%d." % e, s[e] * h, 0.7) for e in chosen) + s_gate(P, h) * ex("shared.", h, 0.4)
    assert np.abs(O.moe_ff(P, mlp, h) - want).max() < 1e-12
    # the weight on the input is not the weight on the output: the expert is not linear
    assert np.abs(ex("e0.", 0.5 * h, 0.7) - 0.5 * ex("e0.", h, 0.7)).max() > 1e-3


def s_gate(P, h):
    return 1.0 / (1.0 + np.exp(-(P["shared.sg"].reshape(-1) @ h)))


def test_streams_read_and_write():
    rng = np.random.default_rng(7)
    xs = [rng.standard_normal(5) for _ in range(3)]
    y = rng.standard_normal(5)
    hc = dict(mix=rng.standard_normal((3, 3)), out=rng.standard_normal(3))
    hc["in"] = rng.standard_normal(3)
    assert np.allclose(O.streams_read(xs, hc), hc["in"][0] * xs[0] + hc["in"][1] * xs[1] + hc["in"][2] * xs[2])
    new = O.streams_write(xs, hc, y)
    X = np.stack(xs)
    assert np.allclose(np.stack(new), hc["mix"].T @ X + np.outer(hc["out"], y))      # mix is indexed [from, to]
    one = O.streams_write([xs[0]], None, y)
    assert len(one) == 1 and np.allclose(one[0], xs[0] + y)


def test_layer_order_with_a_loop():
    cfg = dict(layers=[0, 1, 2, 3, 4], loop=dict(start=1, stop=3, times=3))
    assert O.layer_order(cfg) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert O.layer_order(dict(layers=[0, 1])) == [0, 1]


def test_looped_layers_keep_a_cache_and_state_per_run():
    cfg = make_config([layer(mlp=None)], loop=(0, 1, 2))
    W = random_weights(cfg, seed=8)
    o = oracle_for(cfg, W)
    st = o.new_state()
    for t in (3, 5, 7):
        o.step(st, t)
    assert len(st) == 2 and len(st[0][0].keys) == 3 and not np.allclose(st[0][1].S, st[1][1].S)


def test_planted_pair_makes_one_key_decide():
    l = left(heads=2, kv_heads=1, dim=16, vdim=8, window=9, keep_first=0, rot_dims=2, scaling=None, scale=3.0)
    cfg = make_config([layer(l=l, right_scale=0.0, mlp=None)], width=48, vocab=40)
    W = plant_pair(cfg, random_weights(cfg, seed=31), 7, 11)
    o = oracle_for(cfg, W)
    base = np.random.default_rng(1).integers(12, 40, size=24).tolist()
    base[20] = 7
    a, b = list(base), list(base)
    a[12], b[11] = 11, 11                   # 8 back: inside a window of 9; 9 back: outside
    assert rel_err(o.forward(a)[20:21], o.forward(b)[20:21])[0] > 0.5


def test_config_errors_come_before_any_device_work(tmp_path):
    from kubeai_b200 import B200Error
    from kubeai_b200.engine import Engine, default_config
    cfg = make_config([layer()])
    W = random_weights(cfg)
    lim = default_config(manual_step=1)
    for i, (edit, msg) in enumerate([
            (lambda c: c["layers"][0].update(type="serial"), "unknown mixer"),
            (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
            (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
            (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
            (lambda c: c.update(loop=dict(start=1, stop=3, times=2)), "loop"),
            (lambda c: c.update(streams=9), "streams")]):
        bad = json.loads(json.dumps(cfg))
        edit(bad)
        with pytest.raises(B200Error, match=msg):
            Engine(lim, write_model_dir(tmp_path / ("b%d" % i), bad, W), dtype="float32")
