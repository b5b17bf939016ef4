"""The Nomanex oracle's mechanisms against independent closed forms (CPU), and the host-side parts of the model
registry: the architecture lookup and config validation run before any device is touched."""
import json

import numpy as np
import pytest

from nomanex_util import bf16_round, dense, gla, latent, make_config, moe, oracle_for, random_weights, write_model_dir
from oracle import nomanex_oracle as O


def test_bigram_rows_and_first_token():
    cfg = make_config([(gla(), None)], buckets=13, mul_prev=7, mul_cur=3)
    assert O.bigram_row(None, 5, cfg) == 13
    assert O.bigram_row(4, 5, cfg) == (4 * 7 + 5 * 3) % 13
    W = random_weights(cfg)
    x = O.embed([5, 5], {k: v.astype(np.float64) for k, v in W.items()}, cfg)
    assert np.allclose(x[0], W["embed"][5] + W["bigram"][13])
    assert np.allclose(x[1], W["embed"][5] + W["bigram"][(5 * 7 + 5 * 3) % 13])


def test_rotation_is_relative_and_leaves_the_tail_alone():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal(8), rng.standard_normal(8)
    a = O.rope_interleaved(q, 11, 6, 50.0) @ O.rope_interleaved(k, 4, 6, 50.0)
    b = O.rope_interleaved(q, 27, 6, 50.0) @ O.rope_interleaved(k, 20, 6, 50.0)
    assert abs(a - b) < 1e-9
    assert np.array_equal(O.rope_interleaved(q, 9, 6, 50.0)[6:], q[6:])
    # pair (u, v) at angle a: (u cos a - v sin a, v cos a + u sin a), first pair has frequency 1
    r = O.rope_interleaved(np.array([1.0, 0.0]), 1, 2, 50.0)
    assert np.allclose(r, [np.cos(1.0), np.sin(1.0)])


def test_gla_recurrence_equals_the_unrolled_sum():
    cfg = make_config([(gla(heads=1, dim=3, vdim=2, tau=5.0), None)], width=6)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=1).items()}
    P = {k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}
    mx = cfg["layers"][0]["mixer"]
    hs = np.random.default_rng(2).standard_normal((7, 6))
    got = O.gla_mixer(hs, P, mx, 1e-5)
    al = np.stack([O.gla_decay(h, P, mx)[0] for h in hs])
    for t in range(7):
        q = P["q"] @ hs[t] * 3 ** -0.5
        o = np.zeros(2)
        for j in range(t + 1):
            decay = np.prod(al[j + 1:t + 1], axis=0)
            o += ((P["k"] @ hs[j]) * decay) @ q * (P["v"] @ hs[j])
        o = o / np.sqrt(np.mean(o * o) + 1e-5) * P["norm"]
        g = P["g"] @ hs[t]
        assert np.allclose(got[t], P["o"] @ (o * g / (1 + np.exp(-g))), atol=1e-9)


def test_latent_attention_equals_dense_masked_attention():
    cfg = make_config([(latent(heads=2, dim=3, rot_dim=2, vdim=4, kv_rank=5, window=3), None)], width=6)
    W = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed=3).items()}
    P = {k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}
    mx = cfg["layers"][0]["mixer"]
    hs = np.random.default_rng(4).standard_normal((9, 6))
    got = O.latent_attention_mixer(hs, P, mx, 1e-5)
    n = len(hs)
    c = np.stack([O.rms_unit((P["dkv"] @ h)[:5], 1e-5) * P["dkv.norm"] for h in hs])
    kr = np.stack([O.rope_interleaved((P["dkv"] @ h)[5:], p, 2, mx["rot"]["base"]) for p, h in enumerate(hs)])
    mask = np.array([[0 <= i - j < 3 for j in range(n)] for i in range(n)])
    out = np.zeros((n, 8))
    for hd in range(2):
        K = np.concatenate([c @ P["uk"][hd * 3:hd * 3 + 3].T, kr], axis=1)
        Vv = c @ P["uv"][hd * 4:hd * 4 + 4].T
        Q = np.stack([np.concatenate([(P["q"] @ h).reshape(2, 5)[hd, :3], O.rope_interleaved((P["q"] @ h).reshape(2, 5)[hd, 3:], p, 2, mx["rot"]["base"])])
                      for p, h in enumerate(hs)])
        S = np.where(mask, Q @ K.T * mx["scale"], -np.inf)
        Pm = np.exp(S - S.max(axis=1, keepdims=True))
        Pm /= Pm.sum(axis=1, keepdims=True)
        out[:, hd * 4:hd * 4 + 4] = Pm @ Vv
    want = np.stack([P["o"] @ (out[t] / (1 + np.exp(-(P["g"] @ hs[t])))) for t in range(n)])
    assert np.allclose(got, want, atol=1e-9)


def test_routing_keeps_the_best_groups_and_does_not_renormalise():
    mlp = moe(experts=6, top=2, count=3, keep=2)
    z = np.log(np.array([0.30, 0.01, 0.02, 0.25, 0.22, 0.20]))   # groups (0,1) (2,3) (4,5): best members .30 .25 .22
    ids, ws = O.moe_route(np.ones(1), {"router": z[:, None]}, mlp)
    assert ids == [0, 3]                      # expert 4 (0.22) loses its group although it beats experts 1 and 2
    assert np.allclose(ws, [0.30, 0.25])
    ids, ws = O.moe_route(np.ones(1), {"router": z[:, None]}, moe(experts=6, top=3, count=3, keep=3))
    assert ids == [0, 3, 4] and abs(sum(ws) - 0.77) < 1e-12


def test_dense_unit_clamps_before_the_gate():
    P = {"gate": np.array([[3.0], [-3.0]]), "up": np.array([[5.0], [-5.0]]), "down": np.eye(2)}
    y = O.dense_ff(np.ones(1), P, dense(ff=2, limit=2.0))
    assert np.allclose(y, [2 / (1 + np.exp(-1.702 * 2)) * 3.0, -3 / (1 + np.exp(1.702 * 3)) * -1.0])


def test_bf16_rounding_helper_is_round_to_nearest_even():
    a = np.array([1.0, 1.00390625, 1.005859375, -2.5], dtype=np.float32)   # 1 + 2^-8 is a tie: stays 1.0
    assert bf16_round(a).tolist() == [1.0, 1.0, 1.0078125, -2.5]


def test_registry_and_config_errors_come_before_any_device_work(tmp_path):
    from kubeai_b200 import B200Error
    from kubeai_b200.engine import Engine, default_config
    cfg = make_config([(gla(), None)])
    W = random_weights(cfg)
    lim = default_config(manual_step=1)
    with pytest.raises(B200Error, match="not registered"):
        Engine(lim, write_model_dir(tmp_path / "a", dict(cfg, architecture="Other"), W), dtype="float32")
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(B200Error, match="unknown mixer"):
        Engine(lim, write_model_dir(tmp_path / "b", bad, W), dtype="float32")
    bad = json.loads(json.dumps(make_config([(gla(), moe(experts=6, top=5, count=3, keep=2))])))
    with pytest.raises(B200Error, match="router groups"):
        Engine(lim, write_model_dir(tmp_path / "c", bad, W), dtype="float32")
