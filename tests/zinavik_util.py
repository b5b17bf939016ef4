"""Helpers for the Zinavik tests: small configurations, random bf16-representable weights (optionally with one planted
query/key pair whose score stands out), a model directory written from them, and the slow oracle over the same numbers."""
from __future__ import annotations

import numpy as np

from nomanex_util import bf16_round, feed_portions, feed_whole, open_engine, rel_err, write_model_dir  # noqa: F401  (re-exported)
from oracle.zinavik_oracle import ZinavikOracle


def left(heads=4, kv_heads=2, dim=8, vdim=6, window=7, keep_first=3, rot_dims=None, base=100.0, scaling="default", scale=0.4):
    rot = dict(base=base, dims=dim if rot_dims is None else rot_dims)
    if scaling == "default":
        scaling = dict(factor=4.0, original=16, fast=4.0, slow=0.5)
    if scaling:
        rot["scaling"] = scaling
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=window, keep_first=keep_first), rot=rot, scale=scale)


def right(heads=2, dim=8, vdim=8, decay=None):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=decay if decay is not None else [0.5 + 0.49 * i / max(heads - 1, 1) for i in range(heads)])


def moe(experts=5, top=2, ff=8, limit=1.5, shared=12, shared_limit=1.0):
    m = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))
    if shared:
        m["shared"] = dict(ff=shared, limit=shared_limit)
    return m


def layer(l=None, r=None, mlp="default", left_scale=1.2, right_scale=0.8):
    return dict(type="parallel", mixer=dict(left=l or left(), right=r or right(), left_scale=left_scale, right_scale=right_scale),
                mlp=moe() if mlp == "default" else mlp)


def make_config(layers, width=24, vocab=40, streams=2, loop=None, eps=1e-5, emb_scale=3.0):
    cfg = dict(architecture="Zinavik", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=emb_scale), layers=layers)
    if streams is not None:
        cfg["streams"] = streams
    if loop:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


def random_weights(cfg, seed=0, q_gain=1.0):
    """name -> float32 array whose values are exact in bfloat16."""
    rng = np.random.default_rng(seed)
    Wd, ns = cfg["width"], cfg.get("streams")
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)).astype(np.float32) * gain / np.sqrt(cols))

    def norm(name, n):
        W[name] = bf16_round(1.0 + 0.2 * rng.standard_normal(n).astype(np.float32))

    def hc(prefix):
        if not ns:
            return
        W[prefix + "in"] = bf16_round(1.0 / ns + 0.3 * rng.standard_normal(ns).astype(np.float32))
        W[prefix + "out"] = bf16_round(0.7 + 0.3 * rng.standard_normal(ns).astype(np.float32))
        W[prefix + "mix"] = bf16_round(np.eye(ns, dtype=np.float32) * 0.8 + 0.2 * rng.standard_normal((ns, ns)).astype(np.float32))

    W["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], Wd)).astype(np.float32) * 0.5)
    norm("final.norm", Wd)
    for i, ly in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, ly["mixer"]
        norm(p + "norm1", Wd)
        hc(p + "hc1.")
        l, r = mx["left"], mx["right"]
        G = l.get("kv_heads", l["heads"])
        mat(p + "mix.left.q", l["heads"] * l["dim"], Wd, 2.0 * q_gain)
        mat(p + "mix.left.k", G * l["dim"], Wd, 2.0)
        mat(p + "mix.left.v", G * l["vdim"], Wd, 2.0)
        mat(p + "mix.left.g", l["heads"] * l["vdim"], Wd, 2.0)
        mat(p + "mix.left.o", Wd, l["heads"] * l["vdim"], 2.0)
        mat(p + "mix.right.q", r["heads"] * r["dim"], Wd, 2.0)
        mat(p + "mix.right.k", r["heads"] * r["dim"], Wd, 2.0)
        mat(p + "mix.right.v", r["heads"] * r["vdim"], Wd, 2.0)
        mat(p + "mix.right.g", r["heads"] * r["vdim"], Wd, 2.0)
        mat(p + "mix.right.o", Wd, r["heads"] * r["vdim"], 2.0)
        norm(p + "mix.right.norm", r["heads"] * r["vdim"])
        mlp = ly.get("mlp")
        if not mlp:
            continue
        norm(p + "norm2", Wd)
        hc(p + "hc2.")
        mat(p + "mlp.router", mlp["router"]["experts"], Wd, 3.0)
        for e in range(mlp["router"]["experts"]):
            mat(p + "mlp.e%d.gate" % e, mlp["expert"]["ff"], Wd, 3.0)
            mat(p + "mlp.e%d.up" % e, mlp["expert"]["ff"], Wd, 3.0)
            mat(p + "mlp.e%d.down" % e, Wd, mlp["expert"]["ff"], 2.0)
        if mlp.get("shared"):
            mat(p + "mlp.shared.gate", mlp["shared"]["ff"], Wd, 3.0)
            mat(p + "mlp.shared.up", mlp["shared"]["ff"], Wd, 3.0)
            mat(p + "mlp.shared.down", Wd, mlp["shared"]["ff"], 2.0)
            mat(p + "mlp.shared.sg", 1, Wd, 3.0)
    return W


def plant_pair(cfg, W, query_token, key_token, layer=0, gain=6.0):
    """Make the left branch of `layer` (it must be the first layer, whose input depends on the token alone) score
    key_token's key far above every other key for query_token's queries.  Every key head's projection gets a rank-one
    term q_dir sel^T: sel picks out key_token's normed input and is orthogonal to every other token's (the vocabulary
    must not be larger than the width), q_dir points along the unrotated dimensions of query_token's query (first query
    head of the key head's group).  With unrotated dimensions in the majority and a sharp softmax (config scale), a query_token position then
    copies the values of the visible key_token positions, and its logits change visibly when one of them becomes
    invisible."""
    mx = cfg["layers"][layer]["mixer"]["left"]
    H, G, D = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"]
    eps = cfg["norm"]["eps"]
    ns = cfg.get("streams")
    p = "l%d." % layer
    assert cfg["vocab"] <= cfg["width"]
    x = W["embed"].astype(np.float64) * cfg["embedding"]["scale"] * (W[p + "hc1.in"].astype(np.float64).sum() if ns else 1.0)
    hs = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * W[p + "norm1"].astype(np.float64)      # [vocab, width]
    pick = np.zeros(cfg["vocab"])
    pick[key_token] = 1.0
    sel = np.linalg.lstsq(hs, pick, rcond=None)[0]
    Wk = W[p + "mix.left.k"].astype(np.float64).reshape(G, D, -1)
    Wq = W[p + "mix.left.q"].astype(np.float64).reshape(H, D, -1)
    for g in range(G):
        q = Wq[g * (H // G)] @ hs[query_token]
        q[:(mx.get("rot") or {}).get("dims", 0)] = 0.0        # rotated dimensions turn with the distance: leave them out
        Wk[g] += gain * np.linalg.norm(Wk[g] @ hs[key_token]) * np.outer(q / np.linalg.norm(q), sel)
    W[p + "mix.left.k"] = bf16_round(Wk.reshape(G * D, -1).astype(np.float32))
    return W


def oracle_for(cfg, W):
    return ZinavikOracle(cfg, W)
