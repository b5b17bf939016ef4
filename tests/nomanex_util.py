"""Helpers for the Nomanex tests: small configurations, random bf16-representable weights, a model directory
(config.json + model.safetensors) written from them, and the slow oracle over the same numbers."""
from __future__ import annotations

import json
import os
import struct

import numpy as np

from oracle.nomanex_oracle import NomanexOracle


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), returned as float32."""
    a = np.asarray(a, dtype=np.float32)
    u = a.reshape(-1).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def gla(heads=2, dim=8, vdim=8, tau=8.0):
    return "gla", dict(heads=heads, dim=dim, vdim=vdim, tau=tau)


def latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=12, window=6, base=100.0, rot_dims=None, scale=None):
    mx = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, mask=dict(size=window),
              rot=dict(base=base, dims=rot_dim if rot_dims is None else rot_dims),
              scale=(dim + rot_dim) ** -0.5 if scale is None else scale)
    return "latent_attention", mx


def dense(ff=24, limit=1.5):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(experts=6, top=2, count=3, keep=2, ff=8):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, groups=dict(count=count, keep=keep)))


def make_config(layers, width=24, vocab=40, buckets=13, mul_prev=7, mul_cur=3, eps=1e-5, mult=0.6):
    """layers: list of ((type, mixer), mlp or None) or ("weights_of", j)."""
    out = []
    for ly in layers:
        if ly[0] == "weights_of":
            src = dict(out[ly[1]])
            src["weights_of"] = ly[1]
            out.append(src)
        else:
            (ty, mx), mlp = ly
            out.append(dict(type=ty, mixer=mx, mlp=mlp))
    return dict(architecture="Nomanex", vocab=vocab, width=width, residual_mult=mult, norm=dict(eps=eps),
                embedding=dict(bigram=dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)), layers=out)


def random_weights(cfg, seed=0, a_rank=4, q_gain=1.0):
    """name -> float32 array whose values are exact in bfloat16."""
    rng = np.random.default_rng(seed)
    Wd = cfg["width"]
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = bf16_round(rng.standard_normal((rows, cols)).astype(np.float32) * gain / np.sqrt(cols))

    def norm(name):
        W[name] = bf16_round(1.0 + 0.2 * rng.standard_normal(Wd).astype(np.float32))
        W[name + ".b"] = bf16_round(0.1 * rng.standard_normal(Wd).astype(np.float32))
        W[name + ".alpha"] = bf16_round(np.array(0.7 + 0.2 * rng.random(), dtype=np.float32))

    W["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], Wd)).astype(np.float32))
    W["bigram"] = bf16_round(0.5 * rng.standard_normal((cfg["embedding"]["bigram"]["buckets"] + 1, Wd)).astype(np.float32))
    mat("head", cfg["vocab"], Wd, 2.0)
    norm("final.norm")
    for i, ly in enumerate(cfg["layers"]):
        if "weights_of" in ly:
            continue
        p, mx = "l%d." % i, ly["mixer"]
        norm(p + "norm1")
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        if ly["type"] == "gla":
            mat(p + "mix.q", H * D, Wd, 2.0 * q_gain)
            mat(p + "mix.k", H * D, Wd, 2.0)
            mat(p + "mix.v", H * Dv, Wd, 2.0)
            mat(p + "mix.g", H * Dv, Wd, 2.0)
            mat(p + "mix.o", Wd, H * Dv, 2.0)
            mat(p + "mix.a1", a_rank, Wd, 2.0)
            mat(p + "mix.a2", H * D, a_rank, 2.0)
            W[p + "mix.a2.b"] = bf16_round(2.0 + rng.standard_normal(H * D).astype(np.float32))
            W[p + "mix.norm"] = bf16_round(1.0 + 0.2 * rng.standard_normal(Dv).astype(np.float32))
        else:
            R, C = mx["rot_dim"], mx["kv_rank"]
            mat(p + "mix.q", H * (D + R), Wd, 3.0 * q_gain)
            mat(p + "mix.dkv", C + R, Wd, 2.0)
            W[p + "mix.dkv.norm"] = bf16_round(1.0 + 0.2 * rng.standard_normal(C).astype(np.float32))
            mat(p + "mix.uk", H * D, C, 2.0)
            mat(p + "mix.uv", H * Dv, C, 2.0)
            mat(p + "mix.g", H * Dv, Wd, 2.0)
            mat(p + "mix.o", Wd, H * Dv, 2.0)
        mlp = ly["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], Wd, 3.0)
            mat(p + "mlp.up", mlp["ff"], Wd, 3.0)
            mat(p + "mlp.down", Wd, mlp["ff"], 2.0)
        else:
            mat(p + "mlp.router", mlp["router"]["experts"], Wd, 4.0)
            for e in range(mlp["router"]["experts"]):
                mat(p + "mlp.e%d.up" % e, mlp["expert"]["ff"], Wd, 2.0)
                mat(p + "mlp.e%d.down" % e, Wd, mlp["expert"]["ff"], 2.0)
    return W


def write_safetensors(path, W):
    """The safetensors layout: 8-byte little-endian header length, JSON header, raw data (all tensors as BF16)."""
    header, blobs, at = {}, [], 0
    for name, a in W.items():
        bits = (np.asarray(a, dtype=np.float32).reshape(-1).view(np.uint32) >> 16).astype(np.uint16)
        raw = bits.tobytes()
        header[name] = dict(dtype="BF16", shape=list(a.shape), data_offsets=[at, at + len(raw)])
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(d, cfg, W):
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), W)
    return str(d)


def oracle_for(cfg, W):
    return NomanexOracle(cfg, W)


def open_engine(model_dir, dtype="float32", max_tokens=512, max_seqs=4, budget=None, blocks=None, **kw):
    from kubeai_b200.engine import Engine, default_config
    cfg = default_config(manual_step=1, enable_prefix_caching=0, max_num_seqs=max_seqs,
                         max_batched_tokens=budget or max_tokens, max_model_len=max_tokens,
                         num_kv_blocks=blocks or (max_tokens + 15) // 16 * max_seqs, **kw)
    return Engine(cfg, model_dir, dtype=dtype)


def feed_whole(e, tokens, want=None):
    r = e.feed_open()
    out = e.feed_step([(r, tokens, list(range(len(tokens))) if want is None else want)])
    e.feed_close(r)
    return out


def feed_portions(e, tokens, sizes):
    """The sequence in portions of the given sizes (the last size repeats); logits of every position."""
    r = e.feed_open()
    outs, at, i = [], 0, 0
    while at < len(tokens):
        n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
        outs.append(e.feed_step([(r, tokens[at:at + n], list(range(n)))]))
        at += n
        i += 1
    e.feed_close(r)
    return np.concatenate(outs)


def rel_err(got, want):
    """Per row: RMS over the vocabulary of the mean-free difference, relative to the RMS of the mean-free reference."""
    d = np.asarray(got, dtype=np.float64) - want
    d = d - d.mean(axis=-1, keepdims=True)
    w = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((d ** 2).mean(axis=-1)) / np.sqrt((w ** 2).mean())
