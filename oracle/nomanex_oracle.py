"""TEST INFRASTRUCTURE — plain, slow restatement of the Nomanex decoder, one function per mechanism.

Nomanex is a decoder-only model whose layers are *parallel* (one Dynamic-Tanh norm feeds both the mixer and the
feed-forward, their sum is scaled and added to the residual), whose mixers are either gated linear attention (a
per-key-channel decayed outer-product state, carried from token to token) or latent attention (keys and values are
up-projections of one cached low-rank vector, plus one rotated key part shared by all heads, seen through a sliding
window), and whose feed-forwards are either a clamped gated unit or a group-limited mixture of squared-ReLU experts.
The input embedding adds a hashed bigram row.

Everything here runs token by token in float64 on the CPU and shares no code with the CUDA path
(kubeai_b200/csrc/nomanex.cu and the kernels it launches); tests compare the engine against it.

Notation: x residual [width]; h = dyt(x); m = residual_mult; layer: x <- x + m (mixer(h) + ff(h)).
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def dyt(x, w, b, alpha):
    """Dynamic Tanh: no statistics, tanh(alpha x) w + b."""
    return np.tanh(alpha * x) * w + b


def bigram_row(prev, tok, cfg):
    """Row of the bigram table for `tok` preceded by `prev` (None at a sequence's first token: the table's last row)."""
    bg = cfg["embedding"]["bigram"]
    if prev is None:
        return bg["buckets"]
    return (prev * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]


def embed(tokens, W, cfg):
    out = []
    prev = None
    for t in tokens:
        out.append(W["embed"][t] + W["bigram"][bigram_row(prev, t, cfg)])
        prev = t
    return np.stack(out)


def rope_interleaved(vec, pos, dims, base):
    """Rotate pairs (2i, 2i+1), i < dims/2, of the last axis by pos * base^(-2i/dims); the rest passes unchanged."""
    out = vec.copy()
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        u, v = vec[..., 2 * i], vec[..., 2 * i + 1]
        out[..., 2 * i] = u * math.cos(a) - v * math.sin(a)
        out[..., 2 * i + 1] = v * math.cos(a) + u * math.sin(a)
    return out


def gla_decay(h, P, mx):
    """Per-key-channel decay in (0, 1): sigmoid(W_a2 W_a1 h + b)^(1/tau), laid out [heads, dim]."""
    z = P["a2"] @ (P["a1"] @ h) + P["a2.b"]
    return (sigmoid(z) ** (1.0 / mx["tau"])).reshape(mx["heads"], mx["dim"])


def gla_mixer(hs, P, mx, eps):
    """Gated linear attention over a whole sequence hs [n, width], state from zero."""
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    S = np.zeros((H, D, Dv))
    out = []
    for h in hs:
        q = (P["q"] @ h).reshape(H, D) * D ** -0.5
        k = (P["k"] @ h).reshape(H, D)
        v = (P["v"] @ h).reshape(H, Dv)
        a = gla_decay(h, P, mx)
        S = a[:, :, None] * S + k[:, :, None] * v[:, None, :]
        o = np.einsum("hdv,hd->hv", S, q)
        o = rms_unit(o, eps) * P["norm"]
        g = P["g"] @ h
        y = o.reshape(-1) * (g * sigmoid(g))
        out.append(P["o"] @ y)
    return np.stack(out)


def latent_attention_mixer(hs, P, mx, eps):
    """Sliding-window attention whose keys and values are rebuilt from a cached latent c and one shared rotated key."""
    H, D, R, Dv, C = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    rot, win, scale = mx["rot"], mx["mask"]["size"], mx["scale"]
    cs, krs, out = [], [], []
    for p, h in enumerate(hs):
        q = (P["q"] @ h).reshape(H, D + R)
        qn, qr = q[:, :D], rope_interleaved(q[:, D:], p, rot["dims"], rot["base"])
        d = P["dkv"] @ h
        cs.append(rms_unit(d[:C], eps) * P["dkv.norm"])
        krs.append(rope_interleaved(d[C:], p, rot["dims"], rot["base"]))
        lo = max(0, p - win + 1)
        heads = []
        for hd in range(H):
            Wk = P["uk"][hd * D:(hd + 1) * D]
            Wv = P["uv"][hd * Dv:(hd + 1) * Dv]
            s = np.array([(qn[hd] @ (Wk @ cs[j]) + qr[hd] @ krs[j]) * scale for j in range(lo, p + 1)])
            w = np.exp(s - s.max())
            w /= w.sum()
            heads.append(sum(w[j - lo] * (Wv @ cs[j]) for j in range(lo, p + 1)))
        y = np.concatenate(heads) * sigmoid(P["g"] @ h)
        out.append(P["o"] @ y)
    return np.stack(out)


def dense_ff(h, P, mlp):
    lim = mlp["limit"]
    g = np.minimum(P["gate"] @ h, lim)
    u = np.clip(P["up"] @ h, -lim, lim)
    return P["down"] @ (g * sigmoid(1.702 * g) * (u + 1.0))


def moe_route(h, P, mlp):
    """(expert ids, weights): softmax over all experts, groups of neighbours ranked by their best member, only the
    kept groups' experts are eligible, the `top` largest scores win and are used as they are."""
    r = mlp["router"]
    E, top, G, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    z = (P["router"] @ h).astype(np.float64)
    s = np.exp(z - z.max())
    s /= s.sum()
    per = E // G
    gscore = s.reshape(G, per).max(axis=1)
    kept = np.argsort(-gscore, kind="stable")[:keep]
    allowed = np.zeros(E, bool)
    for g in kept:
        allowed[g * per:(g + 1) * per] = True
    order = [e for e in np.argsort(-s, kind="stable") if allowed[e]][:top]
    return order, [s[e] for e in order]


def moe_ff(h, P, mlp):
    ids, ws = moe_route(h, P, mlp)
    y = 0.0
    for e, w in zip(ids, ws):
        a = np.maximum(P["e%d.up" % e] @ h, 0.0) ** 2
        y = y + w * (P["e%d.down" % e] @ a)
    return y


class NomanexOracle:
    """cfg: the config.json dictionary; W: name -> float64 array (already rounded to the stored dtype)."""

    def __init__(self, cfg, W):
        self.cfg = cfg
        self.W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}

    def _params(self, layer, part):
        pre = "l%d.%s." % (layer, part)
        return {k[len(pre):]: v for k, v in self.W.items() if k.startswith(pre)}

    def _norm(self, x, name):
        return dyt(x, self.W[name], self.W[name + ".b"], float(np.asarray(self.W[name + ".alpha"]).reshape(-1)[0]))

    def forward(self, tokens, return_layers=False):
        """Logits [n, vocab] of one sequence from position 0 (and the residual after every layer run)."""
        cfg, eps, m = self.cfg, self.cfg["norm"]["eps"], self.cfg["residual_mult"]
        x = embed(tokens, self.W, cfg)
        trace = []
        for i, ly in enumerate(cfg["layers"]):
            src = i
            while "weights_of" in cfg["layers"][src]:      # a layer without tensors of its own follows the reference
                src = cfg["layers"][src]["weights_of"]
            hs = self._norm(x, "l%d.norm1" % src)
            mix = self._params(src, "mix")
            if ly["type"] == "gla":
                a = gla_mixer(hs, mix, ly["mixer"], eps)
            elif ly["type"] == "latent_attention":
                a = latent_attention_mixer(hs, mix, ly["mixer"], eps)
            else:
                raise ValueError(ly["type"])
            mlp = ly.get("mlp")
            if mlp is None:
                f = 0.0
            else:
                Pm = self._params(src, "mlp")
                f = np.stack([(dense_ff if mlp["kind"] == "dense" else moe_ff)(h, Pm, mlp) for h in hs])
            x = x + m * (a + f)
            trace.append(x.copy())
        logits = self._norm(x, "final.norm") @ self.W["head"].T
        return (logits, np.stack(trace)) if return_layers else logits

    def greedy(self, prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(np.argmax(self.forward(toks)[-1])))
        return toks[len(prompt):]
