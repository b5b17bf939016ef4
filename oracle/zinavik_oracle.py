"""TEST INFRASTRUCTURE — plain, slow restatement of the Zinavik decoder, one function per mechanism.

Zinavik keeps several residual streams (hyper-connections): a sublayer reads a weighted sum of the streams through an
RMS norm and its output is written back into every stream while the streams are mixed among themselves.  A layer is a
mixer and, optionally, a feed-forward.  The mixer is two branches on the same input, added with fixed weights: "left" is
softmax attention with grouped key/value heads, rotary positions on interleaved pairs under YaRN frequency scaling, a
weightless RMS norm of every rotated query and key head, a sliding window that also keeps the first tokens, and a
sigmoid output gate; "right" is linear attention with one constant decay per head on SiLU-activated inputs, an RMS norm
over the concatenated heads and a sigmoid gate.  The feed-forward is a mixture of clamped gated experts chosen by the
largest sigmoid router scores, whose score scales the expert's *input*, plus a shared expert behind a one-number gate.
A range of layers may run several times with the same weights, each run with its own cache and state.

Everything here runs token by token in float64 on the CPU: the functions take the sequence so far and return the
newest token's output, keeping their caches in plain Python lists.  They share no code with the CUDA path
(kubeai_b200/csrc/zinavik.cu and the kernels it launches); tests compare the engine against them.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


# ---------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """Angular frequency of every pair and the common magnitude of cos and sin.  Plain: f_i = base^(-2i/dims).  With
    scaling {factor, original, fast, slow}: the pair index at which a rotation of `t` turns fits into `original` positions
    is d(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = floor(d(fast)) and hi = ceil(d(slow)) a ramp moves
    the frequency from f_i to f_i / factor; the magnitude is 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return freqs, 1.0

    def d(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(d(sc["fast"])), 0)
    hi = min(math.ceil(d(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(vec, pos, rot):
    """Rotate the pairs (2i, 2i+1), i < dims/2, of the last axis of vec by pos * f_i; dimensions past dims pass unchanged."""
    if not rot or not rot.get("dims"):
        return vec.copy()
    freqs, mag = rotary_frequencies(rot)
    out = vec.copy()
    for i, f in enumerate(freqs):
        c, s = math.cos(pos * f) * mag, math.sin(pos * f) * mag
        u, v = vec[..., 2 * i], vec[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ---------------------------------------------------------------- left branch: windowed softmax attention
def visible(i, j, mask):
    """May the token at position i see the key at position j?"""
    if j > i:
        return False
    return i - j < mask.get("size", 1 << 60) or j < mask.get("keep_first", 0)


class LeftBranch:
    def __init__(self, P, mx, eps):
        self.P, self.mx, self.eps = P, mx, eps
        self.keys, self.values = [], []     # per position: [kv_heads, dim], [kv_heads, vdim]

    def step(self, h):
        mx, P = self.mx, self.P
        H, G, D, Dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
        pos = len(self.keys)
        q = unit_rms(rotate((P["q"] @ h).reshape(H, D), pos, mx.get("rot")), self.eps)
        k = unit_rms(rotate((P["k"] @ h).reshape(G, D), pos, mx.get("rot")), self.eps)
        self.keys.append(k)
        self.values.append((P["v"] @ h).reshape(G, Dv))
        seen = [j for j in range(pos + 1) if visible(pos, j, mx.get("mask", {}))]
        heads = []
        for hd in range(H):
            g = hd // (H // G)
            s = np.array([q[hd] @ self.keys[j][g] for j in seen]) * mx["scale"]
            w = np.exp(s - s.max())
            w /= w.sum()
            heads.append(sum(wj * self.values[j][g] for wj, j in zip(w, seen)))
        return P["o"] @ (np.concatenate(heads) * sigmoid(P["g"] @ h))


# ---------------------------------------------------------------- right branch: constant-decay linear attention
class RightBranch:
    def __init__(self, P, mx, eps):
        self.P, self.mx, self.eps = P, mx, eps
        self.S = np.zeros((mx["heads"], mx["dim"], mx["vdim"]))

    def step(self, h):
        mx, P = self.mx, self.P
        H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
        q, k, v = silu(P["q"] @ h).reshape(H, D), silu(P["k"] @ h).reshape(H, D), silu(P["v"] @ h).reshape(H, Dv)
        decay = mx["decay"] if isinstance(mx["decay"], list) else [mx["decay"]] * H
        out = []
        for hd in range(H):
            self.S[hd] = decay[hd] * self.S[hd] + np.outer(k[hd], v[hd])
            out.append(self.S[hd].T @ q[hd])
        o = rms_norm(np.concatenate(out), P["norm"], self.eps) * sigmoid(P["g"] @ h)
        return P["o"] @ o


# ---------------------------------------------------------------- feed-forward
def clamped_expert(P, h, limit):
    g = np.minimum(P["gate"] @ h, limit)
    u = np.clip(P["up"] @ h, -limit, limit)
    return P["down"] @ (g * sigmoid(1.702 * g) * (u + 1.0))


def route(P, h, router):
    """Chosen experts (largest sigmoid score first, ties to the lower index) and their scores."""
    s = sigmoid(P["router"] @ h)
    order = sorted(range(len(s)), key=lambda e: (-s[e], e))[: router["top"]]
    return order, [s[e] for e in order]


def route_margin(P, h, router):
    """Gap between the last chosen score and the best one left out (inf when every expert is chosen)."""
    s = sorted(sigmoid(P["router"] @ h), reverse=True)
    return s[router["top"] - 1] - s[router["top"]] if router["top"] < len(s) else float("inf")


def moe_ff(P, mlp, h):
    chosen, scores = route(P, h, mlp["router"])
    y = np.zeros_like(h)
    for e, s in zip(chosen, scores):
        y = y + clamped_expert(sub(P, "e%d." % e), s * h, mlp["expert"]["limit"])
    if mlp.get("shared"):
        sh = sub(P, "shared.")
        y = y + sigmoid(sh["sg"].reshape(-1) @ h) * clamped_expert(sh, h, mlp["shared"]["limit"])
    return y


# ---------------------------------------------------------------- hyper-connections
def streams_read(xs, hc):
    """The sublayer's input: sum_s in[s] x_s (one plain residual when there are no stream weights)."""
    if hc is None:
        return xs[0]
    return sum(hc["in"][s] * xs[s] for s in range(len(xs)))


def streams_write(xs, hc, y):
    """All streams at once from the old ones: x_j <- sum_s mix[s, j] x_s + out[j] y."""
    if hc is None:
        return [xs[0] + y]
    n = len(xs)
    return [sum(hc["mix"][s, j] * xs[s] for s in range(n)) + hc["out"][j] * y for j in range(n)]


def sub(P, prefix):
    return {k[len(prefix):]: v for k, v in P.items() if k.startswith(prefix)}


def layer_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


class ZinavikOracle:
    def __init__(self, cfg, W):
        self.cfg = cfg
        self.W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
        self.eps = cfg["norm"]["eps"]
        self.order = layer_order(cfg)

    def _hc(self, layer, q):
        if not self.cfg.get("streams"):
            return None
        return sub(self.W, "l%d.hc%d." % (layer, q))

    def new_state(self):
        runs = []
        for li in self.order:
            mx = self.cfg["layers"][li]["mixer"]
            runs.append((LeftBranch(sub(self.W, "l%d.mix.left." % li), mx["left"], self.eps),
                         RightBranch(sub(self.W, "l%d.mix.right." % li), mx["right"], self.eps)))
        return runs

    def step(self, state, token, layers_out=None, margins_out=None):
        """Advance one sequence by one token; returns its logits.  margins_out collects every router's decision margin."""
        cfg, W, eps = self.cfg, self.W, self.eps
        x0 = W["embed"][token] * cfg.get("embedding", {}).get("scale", 1.0)
        xs = [x0.copy() for _ in range(cfg.get("streams") or 1)]
        for li, (left, right) in zip(self.order, state):
            L = cfg["layers"][li]
            mx = L["mixer"]
            h = rms_norm(streams_read(xs, self._hc(li, 1)), W["l%d.norm1" % li], eps)
            y = mx.get("left_scale", 1.0) * left.step(h) + mx.get("right_scale", 1.0) * right.step(h)
            xs = streams_write(xs, self._hc(li, 1), y)
            if L.get("mlp"):
                h = rms_norm(streams_read(xs, self._hc(li, 2)), W["l%d.norm2" % li], eps)
                if margins_out is not None:
                    margins_out.append(route_margin(sub(W, "l%d.mlp." % li), h, L["mlp"]["router"]))
                xs = streams_write(xs, self._hc(li, 2), moe_ff(sub(W, "l%d.mlp." % li), L["mlp"], h))
            if layers_out is not None:
                layers_out.append(sum(xs))
        return W["embed"] @ rms_norm(sum(xs), W["final.norm"], eps)

    def forward(self, tokens, return_layers=False):
        """Logits of every position [T, vocab]; with return_layers also the summed streams after every layer run
        [runs, T, width]."""
        state = self.new_state()
        logits, per_tok = [], []
        for t in tokens:
            lo = []
            logits.append(self.step(state, int(t), lo))
            per_tok.append(lo)
        out = np.stack(logits)
        if return_layers:
            return out, np.stack([[per_tok[t][r] for t in range(len(tokens))] for r in range(len(self.order))])
        return out

    def routing_margins(self, tokens):
        """Per position, the smallest router margin over all layer runs (inf for a model without routing decisions)."""
        state = self.new_state()
        out = []
        for t in tokens:
            m = []
            self.step(state, int(t), None, m)
            out.append(min(m) if m else float("inf"))
        return np.array(out)

    def generate(self, prompt, n):
        """Greedy continuation: (tokens, smallest top-1 / top-2 margin met on the way)."""
        state = self.new_state()
        lg = None
        for t in prompt:
            lg = self.step(state, int(t))
        out, margin = [], float("inf")
        for _ in range(n):
            top = np.sort(lg)[-2:]
            margin = min(margin, top[1] - top[0])
            nxt = int(np.argmax(lg))
            out.append(nxt)
            lg = self.step(state, nxt)
        return out, margin
