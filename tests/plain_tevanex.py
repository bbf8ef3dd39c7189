"""A plain, slow restatement of the Tevanex decoder in numpy float64, one function per mechanism.

It shares nothing with the package: it reads a config.json dictionary and a mapping tensor name ->
array, runs whole sequences from position 0 and keeps no cache.  The tests compare the engine (which
runs portions, batches and single tokens against pages and state slots) with it.

Notation: W is the model's width, T the tokens of a sequence, H query heads, G key/value heads, D the
query/key size of a head, Dv its value size.
"""

from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def log_sigmoid(x):
    return -np.logaddexp(0.0, -x)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight (None: no weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def soft_cap(x, cap):
    return cap * np.tanh(x / cap)


# ------------------------------------------------------------------ rotation

def rotary_frequencies(dims, base, scaling=None):
    """(f [dims / 2], factor on cos and sin).  f_i = base^(-2i / dims); with ``scaling`` (factor, original, fast,
    slow) pair i's frequency is blended between f_i and f_i / factor by a ramp over the pair index, and the
    rotation's cos and sin grow by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = np.zeros(half)
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, freqs, grow, layout):
    """x [T, heads, D]: the first ``dims`` channels of every head turn by the angle position * freqs[i]; pair i is
    (i, i + dims / 2) in the layout 'half' and (2i, 2i + 1) in the layout 'pairs'.  The rest passes."""
    out = x.copy()
    half = dims // 2
    pos = np.asarray(list(positions), dtype=np.float64)
    for i in range(half):
        a, b = (i, i + half) if layout == "half" else (2 * i, 2 * i + 1)
        c, s = (np.cos(pos * freqs[i]) * grow)[:, None], (np.sin(pos * freqs[i]) * grow)[:, None]
        u, v = x[:, :, a], x[:, :, b]
        out[:, :, a] = u * c - v * s
        out[:, :, b] = v * c + u * s
    return out


# ------------------------------------------------------------------ attention

def chunk_visible(i, j, size):
    """Query position i sees key position j: not later, and in the same block of ``size`` positions counted from 0."""
    return (j <= i) & (True if size is None else (i // size == j // size))       # numbers or arrays


def masked_attention(q, k, v, scale, size=None, softcap=None, sinks=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence from position 0 -> [T, H, Dv].  ``sinks`` [H]: one more
    term exp(sink_h) in the softmax's denominator, which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    seen = chunk_visible(np.arange(T)[:, None], np.arange(T)[None, :], size)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = soft_cap(s, softcap)
        s = np.where(seen, s, -np.inf)
        top = s.max(axis=1)
        if sinks is not None:
            top = np.maximum(top, sinks[h])
        e = np.exp(s - top[:, None])
        denom = e.sum(axis=1)
        if sinks is not None:
            denom = denom + np.exp(sinks[h] - top)
        out[:, h] = (e @ v[:, g]) / denom[:, None]
    return out


def attention_mixer(h, w, p, m, kind, eps):
    """h [T, W] of one sequence.  ``w``: tensors by name, ``p``: the layer's prefix, ``m``: the mixer's entry of
    config.json, ``kind``: 'attention' (pairs a half apart, a sink per head) or 'attention_2' (neighbouring pairs,
    scaled frequencies, capped scores, an output gate)."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, D)       # over the whole projection, before it is cut into heads
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, D)
    v = v.reshape(T, G, Dv)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        second = kind == "attention_2"
        f, grow = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling") if second else None)
        layout = "pairs" if second else "half"
        q = rotate(q, range(T), int(rot["dims"]), f, grow, layout)
        k = rotate(k, range(T), int(rot["dims"]), f, grow, layout)
    size = int(m["mask"]["size"]) if m.get("mask") else None
    if kind == "attention":
        a = masked_attention(q, k, v, float(m["scale"]), size, None, w[p + "sink"])
    else:
        a = masked_attention(q, k, v, float(m["scale"]), size, float(m["softcap"]) if m.get("softcap") else None, None)
    a = a.reshape(T, H * Dv)
    if kind == "attention_2":
        a = a * sigmoid(h @ w[p + "g"].T)
    return a @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------ matrix memory

def matrix_memory(q, k, v, gi, gf):
    """One head of one sequence from an empty memory.  q, k [T, D] (q already scaled), v [T, Dv], gi and gf [T]: the
    logarithms of the input and the forget gate.  The memory C [D, Dv] and the vector n [D] are kept divided by
    exp(m), m being a running maximum that starts at 0."""
    T, D = q.shape
    C, n, m = np.zeros((D, v.shape[1])), np.zeros(D), 0.0
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        m_new = max(gf[t] + m, gi[t])
        keep, take = math.exp(gf[t] + m - m_new), math.exp(gi[t] - m_new)
        C = keep * C + take * np.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_new
        out[t] = (C.T @ q[t]) / (max(abs(n @ q[t]), math.exp(-m)) + 1e-6)
    return out


def mlstm_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, D, Dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, Dv)
    gi = soft_cap(h @ w[p + "i"].T + w[p + "i.b"], cap)
    gf = log_sigmoid(soft_cap(h @ w[p + "f"].T + w[p + "f.b"], cap))
    o = np.stack([matrix_memory(q[:, a], k[:, a], v[:, a], gi[:, a], gf[:, a]) for a in range(H)], axis=1)
    o = rms_norm(o, None, eps).reshape(T, H * Dv) * w[p + "norm"]       # every head by its own root mean square
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward

def limited_expert(x, gate, up, down, limit):
    """x [T, W] -> [T, W]: g = min(gate x, limit), u = clamp(up x, -limit, limit), down (g sigmoid(1.702 g) (u + 1))."""
    g = np.minimum(x @ gate.T, limit)
    u = np.clip(x @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, top):
    """(chosen expert indices [T, top], their weights [T, top]): the largest sigmoid scores, as they are."""
    s = sigmoid(h @ router.T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def moe(h, w, p, mlp):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    chosen, weight = route(h, w[p + "router"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t], weight[t]):
            q = f"{p}e{e}."
            out[t] += limited_expert((c * h[t])[None], w[q + "gate"], w[q + "up"], w[q + "down"], limit)[0]
    if mlp.get("shared"):
        q = p + "shared."
        y = limited_expert(h, w[q + "gate"], w[q + "up"], w[q + "down"], float(mlp["shared"]["limit"]))
        out += y * sigmoid(h @ w[q + "sg"].T)
    assert E == sum(1 for name in w if name.startswith(p + "e") and name.endswith(".gate"))
    return out


# ------------------------------------------------------------------ the model

def owner(cfg, i):
    """The layer whose tensors layer i uses."""
    j = cfg["layers"][i].get("weights_of")
    return i if j is None else int(j)


def forward(cfg, w, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and, if asked, the stream after every layer)."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner(cfg, i)}."
        kind = layer["type"]
        if kind == "mlstm":
            y = mlstm_mixer(x, w, p + "mix.", layer["mixer"], eps)
        else:
            y = attention_mixer(x, w, p + "mix.", layer["mixer"], kind, eps)
        x = x + mult * rms_norm(y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + mult * rms_norm(moe(x, w, p + "mlp.", layer["mlp"]), w[p + "norm2"], eps)
        after.append(x.copy())
    z = rms_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg["logit_scale"])
    z = soft_cap(z, float(cfg["logit_softcap"])) if cfg.get("logit_softcap") else z
    return (z, after) if keep_layers else z
