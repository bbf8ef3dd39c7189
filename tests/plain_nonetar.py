"""A plain, slow restatement of the Nonetar decoder in numpy float64, one function per mechanism.

It shares nothing with the package: it reads a config.json dictionary and a mapping tensor name ->
array, runs whole sequences from position 0 and keeps no cache.  The tests compare the engine (which
runs portions, batches and single tokens against pages and state slots) with it.

Notation: W is the model's width, S the number of residual streams, T the tokens of a sequence.
"""

from __future__ import annotations

import numpy as np


def softplus(x):
    return np.logaddexp(0.0, x)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, weight, eps, one_plus=False):
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight (or 1 + weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    if weight is None:
        return y
    return y * ((1.0 + weight) if one_plus else weight)


def sinusoid(positions, width):
    """[len(positions), width]: entry 2i is sin(p f_i), entry 2i + 1 is cos(p f_i), f_i = 10000^(-2i / width)."""
    out = np.zeros((len(positions), width))
    for n, p in enumerate(positions):
        for c in range(width):
            i = c // 2
            angle = p * 10000.0 ** (-2.0 * i / width)
            out[n, c] = np.sin(angle) if c % 2 == 0 else np.cos(angle)
    return out


def token_shift(h, shift):
    """Row t becomes h[t] + (h[t-1] - h[t]) * shift, with the rows as they were before; row -1 is zero."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (prev - h) * shift


def hyper_read(streams, w_in):
    """streams [S, T, W] -> sum_s w_in[s] streams[s]."""
    return np.einsum("s,stw->tw", w_in, streams)


def hyper_write(streams, y, mix, w_out):
    """new[t'] = sum_s mix[s, t'] old[s] + w_out[t'] y, every stream from the old ones."""
    return np.einsum("sr,stw->rtw", mix, streams) + w_out[:, None, None] * y[None]


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column weighs the token itself), b [C] or None; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    out = np.zeros((T, C))
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += w[:, j] * x[src]
    return out + (0.0 if b is None else b)


def xielu(z, p, q):
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (np.expm1(z) - z) + 0.5 * z
    return np.where(z > 0, pos, neg)


def dense_xielu(h, up, down, act):
    return xielu(h @ up.T, act[0], act[1]) @ down.T


def capped_window_attention(h, P, m, eps):
    """The attention side of the parallel mixer.  P: the side's tensors by their short names; m: its sizes."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ P["q"].T + P["q.b"]).reshape(T, H, D)
    k = (h @ P["k"].T + P["k.b"]).reshape(T, G, D)
    v = (h @ P["v"].T + P["v.b"]).reshape(T, G, Dv)
    q = rms_norm(q, P["q.norm"], eps)
    k = rms_norm(k, P["k.norm"], eps)
    cap = m.get("softcap")
    size = (m.get("mask") or {}).get("size")
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        slope = 2.0 ** (-8.0 * (hd + 1) / H)
        for i in range(T):
            lo = 0 if not size else max(0, i - size + 1)
            js = np.arange(lo, i + 1)
            s = (k[js, g] @ q[i, hd]) * m["scale"] * P["temp"][hd]
            if cap:
                s = cap * np.tanh(s / cap)
            s = s - slope * (i - js)
            w = np.exp(s - s.max())
            out[i, hd] = (w / w.sum()) @ v[js, g]
    return out.reshape(T, H * Dv) @ P["o"].T


def gated_linear_recurrence(h, P, m):
    """The recurrent side of the parallel mixer: two branches, a short convolution, gates per block of
    channels, a diagonal recurrence from a zero state."""
    T = h.shape[0]
    C, nb = m["width"], m["blocks"]
    y = gelu_tanh(h @ P["y"].T + P["y.b"])
    u = causal_conv(h @ P["x"].T + P["x.b"], P["conv"], P["conv.b"])
    bw = C // nb
    ub = u.reshape(T, nb, bw)
    r = sigmoid(np.einsum("bok,tbk->tbo", P["ra"], ub) + P["ra.b"]).reshape(T, C)
    i = sigmoid(np.einsum("bok,tbk->tbo", P["ri"], ub) + P["ri.b"]).reshape(T, C)
    log_a = -8.0 * r * softplus(P["lam"])
    a = np.exp(log_a)
    state = np.zeros(C)
    out = np.zeros((T, C))
    for t in range(T):
        state = a[t] * state + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = state
    return (out * y) @ P["o"].T


def parallel_mixer(h, P, m, eps):
    left = {k[len("left."):]: v for k, v in P.items() if k.startswith("left.")}
    right = {k[len("right."):]: v for k, v in P.items() if k.startswith("right.")}
    return (m["left_scale"] * capped_window_attention(h, left, m["left"], eps)
            + m["right_scale"] * gated_linear_recurrence(h, right, m["right"]))


def state_space_mixer(h, P, m, eps):
    """Selective state space mixer with a scalar decay per head (state N x vdim per head)."""
    T = h.shape[0]
    H, Dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * Dv
    p = h @ P["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P["conv"], P["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, Dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + P["dt_bias"])
    y = np.zeros((T, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((N, Dv))
        rate = np.exp(P["A_log"][hd])
        for t in range(T):
            S = np.exp(-rate * dt[t, hd]) * S + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + P["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_norm(y.reshape(T, ng, inner // ng), None, eps).reshape(T, inner) * P["norm"]
    return y @ P["o"].T


def forward(config, tensors, tokens, layer_outputs=None):
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs``: a list that receives the sum of the
    streams after every layer."""
    W, S, eps = config["width"], int(config["streams"]), config["norm"]["eps"]
    t64 = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    T = len(tokens)
    x = t64["embed"][np.asarray(tokens)] + sinusoid(range(T), W)
    streams = np.stack([x] * S)
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        mix = {k[len(pre) + 4:]: v for k, v in t64.items() if k.startswith(pre + "mix.")}
        u = hyper_read(streams, t64[pre + "hc1.in"])
        h = token_shift(rms_norm(u, t64[pre + "norm1"], eps, one_plus=True), t64[pre + "shift"])
        if layer["type"] == "parallel":
            y = parallel_mixer(h, mix, layer["mixer"], eps)
        elif layer["type"] == "mamba2":
            y = state_space_mixer(h, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        streams = hyper_write(streams, y, t64[pre + "hc1.mix"], t64[pre + "hc1.out"])
        if layer.get("mlp") is not None:
            u = hyper_read(streams, t64[pre + "hc2.in"])
            h = rms_norm(u, t64[pre + "norm2"], eps, one_plus=True)
            y = dense_xielu(h, t64[pre + "mlp.up"], t64[pre + "mlp.down"], t64[pre + "mlp.act"])
            streams = hyper_write(streams, y, t64[pre + "hc2.mix"], t64[pre + "hc2.out"])
        if layer_outputs is not None:
            layer_outputs.append(streams.sum(axis=0))
    x = rms_norm(streams.sum(axis=0), t64["final.norm"], eps, one_plus=True)
    return (x @ t64["head"].T) * config["logit_scale"]
