"""Nonetar without a GPU: the configuration, the model description and its tensor names, what each layer asks of the
cache, and the plain restatement checked against second formulations of its mechanisms."""

import copy

import numpy as np
import pytest

import plain_nonetar as S
import tiny_nonetar as tiny


def _parse(cfg):
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return arch, arch.parse_config(cfg)


def test_description_names_every_tensor():
    arch, cfg = _parse(tiny.MIXED)
    spec = arch.build_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 4] and all(e.before is None for e in spec.schedule)
    assert [layer.block for layer in spec.layers] == ["hyper_prenorm", "hyper_prenorm", "hyper_prenorm_mixer_only",
                                                      "hyper_prenorm", "hyper_prenorm"]
    names = tiny.expected(tiny.MIXED)
    assert names["embed"].shape == (101, 48) and names["head"].shape == (101, 48) and names["final.norm"].shape == (48,)
    # state-space duality: [z | x | B | C | dt] rows of the input product, x B C channels of the convolution
    assert names["l0.mix.in"].shape == (2 * 48 + 2 * 2 * 10 + 4, 48) and names["l0.mix.conv"].shape == (48 + 40, 4)
    assert names["l0.mix.A_log"].shape == (4,) and names["l0.mix.norm"].shape == (48,) and names["l0.mix.o"].shape == (48, 48)
    assert names["l3.mix.in"].shape == (2 * 32 + 2 * 24 + 2, 48) and names["l3.mix.conv"].shape == (32 + 48, 2)
    # attention beside the recurrence
    assert names["l1.mix.left.q"].shape == (64, 48) and names["l1.mix.left.k"].shape == (32, 48)
    assert names["l1.mix.left.v"].shape == (48, 48) and names["l1.mix.left.v.b"].shape == (48,)
    assert names["l1.mix.left.q.norm"].shape == (16,) and names["l1.mix.left.temp"].shape == (4,)
    assert names["l1.mix.left.o"].shape == (48, 96)
    assert names["l1.mix.right.ra"].shape == (3, 12, 12) and names["l1.mix.right.ri.b"].shape == (3, 12)
    assert names["l1.mix.right.conv"].shape == (36, 3) and names["l1.mix.right.lam"].shape == (36,)
    assert names["l4.mix.right.ra"].shape == (5, 8, 8) and names["l4.mix.left.k"].shape == (24, 48)
    # the streams' tensors, the shift, and nothing of a feed-forward where the layer has none
    assert names["l1.hc1.mix"].shape == (3, 3) and names["l1.hc2.in"].shape == (3,) and names["l0.shift"].shape == (48,)
    assert names["l1.mlp.up"].shape == (24, 48) and names["l1.mlp.act"].shape == (2,)
    assert not any(n.startswith(("l2.mlp", "l2.hc2", "l2.norm2")) for n in names)
    assert "l2.hc1.out" in names and "l2.norm1" in names


def test_what_the_config_leaves_out_is_not_there():
    cfg = tiny.config([tiny.parallel(tiny.left(size=None, softcap=None))], streams=1)
    arch, parsed = _parse(cfg)
    spec = arch.build_spec(parsed)
    att = spec.layers[0].parts["mixer"].params["left"].params
    assert att["window"] is None and att["softcap"] is None
    assert tiny.expected(cfg)["l0.hc1.mix"].shape == (1, 1)


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("blocks"), "blocks"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mixer"].pop("norm_groups"), "norm_groups"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "sparse"),
    (lambda c: c["layers"][1].update(type="convolution"), "convolution"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "grouped"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][0]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][0]["mixer"].update(norm_groups=5), "equal parts"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(breakage, needle):
    from kv_cache_optimization_for_llm_b200.config import ConfigError
    cfg = copy.deepcopy(tiny.MIXED)
    breakage(cfg)
    with pytest.raises(ConfigError, match=needle):
        _parse(cfg)


# --------------------------------------------------------------------------- the plain model against second formulations

def test_one_stream_with_unit_weights_is_the_ordinary_residual():
    rng = np.random.default_rng(0)
    x, y = rng.normal(size=(1, 5, 7)), rng.normal(size=(5, 7))
    one = np.ones(1)
    assert np.allclose(S.hyper_read(x, one), x[0])
    assert np.allclose(S.hyper_write(x, y, np.ones((1, 1)), one)[0], x[0] + y)


def test_streams_are_mixed_from_the_old_ones_and_indexed_from_to():
    rng = np.random.default_rng(1)
    x, y = rng.normal(size=(3, 4, 5)), rng.normal(size=(4, 5))
    mix, out = rng.normal(size=(3, 3)), rng.normal(size=3)
    new = S.hyper_write(x, y, mix, out)
    for to in range(3):
        want = sum(mix[frm, to] * x[frm] for frm in range(3)) + out[to] * y
        assert np.allclose(new[to], want)


def test_token_shift_reads_the_unshifted_previous_row():
    rng = np.random.default_rng(2)
    h, mu = rng.normal(size=(6, 4)), rng.uniform(size=4)
    got = S.token_shift(h, mu)
    assert np.allclose(got[0], h[0] * (1 - mu))
    for t in range(1, 6):
        assert np.allclose(got[t], (1 - mu) * h[t] + mu * h[t - 1])


def test_position_vector_interleaves_sine_and_cosine():
    got = S.sinusoid([0, 3, 17], 10)
    f = 10000.0 ** (-np.arange(5) * 2.0 / 10)
    for n, p in enumerate([0, 3, 17]):
        assert np.allclose(got[n, 0::2], np.sin(p * f)) and np.allclose(got[n, 1::2], np.cos(p * f))


def test_xielu_is_smooth_at_zero_and_quadratic_above():
    p, q = 0.3, -0.4
    e = 1e-6
    assert abs(S.xielu(np.array(e), p, q) - S.xielu(np.array(-e), p, q)) < 2e-6
    slope_up = (S.xielu(np.array(e), p, q) - S.xielu(np.array(0.0), p, q)) / e
    slope_dn = (S.xielu(np.array(0.0), p, q) - S.xielu(np.array(-e), p, q)) / e
    assert abs(slope_up - 0.5) < 1e-4 and abs(slope_dn - 0.5) < 1e-4
    z = np.array([2.0])
    assert np.allclose(S.xielu(z, p, q), np.log1p(np.exp(p)) * 4.0 + 1.0)
    z = np.array([-30.0])        # far below zero: a line of slope -softplus(q)
    assert np.allclose(S.xielu(z, p, q), (0.5 + np.log1p(np.exp(q))) * (-1.0 + 30.0) - 15.0)


def _left_weights(rng, W, m):
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"q": rng.normal(size=(H * D, W)), "q.b": rng.normal(size=H * D), "k": rng.normal(size=(G * D, W)),
            "k.b": rng.normal(size=G * D), "v": rng.normal(size=(G * Dv, W)), "v.b": rng.normal(size=G * Dv),
            "q.norm": 1 + 0.1 * rng.normal(size=D), "k.norm": 1 + 0.1 * rng.normal(size=D),
            "temp": 1 + 0.2 * rng.normal(size=H), "o": rng.normal(size=(W, H * Dv))}


def test_attention_sees_exactly_the_window_and_the_bias_grows_with_distance():
    rng = np.random.default_rng(3)
    W, m = 12, tiny.left(heads=4, kv_heads=2, dim=6, vdim=5, scale=0.4, size=4, softcap=3.0)
    P = _left_weights(rng, W, m)
    h = rng.normal(size=(9, W))
    base = S.capped_window_attention(h, P, m, 1e-5)
    moved = h.copy()
    moved[2] += 5.0                                # position 2 is seen by 2 .. 5 and by nobody later
    got = S.capped_window_attention(moved, P, m, 1e-5)
    assert np.allclose(got[6:], base[6:]) and not np.allclose(got[5], base[5]) and np.allclose(got[:2], base[:2])
    # a window as long as the sequence is no window
    wide = S.capped_window_attention(h, P, dict(m, mask={"size": 9}), 1e-5)
    none = S.capped_window_attention(h, P, {k: v for k, v in m.items() if k != "mask"}, 1e-5)
    assert np.allclose(wide, none) and not np.allclose(wide[5:], base[5:])
    # by hand, one head and one row: scores capped after the head's factor, then slope * distance taken off
    T, H, D, Dv, hd, i = 9, 4, 6, 5, 3, 7
    q = S.rms_norm((h @ P["q"].T + P["q.b"]).reshape(T, H, D), P["q.norm"], 1e-5)[i, hd]
    k = S.rms_norm((h @ P["k"].T + P["k.b"]).reshape(T, 2, D), P["k.norm"], 1e-5)[:, hd // 2]
    v = (h @ P["v"].T + P["v.b"]).reshape(T, 2, Dv)[:, hd // 2]
    s = np.array([3.0 * np.tanh((q @ k[j]) * 0.4 * P["temp"][hd] / 3.0) - 2.0 ** (-8.0 * 4 / 4) * (i - j) for j in range(4, 8)])
    w = np.exp(s) / np.exp(s).sum()
    want = np.zeros(H * Dv)
    want[hd * Dv:(hd + 1) * Dv] = w @ v[4:8]
    # the other heads' share of row i comes from the function itself, with this head's output columns zeroed
    Pz = dict(P, o=P["o"].copy())
    Pz["o"][:, hd * Dv:(hd + 1) * Dv] = 0.0
    rest = S.capped_window_attention(h, Pz, m, 1e-5)[i]
    assert np.allclose(base[i], rest + P["o"] @ want)


def test_diagonal_recurrence_in_closed_form():
    rng = np.random.default_rng(4)
    W, m = 10, tiny.right(width=12, blocks=3, conv=3)
    C, bw = 12, 4
    P = {"y": rng.normal(size=(C, W)), "y.b": rng.normal(size=C), "x": rng.normal(size=(C, W)), "x.b": rng.normal(size=C),
         "conv": rng.normal(size=(C, 3)), "conv.b": rng.normal(size=C), "ra": rng.normal(size=(3, bw, bw)),
         "ra.b": rng.normal(size=(3, bw)), "ri": rng.normal(size=(3, bw, bw)), "ri.b": rng.normal(size=(3, bw)),
         "lam": rng.normal(size=C) - 2.0, "o": np.eye(C)[:W]}
    h = rng.normal(size=(7, W)) * 0.5
    got = S.gated_linear_recurrence(h, P, m)
    xin = h @ P["x"].T + P["x.b"]
    u = np.zeros((7, C))
    for t in range(7):
        u[t] = P["conv.b"] + sum(P["conv"][:, 2 - d] * xin[t - d] for d in range(3) if t - d >= 0)
    r, gi = np.zeros((7, C)), np.zeros((7, C))
    for b in range(3):
        sl = slice(b * bw, (b + 1) * bw)
        r[:, sl] = 1 / (1 + np.exp(-(u[:, sl] @ P["ra"][b].T + P["ra.b"][b])))
        gi[:, sl] = 1 / (1 + np.exp(-(u[:, sl] @ P["ri"][b].T + P["ri.b"][b])))
    log_a = -8.0 * r * np.log1p(np.exp(P["lam"]))
    # S_t = sum_j exp(sum_{j < l <= t} log a_l) * sqrt(1 - a_j^2) i_j u_j: the first token is no special case
    state = np.zeros((7, C))
    for t in range(7):
        for j in range(t + 1):
            state[t] += np.exp(log_a[j + 1:t + 1].sum(axis=0)) * np.sqrt(1 - np.exp(2 * log_a[j])) * gi[j] * u[j]
    y = S.gelu_tanh(h @ P["y"].T + P["y.b"])
    assert np.allclose(got, (state * y)[:, :W])


def test_state_space_recurrence_equals_its_attention_like_dual():
    rng = np.random.default_rng(5)
    W, m = 9, {"heads": 4, "vdim": 3, "state": 5, "groups": 2, "norm_groups": 3, "conv": 3}
    H, Dv, N, G, inner = 4, 3, 5, 2, 12
    ch = inner + 2 * G * N
    P = {"in": rng.normal(size=(2 * inner + 2 * G * N + H, W)) * 0.5, "conv": rng.normal(size=(ch, 3)), "conv.b": rng.normal(size=ch),
         "dt_bias": rng.normal(size=H), "A_log": rng.normal(size=H) * 0.5, "D": rng.normal(size=H),
         "norm": 1 + 0.1 * rng.normal(size=inner), "o": rng.normal(size=(W, inner))}
    T = 8
    h = rng.normal(size=(T, W))
    got = S.state_space_mixer(h, P, m, 1e-5)
    p = h @ P["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:inner + ch], p[:, inner + ch:]
    xbc = S.silu(S.causal_conv(xbc, P["conv"], P["conv.b"]))
    x, B, C = xbc[:, :inner].reshape(T, H, Dv), xbc[:, inner:inner + G * N].reshape(T, G, N), xbc[:, inner + G * N:].reshape(T, G, N)
    dt = np.log1p(np.exp(dt + P["dt_bias"]))
    y = np.zeros((T, H, Dv))
    for hd in range(H):
        g = hd // 2
        la = -np.exp(P["A_log"][hd]) * dt[:, hd]
        for t in range(T):
            for j in range(t + 1):          # y_t = sum_{j <= t} (C_t . B_j) exp(sum_{j < l <= t} la_l) dt_j x_j
                y[t, hd] += (C[t, g] @ B[j, g]) * np.exp(la[j + 1:t + 1].sum()) * dt[j, hd] * x[j, hd]
            y[t, hd] += P["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * S.silu(z)
    y = y.reshape(T, 3, 4)
    y = (y / np.sqrt((y ** 2).mean(axis=-1, keepdims=True) + 1e-5)).reshape(T, inner) * P["norm"]
    assert np.allclose(got, y @ P["o"].T)


def test_whole_model_is_causal_and_a_prefix_gives_the_same_rows():
    cfg = tiny.MIXED
    w = {k: v.float().numpy() for k, v in tiny.draw_weights(cfg, seed=0).items()}
    seq = np.random.default_rng(6).integers(0, cfg["vocab"], 30).tolist()
    full = S.forward(cfg, w, seq)
    assert np.allclose(S.forward(cfg, w, seq[:17]), full[:17])
    other = list(seq)
    other[20] = (other[20] + 1) % cfg["vocab"]
    changed = S.forward(cfg, w, other)
    assert np.allclose(changed[:20], full[:20]) and not np.allclose(changed[20], full[20])


def _rms(got, ref):
    return np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean())


def test_a_lost_shift_row_or_state_would_show():
    """The plain model itself, with one mechanism's memory cut at a step's border, differs from the whole by far more
    than the tests' tolerance: the comparisons above can see such a fault."""
    cfg = tiny.MIXED
    w = {k: v.float().numpy().astype(np.float64) for k, v in tiny.draw_weights(cfg, seed=1).items()}
    seq = np.random.default_rng(5).integers(0, cfg["vocab"], 40).tolist()
    ref = S.forward(cfg, w, seq)
    no_shift = dict(w)
    for i in range(len(cfg["layers"])):
        no_shift[f"l{i}.shift"] = np.zeros_like(w[f"l{i}.shift"])
    assert _rms(S.forward(cfg, no_shift, seq), ref) > 0.09
    swapped = dict(w)
    swapped["l1.hc1.mix"] = w["l1.hc1.mix"].T.copy()
    assert _rms(S.forward(cfg, swapped, seq), ref) > 0.09
