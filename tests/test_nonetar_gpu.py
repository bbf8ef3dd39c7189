"""Nonetar on the GPU, against the plain model in tests/plain_nonetar.py (numpy float64): every mechanism alone, then
whole models through the engine's step function, its scheduler, the trace runner and the command line.  Weights and
configurations are made here."""

import os
import tempfile

import numpy as np
import pytest
import torch

import plain_nonetar as S
import tiny_nonetar as tiny
from part_harness import DT, TOL, TOL_MODEL, _Manager, _ctx, _err, _make, _run_in_steps, _same, _w

pytestmark = pytest.mark.gpu


def _f32(a, dev="cuda"):
    return torch.as_tensor(np.asarray(a), dtype=torch.float32).to(dev).contiguous()


# --------------------------------------------------------------------------- embedding, streams, token shift, xIELU

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,streams", [(48, 3), (10, 1), (130, 4)])
def test_embedding_adds_the_position_vector_in_every_stream(dtype, W, streams):
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    rng = np.random.default_rng(0)
    ctx = _ctx(dtype, max_positions=8192)
    table, t64 = _w(rng, (31, W), 0.5)
    emb = _make("embedding", "sinusoid_stream_embedding", {"vocab_size": 31, "hidden_size": W, "streams": streams,
                                                           "base": 10000.0}, {"table": table}, ctx)
    builder = BatchBuilder(256, 4, [64], ctx.device, ctx.status)
    toks = {0: rng.integers(0, 31, 40).tolist(), 1: rng.integers(0, 31, 3).tolist()}
    starts = {0: 0, 1: 4000}        # far positions: the angle itself is a float32 of some thousands
    batch = builder.build([StepEntry(r, toks[r], starts[r], ()) for r in toks],
                          _Manager({0: list(range(16)), 1: list(range(16))}, {0: 0, 1: 1}))
    x = emb.forward(batch).cpu().numpy()
    assert x.shape == (43, streams, W) and int(ctx.status.item()) == 0
    ids = batch.token_ids.cpu().numpy()
    pos = batch.positions.cpu().numpy()
    assert sorted(pos.tolist()) == sorted(list(range(40)) + [4000, 4001, 4002])
    ref = t64[ids] + S.sinusoid(pos.tolist(), W)
    for s in range(streams):
        assert np.abs(x[:, s] - ref).max() < 1e-3 and np.array_equal(x[:, s], x[:, 0])
    near = pos < 1000
    assert np.abs(x[near, 0] - ref[near]).max() < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,streams,two", [(48, 3, True), (36, 1, False), (200, 4, False), (7, 2, True)])
def test_pending_write_read_and_norm_over_the_streams(dtype, W, streams, two):
    """x_t <- sum_s mix[s, t] x_s + out[t] (y + y2), then u = sum_s in[s] x_s and its norm with 1 + weight: one launch.
    The mixing matrix is far from symmetric, so that [from, to] shows."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(1)
    T = 19
    x = rng.normal(size=(T, streams, W))
    mix = rng.normal(size=(streams, streams))
    out_w, in_w, weight = rng.normal(size=streams), rng.normal(size=streams), 0.3 * rng.normal(size=W)
    ys = [_w(rng, (T, W), 1.0) for _ in range(2 if two else 1)]
    xd = _f32(x)
    x32 = xd.cpu().numpy().astype(np.float64)
    pending = ops.PendingStreams([y[0].to(DT[dtype]).cuda() for y in ys], _f32(mix), _f32(out_w))
    h = ops.hyper_norm(xd, pending, _f32(in_w), _f32(weight), 1e-5, True, DT[dtype], DT[dtype])
    y64 = sum(y[1] for y in ys) if dtype == "float32" else sum(y[0].float().numpy().astype(np.float64) for y in ys)
    f = lambda a: np.asarray(_f32(a, "cpu").numpy(), dtype=np.float64)      # the numbers the device got
    new = S.hyper_write(x32.transpose(1, 0, 2), y64, f(mix), f(out_w))
    assert np.abs(xd.cpu().numpy().transpose(1, 0, 2) - new).max() < 1e-5 * np.abs(new).max()
    ref = S.rms_norm(S.hyper_read(new, f(in_w)), f(weight), 1e-5, one_plus=True)
    assert _err(h, ref, dtype) < (1e-5 if dtype == "float32" else 1e-2)
    # selected rows only (what the model's last norm does for the rows whose logits are wanted): the plain sum
    rows = torch.tensor([3, 0, 18], dtype=torch.int32, device="cuda")
    before = xd.clone()
    hs = ops.hyper_norm(xd, None, None, _f32(weight), 1e-5, False, DT[dtype], DT[dtype], rows=rows)
    assert torch.equal(xd, before)
    ref = S.rms_norm(new.sum(axis=0)[[3, 0, 18]], f(weight), 1e-5)
    assert _err(hs, ref, dtype) < (1e-5 if dtype == "float32" else 1e-2)


class _ShiftedNorm:
    """The norm part with token shift, driven like a mixer: its rows are the streams side by side."""

    def __init__(self, norm, streams, W):
        self.norm, self.streams, self.W = norm, streams, W

    def cache_spec(self):
        from kv_cache_optimization_for_llm_b200.cache.specs import SlotStateSpec
        return SlotStateSpec((self.W,), torch.float32)

    def forward(self, rows, batch, binding):
        x = rows.float().reshape(rows.shape[0], self.streams, self.W).contiguous()
        return self.norm.forward(x, None, batch=batch, state=binding.state)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,streams", [(40, 3), (9, 1), (264, 2)])
def test_token_shift_in_portions_single_tokens_and_batches(dtype, W, streams):
    """The previous token's normed row is the request's state: across steps, inside a portion, in a step of single
    tokens (one fused launch), beside other requests; zero in front of the first token whatever the slot held."""
    rng = np.random.default_rng(2)
    ctx = _ctx(dtype)
    weight, in_w, shift = _w(rng, (W,), 0.3), _w(rng, (streams,), 0.5, 0.5), _w(rng, (W,), 0.3, 0.5)
    norm = _make("norm", "hyper_rmsnorm", {"size": W, "streams": streams, "eps": 1e-5, "one_plus": True, "learned": True,
                                           "shift": True}, {"weight": weight[0], "in": in_w[0], "shift": shift[0]}, ctx)
    part = _ShiftedNorm(norm, streams, W)
    xs, refs = {}, {}
    for r, T in enumerate((37, 12, 5)):
        x, x64 = _w(rng, (T, streams * W), 1.0)
        xs[r] = x.to(DT[dtype]).cuda()
        u = S.hyper_read(x64.reshape(T, streams, W).transpose(1, 0, 2), in_w[1])
        refs[r] = S.token_shift(S.rms_norm(u, weight[1], 1e-5, one_plus=True), shift[1])
    whole = _run_in_steps(part, ctx, xs, [[(0, 37)], [(1, 12)], [(2, 5)]])
    cut = _run_in_steps(part, ctx, xs, [[(0, 2), (1, 1)], [(0, 1), (1, 1), (2, 1)], [(0, 7), (1, 1), (2, 2)], [(0, 1), (1, 9)],
                                        [(0, 24), (2, 1)], [(0, 1), (2, 1)], [(0, 1)]])
    one = _run_in_steps(part, ctx, {0: xs[1]}, [[(0, 1)]] * 12)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < (1e-5 if dtype == "float32" else 1e-2)
        assert torch.equal(whole[r], cut[r]), "a token's result must not depend on the cut or on the batch"
    assert torch.equal(one[0], whole[1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,F,p,q", [(40, 56, 0.3, -0.4), (36, 10, -2.0, 1.5), (64, 128, 0.0, 0.0)])
def test_feed_forward_with_xielu(dtype, H, F, p, q):
    rng = np.random.default_rng(3)
    ctx = _ctx(dtype)
    up, down = _w(rng, (F, H), 0.4), _w(rng, (H, F), 0.3)
    act = _w(rng, (2,), 0.0)
    act[0][:] = torch.tensor([p, q])
    ff = _make("feed_forward", "dense_xielu", {"hidden_size": H, "intermediate_size": F},
               {"up": up[0], "down": down[0], "act": act[0]}, ctx)
    x, x64 = _w(rng, (23, H), 1.5)
    got = ff.forward(x.to(DT[dtype]).cuda(), None)
    ref = S.dense_xielu(x64, up[1], down[1], act[0].float().numpy().astype(np.float64))
    assert _err(got, ref, dtype) < TOL[dtype]
    # the activation alone, on both sides of zero and far out
    from kv_cache_optimization_for_llm_b200 import ops
    z = torch.tensor([-30.0, -3.0, -1e-3, 0.0, 1e-3, 0.5, 4.0, 11.0], dtype=torch.float32)
    got = ops.xielu(z.to(DT[dtype]).cuda(), _f32([p, q])).float().cpu().numpy()
    ref = S.xielu(z.to(DT[dtype]).double().numpy(), p, q)
    assert np.abs(got - ref).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(ref).max()


# --------------------------------------------------------------------------- the attention side

def _left_params(H, m, out_scale=1.0, eps=1e-5):
    return {"hidden_size": H, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
            "scale": m["scale"], "window": (m.get("mask") or {}).get("size"), "softcap": m.get("softcap"),
            "slope_power": 8.0, "bias": True, "qk_norm": True, "head_temperature": True, "eps": eps, "out_scale": out_scale}


def _left_weights(rng, H, m):
    Hq, G, D, Dv = (m[k] for k in ("heads", "kv_heads", "dim", "vdim"))
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (("q", "q", (Hq * D, H), 0.3, 0), ("k", "k", (G * D, H), 0.3, 0), ("v", "v", (G * Dv, H), 0.3, 0),
                                         ("q_bias", "q.b", (Hq * D,), 0.5, 0), ("k_bias", "k.b", (G * D,), 0.5, 0),
                                         ("v_bias", "v.b", (G * Dv,), 0.5, 0), ("q_norm", "q.norm", (D,), 0.2, 1.0),
                                         ("k_norm", "k.norm", (D,), 0.2, 1.0), ("temp", "temp", (Hq,), 0.3, 1.0),
                                         ("o", "o", (H, Hq * Dv), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(), dict(heads=6, kv_heads=1, dim=24, vdim=8, scale=0.2, size=5, softcap=1.5),
                                   dict(heads=2, kv_heads=2, dim=8, vdim=40, scale=0.5, size=16, softcap=None),
                                   dict(heads=3, kv_heads=1, dim=64, vdim=64, scale=0.125, size=33, softcap=30.0),
                                   dict(heads=1, kv_heads=1, dim=5, vdim=3, scale=1.0, size=1, softcap=2.0),
                                   dict(heads=4, kv_heads=4, dim=32, vdim=16, scale=0.3, size=None, softcap=8.0),
                                   dict(heads=8, kv_heads=2, dim=40, vdim=24, scale=0.15, size=64, softcap=5.0),
                                   dict(heads=4, kv_heads=2, dim=96, vdim=48, scale=0.1, size=50, softcap=20.0),
                                   dict(heads=8, kv_heads=1, dim=128, vdim=64, scale=0.09, size=40, softcap=None),
                                   dict(heads=2, kv_heads=1, dim=64, vdim=128, scale=0.12, size=None, softcap=3.0)])
def test_attention_alone_in_portions_and_beside_another_request(dtype, shape):
    """Several shapes (grouped and ungrouped heads, key and value sizes that differ, a window of one token, no window,
    no cap), 70 and 33 tokens on pages of 8 that lie scattered; portions end inside pages and on their borders."""
    rng = np.random.default_rng(3)
    ctx = _ctx(dtype)
    H = 40
    m = tiny.left(**shape)
    wt, w64 = _left_weights(rng, H, m)
    mixer = _make("mixer", "shaped_window_attention", _left_params(H, m, out_scale=0.7), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), 0.7 * S.capped_window_attention(x64, w64, m, 1e-5)
    from kv_cache_optimization_for_llm_b200 import ops
    on_tensor_cores = ops.choices["window_flash_attention"]
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    # bfloat16 prompt portions of sizes that are multiples of 8 run on tensor cores, everything else does not
    took = ops.choices["window_flash_attention"] > on_tensor_cores
    assert took == (dtype == "bfloat16" and m["dim"] % 8 == 0 and m["vdim"] % 8 == 0)
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    one = _run_in_steps(mixer, ctx, {0: xs[1]}, [[(0, 1)]] * 33)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]
        assert _same(whole[r], cut[r], dtype), "a token's result must not depend on the cut or on the batch"
    assert _same(one[0], whole[1], dtype), "token by token"


def _spiked(dtype, size, T, query, key, softcap=0.0, slope=None, temp=None, page=8, D=16, flash=False):
    """The attention kernel alone on keys and values made so that one key decides: every query and key is small but
    the pair (query, key), whose raw score is 30; the value of key j is the unit vector j.  Returns what the query at
    ``query`` reads, in a prompt (one portion) and decoded alone, and the plain answer.  ``flash``: the prompt on the
    tensor-core kernel, whose values have at most 128 channels: the value of key j is then the unit vector j mod 128."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    ctx = _ctx(dtype)
    rng = np.random.default_rng(T + query)
    q = rng.normal(size=(T, D)) * 0.01
    k = rng.normal(size=(T, D)) * 0.01
    q[query] = 0
    q[query, 3] = 6.0
    k[key] = 0
    k[key, 3] = 5.0
    Dv = min(T, 128) if flash else T
    v = np.zeros((T, Dv))
    v[np.arange(T), np.arange(T) % Dv] = 1.0
    src = torch.as_tensor(np.concatenate([q, k, v], axis=1), dtype=torch.float32).to(DT[dtype]).cuda()
    s = (q @ k.T).astype(np.float64) * (1.0 if temp is None else temp)
    if softcap:
        s = softcap * np.tanh(s / softcap)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    if slope is not None:
        s = s - slope * (i - j)
    seen = (j <= i) & ((i - j < size) if size else True)
    s = np.where(seen, s, -np.inf)
    w = np.exp(s - s.max(axis=1, keepdims=True))
    ref = (w / w.sum(axis=1, keepdims=True)) @ v
    outs = []
    for steps in ([T], [query] + [1] * (T - query)):
        pages = torch.zeros((T // page + 2, 1, page, D + Dv), dtype=DT[dtype], device="cuda")
        tables = {0: list(range(T // page + 1))[::-1]}
        builder = BatchBuilder(1024, 4, [64], ctx.device, ctx.status)
        at, rows = 0, []
        for n in steps:
            if n == 0:
                continue
            batch = builder.build([StepEntry(0, [0] * n, at, ())], _Manager(tables, {0: 0}))
            part = src[at:at + n].contiguous()
            ops.kv_rows_append(part, D, 2 * D, pages, batch.block_tables[0], batch, 1, D, Dv)
            shape = dict(head_scale=None if temp is None else _f32([temp]), slopes=None if slope is None else _f32([slope]),
                         softcap=softcap)
            if flash and n > 1:
                got = ops.window_flash_attention(part, pages, batch.block_tables[0], batch, 1, 1, D, Dv, 1.0, size, 0, False,
                                                 **shape)
            else:
                got = ops.window_attention(part, 0, pages, batch.block_tables[0], batch, 1, 1, D, Dv, 1.0, size, 0, False,
                                           **shape)
            rows.append(got.float().cpu())
            at += n
        outs.append(torch.cat(rows)[query].numpy())
    assert int(ctx.status.item()) == 0
    return outs, ref[query]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_far_away_and_keys_at_the_edges_of_the_window(dtype):
    """One key whose score stands out among hundreds, placed just inside and just outside the window, on a page's
    border, at the sequence's first token, and at the query itself; the query in a prompt and decoded alone."""
    size, T, query = 37, 250, 245
    tol = 2e-6 if dtype == "float32" else 1e-2
    for key, seen in ((query - size + 1, True), (query - size, False), (0, False), (query, True), (216, True), (215, True),
                      (query - 130, False)):
        (in_prompt, decoded), ref = _spiked(dtype, size, T, query, key)
        for got in (in_prompt, decoded):
            if seen:
                assert got[key] > 0.99 and abs(got[key] - ref[key]) < 1e-2, (key, got[key], ref[key])
            else:
                assert got[key] == 0 and ref[key] == 0, (key, got[key])
            assert np.abs(got - ref).max() < tol
    # no window: a key hundreds of tokens back, and the very first one
    for key in (2, 0):
        (in_prompt, decoded), ref = _spiked(dtype, 0, 250, 249, key)
        assert in_prompt[key] > 0.99 and decoded[key] > 0.99 and np.abs(in_prompt - ref).max() < tol
    # the first tokens of a sequence see fewer keys than the window holds
    (in_prompt, decoded), ref = _spiked(dtype, 4, 8, 2, 0)
    assert in_prompt[0] > 0.99 and np.abs(in_prompt - ref).max() < tol and np.abs(decoded - ref).max() < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cap_factor_and_distance_bias_decide_between_two_keys(dtype):
    """The raw score of 30 is capped at 4, after the head's factor: then a slope of 0.05 over 100 tokens outweighs it,
    and the weight of the far key falls from nearly 1 to what the plain computation says.  With the factor after the
    cap, or with the slope times the key's place instead of the distance, the numbers would be others."""
    T, query, key = 120, 119, 19
    tol = 1e-5 if dtype == "float32" else 2e-2
    (a, b), ref = _spiked(dtype, 0, T, query, key, softcap=4.0)
    assert 0.25 < ref[key] < 0.35 and abs(a[key] - ref[key]) < tol and abs(b[key] - ref[key]) < tol
    (a, b), ref = _spiked(dtype, 0, T, query, key, softcap=4.0, temp=0.05)       # tanh(1.5 / 4) * 4, not 0.05 * 4
    assert 0.02 < ref[key] < 0.05 and abs(a[key] - ref[key]) < tol and abs(b[key] - ref[key]) < tol
    (a, b), ref = _spiked(dtype, 0, T, query, key, softcap=4.0, slope=0.05)
    assert ref[key] < 0.03 and ref[query] > 0.04 and np.abs(a - ref).max() < tol and np.abs(b - ref).max() < tol
    (a, b), ref = _spiked(dtype, 0, T, query, key, slope=0.05)                   # no cap: 30 - 5 still wins
    assert ref[key] > 0.99 and abs(a[key] - ref[key]) < tol and abs(b[key] - ref[key]) < tol
    (a, b), ref = _spiked(dtype, 50, T, query, 70, softcap=4.0, slope=0.02)      # the nearest keys gain on the far one
    assert np.abs(a - ref).max() < tol and np.abs(b - ref).max() < tol and ref[118] > ref[71] * 2


@pytest.mark.parametrize("wide", [False, True])
def test_prompt_portions_on_tensor_cores_see_the_same_keys_and_shape_the_scores_alike(wide, monkeypatch):
    """The tensor-core kernel of prompt portions (tiles of 64 and of 128 query rows) on the cases above: a key that
    stands out just inside and just outside the window, on a tile's and a page's border, far back without a window, at
    the first token; cap, factor and distance bias deciding between two keys."""
    from kv_cache_optimization_for_llm_b200 import ops
    monkeypatch.setattr(ops, "WINDOW_FLASH_WIDE", wide)
    dtype, size, T, query = "bfloat16", 37, 250, 245
    before = ops.choices["window_flash_attention"]
    for key, seen in ((query - size + 1, True), (query - size, False), (0, False), (query, True), (216, True), (215, True),
                      (192, False), (191, False), (query - 130, False)):
        (in_prompt, _), ref = _spiked(dtype, size, T, query, key, flash=True)
        col = key % 128
        if seen:
            assert in_prompt[col] > 0.99 and abs(in_prompt[col] - ref[col]) < 1e-2, (key, in_prompt[col], ref[col])
        else:
            assert in_prompt[col] < 0.05 and ref[col] < 0.05, (key, in_prompt[col])
        assert np.abs(in_prompt - ref).max() < 1e-2
    for key, query_ in ((2, 249), (0, 249), (63, 200), (64, 200), (0, 2)):     # no window; keys at a tile's border
        (in_prompt, _), ref = _spiked(dtype, 0, 250, query_, key, flash=True)
        assert in_prompt[key % 128] > 0.99 and np.abs(in_prompt - ref).max() < 1e-2
    T, query, key, tol = 120, 119, 19, 2e-2
    for kw in (dict(softcap=4.0), dict(softcap=4.0, temp=0.05), dict(softcap=4.0, slope=0.05), dict(slope=0.05)):
        (a, _), ref = _spiked(dtype, 0, T, query, key, flash=True, **kw)
        assert np.abs(a - ref).max() < tol, kw
    (a, _), ref = _spiked(dtype, 50, T, query, 70, softcap=4.0, slope=0.02, flash=True)
    assert np.abs(a - ref).max() < tol and ref[118] > ref[71] * 2
    assert ops.choices["window_flash_attention"] >= before + 19


# --------------------------------------------------------------------------- the two recurrences

def _right_weights(rng, H, m):
    C, nb, taps = m["width"], m["blocks"], m["conv"]
    bw = C // nb
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (("y", "y", (C, H), 0.3, 0), ("y_bias", "y.b", (C,), 0.5, 0), ("x", "x", (C, H), 0.3, 0),
                                         ("x_bias", "x.b", (C,), 0.5, 0), ("conv", "conv", (C, taps), 0.6, 0),
                                         ("conv_bias", "conv.b", (C,), 0.3, 0), ("ra", "ra", (nb, bw, bw), 0.5, 0),
                                         ("ra_bias", "ra.b", (nb, bw), 0.5, 0), ("ri", "ri", (nb, bw, bw), 0.5, 0),
                                         ("ri_bias", "ri.b", (nb, bw), 0.5, 0), ("lam", "lam", (C,), 1.0, -2.0),
                                         ("o", "o", (H, C), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


def _right_params(H, m, out_scale=1.0):
    return {"hidden_size": H, "width": m["width"], "blocks": m["blocks"], "conv": m["conv"], "decay_scale": 8.0,
            "out_scale": out_scale}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,blocks,taps", [(36, 3, 3), (16, 1, 2), (40, 5, 4), (64, 64, 1), (132, 2, 5), (7, 7, 3)])
def test_gated_linear_recurrence_alone_in_portions_and_beside_another_request(dtype, width, blocks, taps):
    """Blocks of 12, 16, 8, 1, 66 and 1 channels; one to five taps; portions shorter than the taps; a step of single
    tokens; slots that held rubbish."""
    rng = np.random.default_rng(4)
    ctx = _ctx(dtype)
    H = 40
    m = tiny.right(width, blocks, taps)
    wt, w64 = _right_weights(rng, H, m)
    mixer = _make("mixer", "gated_linear_recurrence", _right_params(H, m, out_scale=1.3), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), 1.3 * S.gated_linear_recurrence(x64, w64, m)
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    one = _run_in_steps(mixer, ctx, {0: xs[1]}, [[(0, 1)]] * 33)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]
        assert _same(whole[r], cut[r], dtype), "a token's result must not depend on the cut or on the batch"
    assert _same(one[0], whole[1], dtype), "token by token"


def _ssd_weights(rng, H, m):
    Hd, Dv, N, G, taps = (m[k] for k in ("heads", "vdim", "state", "groups", "conv"))
    inner, ch = Hd * Dv, Hd * Dv + 2 * G * N
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (("in", "in", (2 * inner + 2 * G * N + Hd, H), 0.3, 0), ("conv", "conv", (ch, taps), 0.6, 0),
                                         ("conv_bias", "conv.b", (ch,), 0.3, 0), ("dt_bias", "dt_bias", (Hd,), 0.5, -1.0),
                                         ("A_log", "A_log", (Hd,), 0.5, 0), ("D", "D", (Hd,), 0.5, 1.0),
                                         ("norm", "norm", (inner,), 0.2, 1.0), ("o", "o", (H, inner), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


def _ssd_params(H, m, eps=1e-5):
    return {"hidden_size": H, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
            "norm_groups": m["norm_groups"], "conv": m["conv"], "eps": eps}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(), dict(heads=2, vdim=16, state=24, groups=1, norm_groups=1, conv=2),
                                   dict(heads=6, vdim=8, state=5, groups=3, norm_groups=6, conv=3),
                                   dict(heads=3, vdim=5, state=7, groups=3, norm_groups=5, conv=1),
                                   dict(heads=1, vdim=64, state=128, groups=1, norm_groups=2, conv=4),
                                   dict(heads=8, vdim=32, state=16, groups=2, norm_groups=4, conv=4)])
def test_state_space_duality_alone_in_portions_and_beside_another_request(dtype, shape):
    """Groups shared by two heads, one group, a group per head; norm groups that are more, fewer and as many as the
    groups of B and C; one tap; states of 5 to 128 rows."""
    rng = np.random.default_rng(5)
    ctx = _ctx(dtype)
    H = 40
    m = tiny.mamba(**shape)["mixer"]
    wt, w64 = _ssd_weights(rng, H, m)
    mixer = _make("mixer", "state_space_duality", _ssd_params(H, m), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.state_space_mixer(x64, w64, m, 1e-5)
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    one = _run_in_steps(mixer, ctx, {0: xs[1]}, [[(0, 1)]] * 33)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]
        assert _same(whole[r], cut[r], dtype), "a token's result must not depend on the cut or on the batch"
    assert _same(one[0], whole[1], dtype), "token by token"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["gated_linear_recurrence", "state_space_duality"])
def test_long_runs_are_walked_in_chunks_side_by_side(dtype, kind):
    """A step with a run of 256 tokens or more cuts its runs into chunks that begin from summaries of the chunks
    before them.  Runs of 700, of 5 * 64 + 1 and of 1024 tokens: alone, two in one step, and in portions that end
    inside a chunk and exactly at a chunk's end, beside single tokens of a third request (which then come first in
    the step) and in slots that held rubbish.  Every form against the plain walk."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(11)
    ctx = _ctx(dtype, max_positions=2048)
    H = 40
    if kind == "gated_linear_recurrence":
        m = tiny.right(36, 3, 3)
        wt, w64 = _right_weights(rng, H, m)
        mixer = _make("mixer", kind, _right_params(H, m), wt, ctx)
        plain = lambda x64: S.gated_linear_recurrence(x64, w64, m)
        counter = "diag_scan_chunked"
    else:
        m = tiny.mamba(heads=4, vdim=8, state=12, groups=2, norm_groups=2, conv=3)["mixer"]
        wt, w64 = _ssd_weights(rng, H, m)
        mixer = _make("mixer", kind, _ssd_params(H, m), wt, ctx)
        plain = lambda x64: S.state_space_mixer(x64, w64, m, 1e-5)
        counter = "ssd_scan_chunked"
    xs, refs = {}, {}
    for r, T in enumerate((700, 321, 6, 1024)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), plain(x64)
    before = ops.choices[counter]
    runs = {
        "alone": [[(0, 700)], [(1, 321)], [(3, 1024)]],
        "together": [[(0, 700), (1, 321)], [(3, 512)], [(3, 512)]],
        "in portions": [[(0, 300), (2, 1)], [(2, 1), (0, 256), (1, 320)], [(0, 144), (1, 1), (2, 1)], [(2, 2)],
                        [(3, 257), (2, 1)], [(3, 767)]],
    }
    for name, steps in runs.items():
        got = _run_in_steps(mixer, ctx, {r: xs[r] for r in {q for st in steps for q, _ in st}}, steps, page=16, state_slots=4)
        for r in got:
            assert _err(got[r], refs[r], dtype) < TOL[dtype], (name, r)
    assert ops.choices[counter] >= before + 10


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["gated_linear_recurrence", "state_space_duality"])
def test_states_are_carried_over_hundreds_of_tokens(dtype, kind):
    """Decays near one (lam and the step sizes far below zero), so that the first tokens still weigh after 400: a
    prompt of 150, then 250 single tokens, against the whole sequence at once; and a state lost on the way would show."""
    rng = np.random.default_rng(6)
    ctx = _ctx(dtype)
    H, T = 24, 400
    x, x64 = _w(rng, (T, H), 1.0)
    if kind == "gated_linear_recurrence":
        m = tiny.right(32, 4, 3)
        wt, w64 = _right_weights(rng, H, m)
        wt["lam"], w64["lam"] = _w(rng, (32,), 0.3, -7.0)
        mixer = _make("mixer", kind, _right_params(H, m), wt, ctx)
        ref = S.gated_linear_recurrence(x64, w64, m)
        cold = S.gated_linear_recurrence(x64[150:], w64, m)
    else:
        m = tiny.mamba(heads=4, vdim=8, state=12, groups=2, norm_groups=2, conv=3)["mixer"]
        wt, w64 = _ssd_weights(rng, H, m)
        wt["dt_bias"], w64["dt_bias"] = _w(rng, (4,), 0.3, -6.5)
        wt["D"], w64["D"] = _w(rng, (4,), 0.0)          # nothing of the token itself beside the state's read-out
        mixer = _make("mixer", kind, _ssd_params(H, m), wt, ctx)
        ref = S.state_space_mixer(x64, w64, m, 1e-5)
        cold = S.state_space_mixer(x64[150:], w64, m, 1e-5)
    assert np.abs(cold[-1] - ref[-1]).max() > 0.05 * np.abs(ref[-1]).max(), "the test's weights forget too fast"
    xs = {0: x.to(DT[dtype]).cuda()}
    got = _run_in_steps(mixer, ctx, xs, [[(0, 150)]] + [[(0, 1)]] * 250)
    assert _err(got[0][150:], ref[150:], dtype) < TOL[dtype]
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 400)]])
    # a run this long is walked in chunks that begin from summaries, which rounds differently from one walk
    assert _err(whole[0], ref, dtype) < TOL[dtype]
    assert _err(whole[0], got[0].double().numpy(), dtype) < TOL[dtype]


# --------------------------------------------------------------------------- whole models

def _runner(folder, dtype, **kw):
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    args = dict(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, max_num_batched_tokens=256, max_model_len=160,
                use_cuda_graphs=False)
    args.update(kw)
    return ModelRunner(folder, EngineConfig(**args))


def _logit_err(got, ref, dtype="float32"):
    if dtype == "float32":
        return np.abs(got - ref).max() / np.abs(ref).max()
    return np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean())


def _close(a, b, dtype):
    """Two runs of the engine that cut the same tokens differently."""
    return _logit_err(a, b, dtype) < (2e-5 if dtype == "float32" else TOL_MODEL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_model_prefill_decoding_portions_batches_and_reuse(dtype):
    """A model with both kinds of mixer and a layer without feed-forward.  Whole prompts; token by token; portions
    of 2, 3, 7, ... beside single tokens of another request; then requests that end and others that take over their
    slots and pages in a pool that holds two of them at most; 60 decoded tokens in a row, past every window."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_nt_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=1)
    r = _runner(folder, dtype)
    assert len(r.spec.schedule) == 5 and len(r.cache.states) == 5        # every layer keeps a state: its shifted row
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (90, 37, 61, 1, 150)]
    refs = [S.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    whole = r.step([StepEntry(0, seqs[1], 0, range(37))]).cpu().numpy()
    assert _logit_err(whole, refs[1], dtype) < tol
    r.release(0)
    single = np.concatenate([r.step([StepEntry(1, [t], i, [0])]).cpu().numpy() for i, t in enumerate(seqs[1])])
    assert _logit_err(single, refs[1], dtype) < tol
    assert _close(whole, single, dtype)
    r.release(1)
    got2 = [r.step([StepEntry(12, seqs[2][:20], 0, range(20))]).cpu().numpy()]
    pos0, pos2, got0 = 0, 20, []
    for n in (2, 3, 7, 1, 8, 16, 2, 9, 5, 1, 1, 30, 2, 3):
        entries = [StepEntry(10, seqs[0][pos0:pos0 + n], pos0, range(n))]
        if pos2 < len(seqs[2]):
            entries.insert(0 if n % 2 else 1, StepEntry(12, [seqs[2][pos2]], pos2, [0]))
        if n == 7:
            entries.append(StepEntry(13, seqs[3], 0, [0]))
        out = r.step(entries).cpu().numpy()
        i = 0
        for e in entries:
            k = len(e.want)
            if e.request_id == 10:
                got0.append(out[i:i + k])
            elif e.request_id == 12:
                got2.append(out[i:i + k])
                pos2 += 1
            else:
                assert _logit_err(out[i:i + k], refs[3], dtype) < tol
                r.release(13)
            i += k
        pos0 += n
    assert pos0 == 90
    assert _logit_err(np.concatenate(got0), refs[0], dtype) < tol
    assert _logit_err(np.concatenate(got2), refs[2][:pos2], dtype) < tol
    r.check_status()
    r.release(10)
    r.release(12)
    assert r.manager.check() == ""
    long = [r.step([StepEntry(20, seqs[4][:90], 0, range(90))]).cpu().numpy()]
    for i in range(90, 150):
        long.append(r.step([StepEntry(20, [seqs[4][i]], i, [0])]).cpu().numpy())
    assert _logit_err(np.concatenate(long), refs[4], dtype) < tol
    r.check_status()
    r.release(20)
    assert all(r.manager.free_pages(g) == 40 for g in range(r.manager.num_groups()))


@pytest.mark.parametrize("layers,width,streams", [
    # one layer of each kind alone; a single stream (the ordinary residual with learned weights)
    ([tiny.parallel(tiny.left(heads=2, kv_heads=1, dim=8, vdim=8, size=6), tiny.right(16, 2, 2))], 40, 1),
    ([tiny.mamba(heads=2, vdim=16, state=8, groups=2, norm_groups=1, conv=3, mlp=tiny.dense(24))], 40, 2),
    # where the numbers that could be equal are not: query against key/value heads, heads against blocks against
    # groups against norm groups against streams, the attention's taps against the state space's
    ([tiny.parallel(tiny.left(heads=6, kv_heads=3, dim=24, vdim=40, scale=0.11, size=9, softcap=2.5), tiny.right(80, 5, 4),
                    left_scale=0.3, right_scale=1.7, mlp=tiny.dense(72)),
      tiny.mamba(heads=6, vdim=12, state=20, groups=2, norm_groups=9, conv=2),
      tiny.parallel(tiny.left(heads=1, kv_heads=1, dim=96, vdim=16, scale=0.05, size=64, softcap=None), tiny.right(24, 24, 1),
                    mlp=tiny.dense(8)),
      tiny.mamba(heads=4, vdim=8, state=16, groups=4, norm_groups=1, conv=5, mlp=tiny.dense(104))], 104, 4),
    # sizes that are no multiples of eight: nothing may rest on 16-byte rows
    ([tiny.parallel(tiny.left(heads=3, kv_heads=1, dim=5, vdim=3, scale=0.4, size=7, softcap=3.0), tiny.right(21, 3, 3),
                    mlp=tiny.dense(18)),
      tiny.mamba(heads=3, vdim=5, state=7, groups=1, norm_groups=3, conv=3, mlp=tiny.dense(6))], 36, 3),
    # no window at all, and the same mixer twice in a row
    ([tiny.parallel(tiny.left(size=None)), tiny.parallel(tiny.left(size=None, softcap=None), mlp=tiny.dense(16)),
      tiny.mamba(), tiny.mamba(mlp=tiny.dense(16))], 48, 2),
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_orders_of_layers_sizes_and_numbers_of_streams(layers, width, streams, dtype):
    """A prompt in three portions and four tokens one by one, against the plain model."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_nt_")
    cfg = tiny.config(layers, width=width, vocab=53, streams=streams, logit_scale=1.6, eps=1e-6)
    w = tiny.write_model(folder, cfg, seed=2)
    r = _runner(folder, dtype)
    seq = np.random.default_rng(1).integers(0, 53, 44).tolist()
    ref = S.forward(cfg, w, seq)
    got, pos = [], 0
    for n in (11, 2, 27, 1, 1, 1, 1):
        got.append(r.step([StepEntry(0, seq[pos:pos + n], pos, range(n))]).cpu().numpy())
        pos += n
    assert _logit_err(np.concatenate(got), ref, dtype) < TOL_MODEL[dtype]
    r.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype):
    """Prompts of unequal length through ``LLM.generate``: the scheduler's portions (a token budget of 24 per step),
    decode steps replayed from CUDA graphs, the engine one step ahead, five requests in three seats.  Every sampled
    row's logits are compared with the plain model on the final sequences, and in float32 the greedy tokens themselves."""
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    from logit_hook import LogitRecorder
    folder = tempfile.mkdtemp(prefix="kvb200_nt_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=4)
    llm = LLM(folder, dtype=dtype, page_size=8, num_pages=48, max_num_seqs=3, max_num_batched_tokens=24,
              max_model_len=128, use_cuda_graphs=True, run_ahead=True)
    rec = LogitRecorder(llm.engine.runner)
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (3, 41, 17, 1, 30)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert [len(o) for o in outs] == [12] * 5
    seqs = {i: prompts[i] + outs[i] for i in range(5)}
    plain = {i: S.forward(cfg, w, seqs[i]) for i in seqs}
    if dtype == "float32":
        n, worst = rec.compare(seqs, lambda i: plain[i], TOL_MODEL[dtype], "greedy generation")
    else:       # the measure of this file's other bfloat16 comparisons: over all of a request's rows at once
        got = rec.collect(seqs)
        n = sum(len(ps) for ps, _ in got.values())
        for i, (ps, rows) in got.items():
            assert _logit_err(rows, plain[i][ps], dtype) < TOL_MODEL[dtype], f"greedy generation: request {i}"
    assert n >= 60 and llm.engine.runner._graphs
    if dtype == "float32":
        for i in seqs:
            for j, tok in enumerate(outs[i]):
                row = plain[i][len(prompts[i]) + j - 1]
                assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (i, j)
    assert llm.engine.runner.manager.check() == ""


@pytest.mark.parametrize("dtype,flags", [("float32", ()), ("bfloat16", ()), ("float32", ("--cuda-graphs",))])
def test_replay_through_the_trace_runner(dtype, flags):
    """bin/trace_run on a Nonetar folder: each request whole, then four live requests whose portions (down to two
    tokens) run beside single tokens in a pool that holds exactly them, in four state slots; requests that end hand
    pages and slots to the ones that follow."""
    from trace_driver import TraceRun, ceil64
    folder = tempfile.mkdtemp(prefix="kvb200_nt_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=6)
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (70, 33, 50, 21)]
    refs = [S.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    tr = TraceRun(folder, dtype, sum(ceil64(len(s)) for s in seqs), ("--page-size", "8") + tuple(flags))
    try:
        for r, s in enumerate(seqs):
            got = tr.step([(f"w{r}", s, range(len(s)))], end=[f"w{r}"])
            assert _logit_err(got, refs[r], dtype) < tol, f"whole request {r}"
        for round_ in range(2):         # the second round runs in slots and pages that the first gave back
            plans = {0: [5, 2, 16, 9, 2, 30] + [1] * 6, 1: [1, 1, 20, 2] + [1] * 9, 2: [33, 2, 3, 2] + [1] * 10,
                     3: [2, 2, 2, 7] + [1] * 8}
            pos = {r: 0 for r in plans}
            step = 0
            while plans:
                entries, expect, ends = [], [], []
                for r in sorted(plans):
                    if step < r:        # they start one step apart
                        continue
                    n = plans[r].pop(0)
                    entries.append((f"m{round_}_{r}", seqs[r][pos[r]:pos[r] + n], range(n)))
                    expect.append(refs[r][pos[r]:pos[r] + n])
                    pos[r] += n
                    if not plans[r]:
                        assert pos[r] == len(seqs[r])
                        ends.append(f"m{round_}_{r}")
                        del plans[r]
                got = tr.step(entries, end=ends)
                assert _logit_err(got, np.concatenate(expect), dtype) < tol, f"round {round_}, mixed step {step}"
                step += 1
    finally:
        tr.close()


def test_command_line_serves_the_design():
    """The engine's command line on a Nonetar folder: requests on standard input in the wire format, greedy tokens
    back as JSON lines; each token is the plain model's best (ties within 1e-4 allowed)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = tempfile.mkdtemp(prefix="kvb200_nt_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=8)
    rng = np.random.default_rng(4)
    prompts = {3: rng.integers(0, cfg["vocab"], 9).tolist(), 11: rng.integers(0, cfg["vocab"], 26).tolist()}
    lines = [f"{rid} 6 1 " + " ".join(map(str, toks)) for rid, toks in prompts.items()]
    env = dict(os.environ, IGNORE_EOS="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-m", "kv_cache_optimization_for_llm_b200.cli", folder, "--dtype", "float32",
                        "--page-size", "4", "--num-pages", "64", "--max-num-seqs", "4", "--max-model-len", "64"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [json.loads(line) for line in p.stdout.splitlines() if line.strip()]
    for rid, prompt in prompts.items():
        toks = [m["tok"] for m in out if m.get("id") == rid and "tok" in m]
        assert len(toks) == 6
        logits = S.forward(cfg, w, prompt + toks)
        for j, tok in enumerate(toks):
            row = logits[len(prompt) + j - 1]
            assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (rid, j)
